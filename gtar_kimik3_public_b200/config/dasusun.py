"""Configuration of the Dasusun decoder (config.json key ``"architecture": "Dasusun"``).

The file is nested: ``vocab``, ``width``, ``norm.eps``, ``canon.taps`` and a list ``layers`` whose entries give the
layer's ``type`` (which mixer), the mixer's sizes under ``mixer`` and the feed-forward under ``mlp`` (null: none).
Every size and every constant that the file gives is read from it; what the design fixes (the form of the norms,
GELU's constants, the rotation's pairing) is in the parts.
"""

from __future__ import annotations

import dataclasses
from typing import Any, ClassVar

from .base import ConfigError, ModelConfig

MIXERS = ("latent_attention",)
FEED_FORWARDS = ("dense",)


def _need(where: str, table: Any, keys: tuple[str, ...], optional: tuple[str, ...] = ()) -> dict:
    if not isinstance(table, dict):
        raise ConfigError(f"DasusunConfig: {where} must be an object")
    missing = [k for k in keys if k not in table]
    unknown = [k for k in table if k not in keys and k not in optional]
    if missing or unknown:
        parts = ([f"missing keys {sorted(missing)}"] if missing else []) + ([f"unknown keys {sorted(unknown)}"] if unknown else [])
        raise ConfigError(f"DasusunConfig: {where}: " + "; ".join(parts))
    return table


def _positive_int(where: str, value: Any) -> int:
    if isinstance(value, bool) or not isinstance(value, (int, float)) or int(value) != value or value <= 0:
        raise ConfigError(f"DasusunConfig: {where} must be a positive integer, got {value!r}")
    return int(value)


def _positive(where: str, value: Any) -> float:
    if isinstance(value, bool) or not isinstance(value, (int, float)) or not value > 0:
        raise ConfigError(f"DasusunConfig: {where} must be a positive number, got {value!r}")
    return float(value)


@dataclasses.dataclass(frozen=True)
class DasusunConfig(ModelConfig):
    vocab: int
    width: int
    layers: list
    norm: dict
    canon: dict | None = None  # absent or null: no input convolution
    initializer_range: float | None = None  # only read by the random-weights mode
    max_position_embeddings: int | None = None  # longest sequence a request may reach (optional)

    ARCH_NAMES: ClassVar[tuple[str, ...]] = ("Dasusun",)
    IGNORED_KEYS: ClassVar[frozenset[str]] = frozenset({"architecture", "torch_dtype", "dtype"})

    @property
    def eps(self) -> float:
        return float(self.norm["eps"])

    @property
    def taps(self) -> int:
        return int(self.canon["taps"]) if self.canon else 0

    def to_dict(self) -> dict[str, Any]:
        out = {k: v for k, v in dataclasses.asdict(self).items() if v is not None}
        out["architecture"] = self.ARCH_NAMES[0]
        return out

    def validate(self) -> None:
        _positive_int("vocab", self.vocab)
        _positive_int("width", self.width)
        _positive("norm.eps", _need("norm", self.norm, ("eps",))["eps"])
        if self.canon is not None:
            _positive_int("canon.taps", _need("canon", self.canon, ("taps",))["taps"])
        if not isinstance(self.layers, list) or not self.layers:
            raise ConfigError("DasusunConfig: layers must be a list with at least one layer")
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]"
            _need(where, layer, ("type", "mixer"), ("mlp",))
            if layer["type"] not in MIXERS:
                raise ConfigError(f"DasusunConfig: {where}.type {layer['type']!r} is not a mixer of this design (known: {list(MIXERS)})")
            m = _need(where + ".mixer", layer["mixer"], ("heads", "dim", "rot_dim", "vdim", "q_rank", "kv_rank", "scale"),
                      ("rot", "mask"))
            for key in ("heads", "dim", "vdim", "q_rank", "kv_rank"):
                _positive_int(f"{where}.mixer.{key}", m[key])
            _positive(f"{where}.mixer.scale", m["scale"])
            rot_dim = m["rot_dim"]
            if isinstance(rot_dim, bool) or not isinstance(rot_dim, int) or rot_dim < 0:
                raise ConfigError(f"DasusunConfig: {where}.mixer.rot_dim must be a non-negative integer, got {rot_dim!r}")
            rot = m.get("rot")
            if rot is not None:
                _need(where + ".mixer.rot", rot, ("base", "dims"), ("scaling",))
                dims = _positive_int(f"{where}.mixer.rot.dims", rot["dims"])
                _positive(f"{where}.mixer.rot.base", rot["base"])
                if dims % 2 or dims > rot_dim:
                    raise ConfigError(f"DasusunConfig: {where}.mixer.rot.dims ({dims}) must be even and at most rot_dim ({rot_dim})")
                if rot.get("scaling") is not None:
                    scaling = _need(where + ".mixer.rot.scaling", rot["scaling"], ("factor", "original", "fast", "slow"))
                    for key in ("factor", "original", "fast", "slow"):
                        _positive(f"{where}.mixer.rot.scaling.{key}", scaling[key])
            if m.get("mask") is not None:
                _positive_int(f"{where}.mixer.mask.size", _need(where + ".mixer.mask", m["mask"], ("size",))["size"])
            mlp = layer.get("mlp")
            if mlp is not None:
                _need(where + ".mlp", mlp, ("kind", "ff"))
                if mlp["kind"] not in FEED_FORWARDS:
                    raise ConfigError(f"DasusunConfig: {where}.mlp.kind {mlp['kind']!r} is not a feed-forward of this design "
                                      f"(known: {list(FEED_FORWARDS)})")
                _positive_int(f"{where}.mlp.ff", mlp["ff"])
        if self.max_position_embeddings is not None:
            _positive_int("max_position_embeddings", self.max_position_embeddings)
