"""Configuration of the Pofadra decoder (config.json key ``"architecture": "Pofadra"``).

The file is nested: ``vocab``, ``width``, ``norm.eps``, ``embedding.scale``, ``logit_softcap`` and a list ``layers`` whose
entries give the layer's ``type`` (which mixer: ``channel_delta`` or ``attention``), the mixer's sizes under ``mixer`` and
the feed-forward under ``mlp`` (null: none).  Every size and every constant that the file gives is read from it; what
the design fixes (the norms' form, the unit lengths' epsilon, SiLU, the sink of the softmax, the rotation's pairing) is
in the parts.  Sizes that only a tensor's shape gives (the inner sizes of the delta rule's low-rank paths) are read off
the tensors at load; a file may name them (``decay_rank``, ``gate_rank``) for the random-weights mode.
"""

from __future__ import annotations

import dataclasses
from typing import Any, ClassVar

from .base import ConfigError, ModelConfig

MIXERS = ("channel_delta", "attention")
FEED_FORWARDS = ("moe",)


def _need(where: str, table: Any, keys: tuple[str, ...], optional: tuple[str, ...] = ()) -> dict:
    if not isinstance(table, dict):
        raise ConfigError(f"PofadraConfig: {where} must be an object")
    missing = [k for k in keys if k not in table]
    unknown = [k for k in table if k not in keys and k not in optional]
    if missing or unknown:
        parts = ([f"missing keys {sorted(missing)}"] if missing else []) + ([f"unknown keys {sorted(unknown)}"] if unknown else [])
        raise ConfigError(f"PofadraConfig: {where}: " + "; ".join(parts))
    return table


def _positive_int(where: str, value: Any) -> int:
    if isinstance(value, bool) or not isinstance(value, (int, float)) or int(value) != value or value <= 0:
        raise ConfigError(f"PofadraConfig: {where} must be a positive integer, got {value!r}")
    return int(value)


def _positive(where: str, value: Any) -> float:
    if isinstance(value, bool) or not isinstance(value, (int, float)) or not value > 0:
        raise ConfigError(f"PofadraConfig: {where} must be a positive number, got {value!r}")
    return float(value)


@dataclasses.dataclass(frozen=True)
class PofadraConfig(ModelConfig):
    vocab: int
    width: int
    layers: list
    norm: dict
    embedding: dict | None = None  # absent: the table's rows enter the stream as they are
    logit_softcap: float | None = None  # absent or null: logits are not capped
    initializer_range: float | None = None  # only read by the random-weights mode
    max_position_embeddings: int | None = None  # longest sequence a request may reach (optional)

    ARCH_NAMES: ClassVar[tuple[str, ...]] = ("Pofadra",)
    IGNORED_KEYS: ClassVar[frozenset[str]] = frozenset({"architecture", "torch_dtype", "dtype"})

    @property
    def eps(self) -> float:
        return float(self.norm["eps"])

    @property
    def embedding_scale(self) -> float:
        return float(self.embedding["scale"]) if self.embedding else 1.0

    def to_dict(self) -> dict[str, Any]:
        out = {k: v for k, v in dataclasses.asdict(self).items() if v is not None}
        out["architecture"] = self.ARCH_NAMES[0]
        return out

    def validate(self) -> None:
        _positive_int("vocab", self.vocab)
        _positive_int("width", self.width)
        _positive("norm.eps", _need("norm", self.norm, ("eps",))["eps"])
        if self.embedding is not None:
            _positive("embedding.scale", _need("embedding", self.embedding, ("scale",))["scale"])
        if self.logit_softcap is not None:
            _positive("logit_softcap", self.logit_softcap)
        if not isinstance(self.layers, list) or not self.layers:
            raise ConfigError("PofadraConfig: layers must be a list with at least one layer")
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]"
            _need(where, layer, ("type", "mixer"), ("mlp",))
            kind = layer["type"]
            if kind not in MIXERS:
                raise ConfigError(f"PofadraConfig: {where}.type {kind!r} is not a mixer of this design (known: {list(MIXERS)})")
            if kind == "channel_delta":
                m = _need(where + ".mixer", layer["mixer"], ("heads", "kv_heads", "dim", "vdim", "conv"), ("decay_rank", "gate_rank"))
                for key in ("heads", "kv_heads", "dim", "vdim", "conv"):
                    _positive_int(f"{where}.mixer.{key}", m[key])
                for key in ("decay_rank", "gate_rank"):
                    if m.get(key) is not None:
                        _positive_int(f"{where}.mixer.{key}", m[key])
                if m["dim"] % 4 or m["dim"] > 256:
                    raise ConfigError(f"PofadraConfig: {where}.mixer.dim ({m['dim']}) must be a multiple of 4, at most 256")
            else:
                m = _need(where + ".mixer", layer["mixer"], ("heads", "kv_heads", "dim", "vdim", "scale"), ("rot", "mask"))
                for key in ("heads", "kv_heads", "dim", "vdim"):
                    _positive_int(f"{where}.mixer.{key}", m[key])
                _positive(f"{where}.mixer.scale", m["scale"])
                if m["vdim"] != m["dim"]:
                    raise ConfigError(f"PofadraConfig: {where}.mixer: the values are the keys, so vdim ({m['vdim']}) must equal dim ({m['dim']})")
                if m["dim"] % 8:
                    raise ConfigError(f"PofadraConfig: {where}.mixer.dim ({m['dim']}) must be a multiple of 8")
                rot = m.get("rot")
                if rot is not None:
                    _need(where + ".mixer.rot", rot, ("base", "dims"))
                    dims = _positive_int(f"{where}.mixer.rot.dims", rot["dims"])
                    _positive(f"{where}.mixer.rot.base", rot["base"])
                    if dims % 2 or dims > m["dim"]:
                        raise ConfigError(f"PofadraConfig: {where}.mixer.rot.dims ({dims}) must be even and at most dim ({m['dim']})")
                if m.get("mask") is not None:
                    _positive_int(f"{where}.mixer.mask.size", _need(where + ".mixer.mask", m["mask"], ("size",))["size"])
            if m["heads"] % m["kv_heads"]:
                raise ConfigError(f"PofadraConfig: {where}.mixer.heads ({m['heads']}) must be a multiple of kv_heads ({m['kv_heads']})")
            mlp = layer.get("mlp")
            if mlp is not None:
                _need(where + ".mlp", mlp, ("kind", "expert", "router"))
                if mlp["kind"] not in FEED_FORWARDS:
                    raise ConfigError(f"PofadraConfig: {where}.mlp.kind {mlp['kind']!r} is not a feed-forward of this design "
                                      f"(known: {list(FEED_FORWARDS)})")
                _positive_int(f"{where}.mlp.expert.ff", _need(where + ".mlp.expert", mlp["expert"], ("ff",))["ff"])
                r = _need(where + ".mlp.router", mlp["router"], ("experts", "top", "scale"), ("groups",))
                experts, top = _positive_int(f"{where}.mlp.router.experts", r["experts"]), _positive_int(f"{where}.mlp.router.top", r["top"])
                _positive(f"{where}.mlp.router.scale", r["scale"])
                count = keep = 1
                if r.get("groups") is not None:
                    g = _need(where + ".mlp.router.groups", r["groups"], ("count", "keep"))
                    count, keep = _positive_int(f"{where}.mlp.router.groups.count", g["count"]), _positive_int(f"{where}.mlp.router.groups.keep", g["keep"])
                if experts % count or keep > count or top > keep * (experts // count):
                    raise ConfigError(f"PofadraConfig: {where}.mlp.router: {top} of {experts} experts cannot be chosen from {keep} of {count} equal groups")
        if self.max_position_embeddings is not None:
            _positive_int("max_position_embeddings", self.max_position_embeddings)
