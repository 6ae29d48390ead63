"""The Dasusun decoder put together from parts.

Token embedding; per layer a ``SandwichBlock`` (norms before and after each branch with weights kept around zero,
per-channel layer scale, a causal convolution in front of the mixer, the depth mix of all earlier results) around a
latent-attention mixer with a sliding window and scaled rotary positions, and a GELU feed-forward (or none); the
model's last norm; logits through the embedding table.  Each layer's sizes come from its own entry of the config, so
layers may differ in everything.  Tensor names: ``embed``, ``l<i>.<part>``, ``final.norm``.
"""

from __future__ import annotations

from ..config.dasusun import DasusunConfig
from ..parts.base import build_part
from ..parts.embedding import OutputHead, TokenEmbedding
from .model import ModelPlan, RunEntry


def _position(rot: dict | None, shared: dict):
    """One table per distinct rotation (layers with the same constants read the same tables)."""
    if not rot:
        return None
    scaling = rot.get("scaling")
    key = (int(rot["dims"]), float(rot["base"]), tuple(sorted(scaling.items())) if scaling else None)
    if key not in shared:
        if scaling:
            shared[key] = build_part("position", "rope_scaled", dim=int(rot["dims"]), base=float(rot["base"]),
                                     factor=float(scaling["factor"]), original=float(scaling["original"]),
                                     fast=float(scaling["fast"]), slow=float(scaling["slow"]))
        else:
            shared[key] = build_part("position", "rope", dim=int(rot["dims"]), base=float(rot["base"]))
    return shared[key]


def build_dasusun_plan(config: DasusunConfig) -> ModelPlan:
    width, eps = config.width, config.eps
    positions: dict = {}

    def norm(name: str):
        return build_part("norm", "rmsnorm", size=width, eps=eps, weight_offset=1.0, weight_name=name)

    layers = []
    for place, spec in enumerate(config.layers):
        m = spec["mixer"]
        mixer = build_part(
            "mixer", spec["type"], hidden_size=width, n_heads=m["heads"], head_dim=m["dim"], rot_dim=m["rot_dim"],
            value_dim=m["vdim"], q_rank=m["q_rank"], kv_rank=m["kv_rank"], scale=m["scale"], norm_eps=eps,
            position=_position(m.get("rot"), positions), window=(m.get("mask") or {}).get("size"),
        )
        mlp = spec.get("mlp")
        ffn = None
        if mlp is not None:
            ffn = build_part("feed_forward", "gelu", hidden_size=width, intermediate_size=mlp["ff"], up_name="up", down_name="down")
        layers.append(build_part(
            "block", "sandwich", width=width, place=place, norm_in=norm("norm1"), mixer=mixer, norm_out_1=norm("norm1b"),
            norm_mid=norm("norm2") if ffn is not None else None, feed_forward=ffn,
            norm_out_2=norm("norm2b") if ffn is not None else None, conv_taps=config.taps,
        ))
    for block, follower in zip(layers, layers[1:]):
        block.next_block = follower
    embedding = TokenEmbedding(config.vocab, width, weight_name="embed")
    return ModelPlan(
        embedding=embedding,
        layers=layers,
        final_norm=norm("norm"),
        head=OutputHead(width, config.vocab, tied_to=embedding),
        run_list=[RunEntry(i) for i in range(len(layers))],
        positions=list(positions.values()),
        embedding_prefix="",
        layer_prefix="l{}.",
        final_norm_prefix="final.",
        head_prefix="lm_head.",
        keep_streams=len(layers) + 1,
    )
