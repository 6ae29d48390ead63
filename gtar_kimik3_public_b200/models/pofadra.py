"""The Pofadra decoder put together from parts.

Token embedding times a constant; per layer a ``ParallelBlock`` (one RMS norm that both branches read, their sum added
to the stream) around either the gated delta rule with per-channel decay (``channel_delta``: a recurrent state per
sequence) or windowed attention whose values are its keys (``attention``: norms over whole projections, partial
rotation, a sink in the softmax, an output gate), and a feed-forward of routed experts (or none); the model's last
norm; an output head of its own whose logits are capped by a tanh.  Each layer's sizes come from its own entry of the
config, so layers may differ in everything and come in any order.  Tensor names: ``embed``, ``l<i>.norm1``,
``l<i>.mix.*``, ``l<i>.mlp.*``, ``final.norm``, ``head``.
"""

from __future__ import annotations

from ..config.pofadra import PofadraConfig
from ..parts.base import build_part
from ..parts.embedding import OutputHead, TokenEmbedding
from .model import ModelPlan, RunEntry


def build_pofadra_plan(config: PofadraConfig) -> ModelPlan:
    width, eps = config.width, config.eps
    positions: dict = {}

    def rotation(rot: dict | None):
        """One table per distinct rotation (layers with the same constants read the same tables)."""
        if not rot:
            return None
        key = (int(rot["dims"]), float(rot["base"]))
        if key not in positions:
            positions[key] = build_part("position", "rope", dim=key[0], base=key[1], precise=True)
        return positions[key]

    layers = []
    for spec in config.layers:
        m = spec["mixer"]
        if spec["type"] == "channel_delta":
            mixer = build_part("mixer", "channel_delta", hidden_size=width, n_heads=m["heads"], n_kv_heads=m["kv_heads"],
                               key_dim=m["dim"], value_dim=m["vdim"], conv_taps=m["conv"], norm_eps=eps,
                               decay_rank=m.get("decay_rank"), gate_rank=m.get("gate_rank"))
        else:
            mixer = build_part("mixer", "wide_norm_attention", hidden_size=width, n_q_heads=m["heads"], n_kv_heads=m["kv_heads"],
                               head_dim=m["dim"], norm_eps=eps, scale=m["scale"], position=rotation(m.get("rot")),
                               window=(m.get("mask") or {}).get("size"), sink=True, gated=True)
        mlp = spec.get("mlp")
        ffn = None
        if mlp is not None:
            r = mlp["router"]
            groups = r.get("groups") or {"count": 1, "keep": 1}
            ffn = build_part("feed_forward", "routed_experts", hidden_size=width, expert_size=mlp["expert"]["ff"], n_experts=r["experts"],
                             top=r["top"], route_scale=r["scale"], n_groups=groups["count"], keep_groups=groups["keep"])
        norm = build_part("norm", "rmsnorm", size=width, eps=eps, weight_name="norm1")
        layers.append(build_part("block", "parallel", norm=norm, mixer=mixer, feed_forward=ffn))
    return ModelPlan(
        embedding=TokenEmbedding(config.vocab, width, weight_name="embed", scale=config.embedding_scale),
        layers=layers,
        final_norm=build_part("norm", "rmsnorm", size=width, eps=eps, weight_name="norm"),
        head=OutputHead(width, config.vocab, weight_name="head", softcap=config.logit_softcap),
        run_list=[RunEntry(i) for i in range(len(layers))],
        positions=list(positions.values()),
        embedding_prefix="",
        layer_prefix="l{}.",
        final_norm_prefix="final.",
        head_prefix="",
    )
