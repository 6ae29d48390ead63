"""Grouped-query attention whose values are its keys, with norms over whole projections, a gate and a sink.

``q = W_q x`` (``n_q_heads`` heads of ``head_dim``) and ``k = W_k x`` (``n_kv_heads`` heads) are each RMS-normed over the
WHOLE projection (all heads at once, one weight per entry), then the first ``position.dim`` entries of every head are
rotated by position (entry ``i`` paired with ``i + dim/2``) and the rest pass.  The values are the keys as projected,
before norm and rotation: there is no value projection.  Scores are ``q . k * scale`` over a causal sliding window; with
``sink`` the softmax has one more term in its denominator, ``p_j = exp(s_j) / (1 + sum_i exp(s_i))``.  With ``gated``
the concatenated heads are multiplied by ``sigmoid(W_g x)`` before the output projection.

One packed product q | k | gate; one kernel for both norms, the rotation and the cache write (finished keys into the key
pages, keys as projected into the value pages); attention over the pages; the gate; the output projection.
"""

from __future__ import annotations

import torch

from ..ops import attention as attention_ops
from ..ops import functional as F
from ..ops.linear import linear
from .base import KVRequest, Mixer, PositionEncoding, StepContext, TensorSpec, register_part
from .delta_rule import _pad_rows

_NAMES = {"q": "q", "k": "k", "q_norm": "q.norm", "k_norm": "k.norm", "g": "g", "o": "o"}


class WideNormAttention(Mixer):
    graph_safe = True

    def __init__(self, hidden_size: int, n_q_heads: int, n_kv_heads: int, head_dim: int, norm_eps: float, scale: float,
                 position: PositionEncoding | None = None, window: int | None = None, sink: bool = True, gated: bool = True,
                 names: dict[str, str] | None = None):
        if n_q_heads % n_kv_heads:
            raise ValueError("query heads must be a multiple of key heads")
        self.hidden_size, self.n_q, self.n_kv, self.head_dim = int(hidden_size), int(n_q_heads), int(n_kv_heads), int(head_dim)
        self.norm_eps, self.scale, self.position = float(norm_eps), float(scale), position
        self.window = None if not window else int(window)
        self.sink, self.gated = bool(sink), bool(gated)
        self.rot = 0 if position is None else int(position.dim)
        if self.rot > self.head_dim:
            raise ValueError(f"{self.rot} rotated entries in heads of {self.head_dim}")
        self.names = {**_NAMES, **(names or {})}
        self.w_in = self.w_o = self.q_norm = self.k_norm = None

    def tensor_specs(self):
        n, W, nq, nk = self.names, self.hidden_size, self.n_q * self.head_dim, self.n_kv * self.head_dim
        specs = {n["q"]: TensorSpec((nq, W)), n["k"]: TensorSpec((nk, W)), n["q_norm"]: TensorSpec((nq,), "vector"),
                 n["k_norm"]: TensorSpec((nk,), "vector"), n["o"]: TensorSpec((W, nq))}
        if self.gated:
            specs[n["g"]] = TensorSpec((nq, W))
        return specs

    def load(self, tensors):
        n = self.names
        mats = [tensors[n["q"]], tensors[n["k"]]] + ([tensors[n["g"]]] if self.gated else [])
        if len({m.dtype for m in mats}) != 1:
            mats = [m.float() for m in mats]
        self.w_in = _pad_rows(torch.cat(mats, dim=0)).contiguous()
        self.w_o = tensors[n["o"]].contiguous()
        self.q_norm = tensors[n["q_norm"]].float().contiguous()
        self.k_norm = tensors[n["k_norm"]].float().contiguous()

    def weight_bytes(self):
        return sum(t.numel() * t.element_size() for t in (self.w_in, self.w_o))

    def cache_request(self):
        return KVRequest(self.n_kv, self.head_dim, self.window)

    def forward(self, x, ctx: StepContext, cache: F.PagedKV) -> torch.Tensor:
        cos = sin = None
        if self.rot:
            cos, sin = self.position.cos, self.position.sin
        write = not ctx.extras.get("cache_read_only", False)
        proj = linear(x, self.w_in)
        q = F.wide_norm_rope_write(proj, self.n_q, self.n_kv, self.head_dim, self.q_norm, self.k_norm, self.norm_eps, cos, sin,
                                   self.rot, ctx.tok_pos, ctx.tok_seq, ctx.slots, cache, ctx.max_position, write)
        o = attention_ops.paged_attention(q, cache, ctx, self.scale, self.window or 0, sink=self.sink)
        o = o.view(ctx.n_tokens, self.n_q * self.head_dim)
        if self.gated:
            o = F.sigmoid_gate(o, proj, (self.n_q + self.n_kv) * self.head_dim)
        return linear(o, self.w_o)


register_part("mixer", "wide_norm_attention", WideNormAttention)
