"""A recurrent mixer: the gated delta rule with a decay per head and key channel.

Per head a state ``S [d, dv]`` of 32-bit floats, zero at the start of a sequence, is carried from token to token:

    S <- diag(g_t) S ;  u_t = beta_t (v_t - S^T k_t) ;  S <- S + k_t u_t^T ;  o_t = S^T q_t

``q_t, k_t`` (``n_kv_heads`` heads of ``key_dim``; value head ``h`` reads key head ``h // (n_heads / n_kv_heads)``) and
``v_t`` (``n_heads`` heads of ``value_dim``) are projections of the layer's input that pass a short causal convolution
over time (per channel, no bias, zeros before the start) and SiLU; q and k are then scaled to unit length per head
(``x / sqrt(sum x^2 + 1e-6)``), q also by ``key_dim ** -0.5``.  ``beta_t = sigmoid(W_b x)`` per head, and the decay
``g_t = exp(-exp(A_h) * softplus(W_a2 (W_a1 x) + dt_bias))`` per head and key channel.  A head's read-out is divided by its
root mean square over ``value_dim``, multiplied by one weight vector for all heads and by ``sigmoid(W_g2 (W_g1 x))``, and
the heads go through the output projection.

What a sequence keeps between steps: the states of all heads and the convolutions' last ``taps - 1`` inputs.

A step's kernels: the packed projection q | k | v | b; the packed first halves of the two low-rank paths and one product
for their second halves (a block-diagonal matrix); one kernel for convolutions, activations, unit lengths, decays and
beta; one that moves the convolution state on; the recurrence; norm and gate; the output projection.  Prompts,
portions of prompts and single tokens take the same path.
"""

from __future__ import annotations

import torch

from ..ops import functional as F
from ..ops.linear import linear
from .base import Mixer, StateRequest, StepContext, TensorSpec, register_part

_NAMES = {"q": "q", "k": "k", "v": "v", "q_conv": "q.conv", "k_conv": "k.conv", "v_conv": "v.conv", "b": "b", "a_log": "A_log",
          "norm": "norm", "a1": "a1", "a2": "a2", "dt_bias": "dt_bias", "g1": "g1", "g2": "g2", "o": "o"}


def _pad_rows(t: torch.Tensor, multiple: int = 8) -> torch.Tensor:
    extra = -t.shape[0] % multiple
    return t if not extra else torch.cat([t, t.new_zeros((extra, t.shape[1]))], dim=0)


class ChannelDeltaRule(Mixer):
    graph_safe = True  # kernels only; starts, slots and lengths are read from device memory

    def __init__(self, hidden_size: int, n_heads: int, n_kv_heads: int, key_dim: int, value_dim: int, conv_taps: int,
                 norm_eps: float, decay_rank: int | None = None, gate_rank: int | None = None, names: dict[str, str] | None = None):
        """``decay_rank`` / ``gate_rank``: inner sizes of the two low-rank paths.  A model file chooses them by its tensors'
        shapes; the numbers given here (default: ``key_dim // 2`` rounded up to a multiple of 8) are what the
        random-weights mode writes."""
        if n_heads % n_kv_heads:
            raise ValueError("value heads must be a multiple of key heads")
        self.hidden_size, self.n_heads, self.n_kv = int(hidden_size), int(n_heads), int(n_kv_heads)
        self.d, self.dv, self.taps, self.norm_eps = int(key_dim), int(value_dim), int(conv_taps), float(norm_eps)
        if min(self.hidden_size, self.n_heads, self.n_kv, self.d, self.dv, self.taps) <= 0:
            raise ValueError("delta rule sizes must be positive")
        default = -(-max(self.d // 2, 8) // 8) * 8
        self.decay_rank, self.gate_rank = int(decay_rank or default), int(gate_rank or default)
        self.names = {**_NAMES, **(names or {})}
        self.channels = 2 * self.n_kv * self.d + self.n_heads * self.dv
        self.w_in = self.w_low1 = self.w_low2 = self.w_o = self.conv_w = self.a_log = self.dt_bias = self.norm_w = None

    def tensor_specs(self):
        n, W, H, G, d, dv = self.names, self.hidden_size, self.n_heads, self.n_kv, self.d, self.dv
        conv = (0.0, 0.4)
        return {
            n["q"]: TensorSpec((G * d, W)), n["q_conv"]: TensorSpec((G * d, self.taps), init=conv),
            n["k"]: TensorSpec((G * d, W)), n["k_conv"]: TensorSpec((G * d, self.taps), init=conv),
            n["v"]: TensorSpec((H * dv, W)), n["v_conv"]: TensorSpec((H * dv, self.taps), init=conv),
            n["b"]: TensorSpec((H, W)),
            n["a_log"]: TensorSpec((H,), "vector", init=(-1.0, 0.7)),
            n["norm"]: TensorSpec((dv,), "vector"),
            n["a1"]: TensorSpec((self.decay_rank, W), free=(0,)), n["a2"]: TensorSpec((H * d, self.decay_rank), free=(1,)),
            n["dt_bias"]: TensorSpec((H * d,), "vector", init=(-1.0, 1.0)),
            n["g1"]: TensorSpec((self.gate_rank, W), free=(0,)), n["g2"]: TensorSpec((H * dv, self.gate_rank), free=(1,)),
            n["o"]: TensorSpec((W, H * dv)),
        }

    def load(self, tensors):
        n, H, d, dv = self.names, self.n_heads, self.d, self.dv
        get = lambda key: tensors[n[key]]
        a1, a2, g1, g2 = get("a1"), get("a2"), get("g1"), get("g2")
        if a1.shape[0] != a2.shape[1] or g1.shape[0] != g2.shape[1]:
            raise ValueError(f"the low-rank paths' halves do not meet: {tuple(a1.shape)} x {tuple(a2.shape)}, {tuple(g1.shape)} x {tuple(g2.shape)}")
        self.decay_rank, self.gate_rank = int(a1.shape[0]), int(g1.shape[0])
        mats = [get("q"), get("k"), get("v"), get("b"), a1, a2, g1, g2]
        kind = torch.float32 if any(m.dtype == torch.float32 for m in mats) else mats[0].dtype
        cast = lambda t: t.to(kind)
        self.w_in = _pad_rows(torch.cat([cast(get("q")), cast(get("k")), cast(get("v")), cast(get("b"))], dim=0)).contiguous()
        low1 = _pad_rows(torch.cat([cast(a1), cast(g1)], dim=0))
        self.w_low1 = low1.contiguous()
        low2 = low1.new_zeros((H * d + H * dv, low1.shape[0]))
        low2[:H * d, :self.decay_rank] = cast(a2)
        low2[H * d:, self.decay_rank:self.decay_rank + self.gate_rank] = cast(g2)
        self.w_low2 = low2.contiguous()
        self.w_o = get("o").contiguous()
        self.conv_w = torch.cat([get("q_conv"), get("k_conv"), get("v_conv")], dim=0).float().contiguous()
        self.a_log, self.dt_bias, self.norm_w = (get(k).float().contiguous() for k in ("a_log", "dt_bias", "norm"))

    def weight_bytes(self):
        return sum(t.numel() * t.element_size() for t in (self.w_in, self.w_low1, self.w_low2, self.w_o, self.conv_w))

    def cache_request(self):
        requests = [StateRequest((self.n_heads, self.d, self.dv), torch.float32)]
        if self.taps > 1:
            requests.append(StateRequest((self.taps - 1, self.channels), torch.float32))
        return requests

    def forward(self, x, ctx: StepContext, cache) -> torch.Tensor:
        if ctx.extras.get("cache_read_only", False):
            raise ValueError("a recurrent mixer advances its state at every step: it cannot run on another entry's storage")
        state = cache[0]
        conv_state = cache[1] if self.taps > 1 else None
        proj = linear(x, self.w_in)
        low = linear(linear(x, self.w_low1), self.w_low2, torch.float32)
        q, k, v, g, beta = F.delta_prepare(proj, low, self.conv_w, conv_state, self.a_log, self.dt_bias, ctx.tok_pos, ctx.tok_seq,
                                           ctx.cu_q, ctx.slots, self.n_heads, self.n_kv, self.d, self.dv, self.taps,
                                           roll_single=ctx.all_single)
        if conv_state is not None and not ctx.all_single:
            F.conv_roll(proj, conv_state, ctx.cu_q, ctx.slots, ctx.n_seqs, self.channels)
        o = F.delta_scan(q, k, v, g, beta, state, ctx.cu_q, ctx.slots, ctx.n_seqs)
        y = F.head_norm_gate(o, self.norm_w, low, self.n_heads * self.d, self.norm_eps, ctx.dtype)
        return linear(y, self.w_o)


register_part("mixer", "channel_delta", ChannelDeltaRule)
