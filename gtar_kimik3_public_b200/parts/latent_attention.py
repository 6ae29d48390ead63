"""Attention whose keys and values are made from one cached latent per position.

Queries go through a latent of their own: ``c_q = rmsnorm(W_dq x)``, ``q = W_uq c_q``, laid out head by head as
``[dim unrotated | rot_dim rotated]``.  ``W_dkv x`` gives the kv latent (``kv_rank`` entries, then RMS-normed) and
``rot_dim`` more entries that are one rotated key part for all heads.  Per head the unrotated key is ``U_k c`` and the
value ``U_v c``; the score is ``(q_n . U_k c + q_r . k_r) * scale`` over the visible keys (causal, optionally a sliding
window), an ordinary softmax, and the heads' outputs go through ``W_o``.

Only the normed latent and the rotated key part are kept per position (one row for all heads).  The per-head
matrices never touch the cache: ``q_n . U_k c = (U_k^T q_n) . c``, so the query is carried into the latent before
attention, attention runs over the cached rows with the latent as the value, and ``U_v`` is applied to the result.

A step's kernels: the packed down-projection ``[W_dq; W_dkv]``; one kernel for both norms, the key part's rotation and
the cache write; the up-projection of the queries; a batched product (one per head) that carries the queries; the
attention kernel, which rotates the queries' own part itself; a batched product for the values; the output projection.
"""

from __future__ import annotations

import torch

from ..ops import attention as attention_ops
from ..ops import functional as F
from ..ops.linear import linear
from .base import Mixer, PositionEncoding, RowsRequest, StepContext, TensorSpec, register_part

_NAMES = {"dq": "dq", "dq_norm": "dq.norm", "uq": "uq", "dkv": "dkv", "dkv_norm": "dkv.norm", "uk": "uk", "uv": "uv", "o": "o"}


class LatentAttention(Mixer):
    graph_safe = True  # kernels only; every per-step number is read from device memory

    def __init__(self, hidden_size: int, n_heads: int, head_dim: int, rot_dim: int, value_dim: int, q_rank: int, kv_rank: int,
                 scale: float, norm_eps: float, position: PositionEncoding | None, window: int | None = None,
                 names: dict[str, str] | None = None):
        """``position``: tables of cos and sin for ``position.dim`` of the ``rot_dim`` rotated entries (the first ones;
        the rest pass unchanged), or None for no rotation.  ``scale`` multiplies every score as it is given."""
        self.hidden_size, self.n_heads, self.head_dim, self.rot_dim = int(hidden_size), int(n_heads), int(head_dim), int(rot_dim)
        self.value_dim, self.q_rank, self.kv_rank = int(value_dim), int(q_rank), int(kv_rank)
        self.scale, self.norm_eps, self.position = float(scale), float(norm_eps), position
        self.window = None if not window else int(window)
        self.rot_dims = 0 if position is None else int(position.dim)
        if self.rot_dims > self.rot_dim:
            raise ValueError(f"{self.rot_dims} rotated dimensions in a part of {self.rot_dim}")
        if min(self.n_heads, self.head_dim, self.value_dim, self.q_rank, self.kv_rank) <= 0 or self.rot_dim < 0:
            raise ValueError("latent attention sizes must be positive")
        self.names = {**_NAMES, **(names or {})}
        self.w_down = self.w_uq = self.w_uk_t = self.w_uv = self.w_o = self.q_norm = self.kv_norm = None

    def tensor_specs(self):
        n, H = self.names, self.n_heads
        return {
            n["dq"]: TensorSpec((self.q_rank, self.hidden_size)),
            n["dq_norm"]: TensorSpec((self.q_rank,), "vector"),
            n["uq"]: TensorSpec((H * (self.head_dim + self.rot_dim), self.q_rank)),
            n["dkv"]: TensorSpec((self.kv_rank + self.rot_dim, self.hidden_size)),
            n["dkv_norm"]: TensorSpec((self.kv_rank,), "vector"),
            n["uk"]: TensorSpec((H * self.head_dim, self.kv_rank)),
            n["uv"]: TensorSpec((H * self.value_dim, self.kv_rank)),
            n["o"]: TensorSpec((self.hidden_size, H * self.value_dim)),
        }

    def load(self, tensors):
        n, H = self.names, self.n_heads
        down = [tensors[n["dq"]], tensors[n["dkv"]]]
        if down[0].dtype != down[1].dtype:
            down = [t.float() for t in down]
        self.w_down = torch.cat(down, dim=0).contiguous()  # one product for both latents
        self.w_uq = tensors[n["uq"]].contiguous()
        # per head: [kv_rank, dim] so that the product with a head's unrotated query gives its carried form
        self.w_uk_t = tensors[n["uk"]].view(H, self.head_dim, self.kv_rank).transpose(1, 2).contiguous()
        self.w_uv = tensors[n["uv"]].view(H, self.value_dim, self.kv_rank).contiguous()
        self.w_o = tensors[n["o"]].contiguous()
        self.q_norm = tensors[n["dq_norm"]].float().contiguous()
        self.kv_norm = tensors[n["dkv_norm"]].float().contiguous()

    def weight_bytes(self):
        return sum(t.numel() * t.element_size() for t in (self.w_down, self.w_uq, self.w_uk_t, self.w_uv, self.w_o))

    def cache_request(self):
        return RowsRequest(self.kv_rank + self.rot_dim, self.window)

    def forward(self, x, ctx: StepContext, cache: F.PagedRows) -> torch.Tensor:
        T, H, dn, dr, R = ctx.n_tokens, self.n_heads, self.head_dim, self.rot_dim, self.kv_rank
        cos = sin = None
        if self.rot_dims:
            cos, sin = self.position.cos, self.position.sin
        write = not ctx.extras.get("cache_read_only", False)
        both = linear(x, self.w_down)
        c_q = F.latent_prepare(both, self.q_rank, R, dr, self.rot_dims, self.q_norm, self.kv_norm, self.norm_eps, cos, sin,
                               ctx.tok_pos, ctx.tok_seq, ctx.slots, cache, ctx.max_position, write)
        q = linear(c_q, self.w_uq).view(T, H, dn + dr)
        carried = torch.empty((H, T, R), dtype=x.dtype, device=x.device)
        F.linear_batched(q[:, :, :dn].transpose(0, 1), self.w_uk_t, carried)
        mixed = torch.empty((H, T, R), dtype=x.dtype, device=x.device)
        attention_ops.latent_attention(carried.transpose(0, 1), q, dn, dr, self.rot_dims, cos, sin, cache, ctx, self.scale,
                                       self.window or 0, mixed.transpose(0, 1))
        o = torch.empty((T, H * self.value_dim), dtype=x.dtype, device=x.device)
        F.linear_batched(mixed, self.w_uv, o.view(T, H, self.value_dim).transpose(0, 1))
        return linear(o, self.w_o)


register_part("mixer", "latent_attention", LatentAttention)
