"""A plain, slow implementation of the Pofadra decoder, written from the design's equations.

Whole sequences, no cache, one function per mechanism, PyTorch in one working precision
(float64 for the oracle).  It shares no code with the library under test: it reads a dict of
tensors keyed by the model file's names and the config as a plain dict.

Notation: T tokens, W the model width; a mixer has H heads and G key heads (query or value head
``h`` reads key head ``h // (H / G)``), ``d`` key entries and ``dv`` value entries per head.
"""

from __future__ import annotations

import math

import torch

# When set to torch.bfloat16 every matrix product rounds its operands and its result to that type, while
# norms, angles, scores, softmax, the recurrence and the residual sums stay in the working precision: the
# "standard low-precision implementation" that the bfloat16 tests measure the library against.
LOWP: torch.dtype | None = None


def mm(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    if LOWP is None:
        return a @ b
    wide = a.dtype
    return (a.to(LOWP).to(wide) @ b.to(LOWP).to(wide)).to(LOWP).to(wide)


def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps): eps inside the root."""
    return x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps)


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def short_conv(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """x [T, C], w [C, taps]: y_t = sum_j w[:, j] * x_(t - taps + 1 + j), zeros before the start."""
    taps = w.shape[1]
    y = torch.zeros_like(x)
    for j in range(taps):
        back = taps - 1 - j
        if back == 0:
            y = y + w[:, j] * x
        elif back < x.shape[0]:
            y[back:] = y[back:] + w[:, j] * x[:-back]
    return y


def unit(x: torch.Tensor) -> torch.Tensor:
    """Rows scaled to length one: x / sqrt(sum(x^2) + 1e-6)."""
    return x / torch.sqrt(x.pow(2).sum(-1, keepdim=True) + 1e-6)


def delta_recurrence(q, k, v, g, beta):
    """One head.  q, k, g [T, d]; v [T, dv]; beta [T].  S [d, dv] starts at zero; per token
    S = g * S (rows), u = beta (v - S^T k), S += k u^T, o = S^T q."""
    T, d = q.shape
    S = torch.zeros(d, v.shape[1], dtype=q.dtype)
    out = []
    for t in range(T):
        S = g[t][:, None] * S
        u = beta[t] * (v[t] - S.T @ k[t])
        S = S + torch.outer(k[t], u)
        out.append(S.T @ q[t])
    return torch.stack(out)


def channel_delta(h: torch.Tensor, w: dict, p: str, m: dict, eps: float) -> torch.Tensor:
    """The gated delta rule with a decay per head and key channel.  h [T, W] -> [T, W]."""
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = silu(short_conv(mm(h, w[p + "q"].T), w[p + "q.conv"])).view(T, G, d)
    k = silu(short_conv(mm(h, w[p + "k"].T), w[p + "k.conv"])).view(T, G, d)
    v = silu(short_conv(mm(h, w[p + "v"].T), w[p + "v.conv"])).view(T, H, dv)
    q = unit(q) * d ** -0.5
    k = unit(k)
    beta = torch.sigmoid(mm(h, w[p + "b"].T))  # [T, H]
    step = torch.nn.functional.softplus(mm(mm(h, w[p + "a1"].T), w[p + "a2"].T) + w[p + "dt_bias"]).view(T, H, d)
    g = torch.exp(-torch.exp(w[p + "A_log"])[None, :, None] * step)
    gate = torch.sigmoid(mm(mm(h, w[p + "g1"].T), w[p + "g2"].T)).view(T, H, dv)
    outs = []
    for head in range(H):
        kh = head // (H // G)
        o = delta_recurrence(q[:, kh], k[:, kh], v[:, head], g[:, head], beta[:, head])
        outs.append(rms(o, eps) * w[p + "norm"] * gate[:, head])
    return mm(torch.stack(outs, 1).reshape(T, H * dv), w[p + "o"].T)


def rotate_part(x: torch.Tensor, dims: int, base: float) -> torch.Tensor:
    """x [T, heads, d]: the first ``dims`` entries of each head turn by position * base^(-2i/dims), entry i paired
    with i + dims/2; the rest pass."""
    T = x.shape[0]
    half = dims // 2
    f = base ** (-2.0 * torch.arange(half, dtype=x.dtype) / dims)
    a = torch.arange(T, dtype=x.dtype)[:, None] * f[None, :]
    cos, sin = a.cos()[:, None, :], a.sin()[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * cos - v * sin, v * cos + u * sin, x[..., dims:]], -1)


def window_attention(h: torch.Tensor, w: dict, p: str, m: dict, eps: float) -> torch.Tensor:
    """Attention whose values are the keys as projected; norm over the whole projection; rotation on part of a
    head; sliding window; a softmax with one more in the denominator; output gate."""
    H, G, d = m["heads"], m["kv_heads"], m["dim"]
    T = h.shape[0]
    q = mm(h, w[p + "q"].T)
    k = mm(h, w[p + "k"].T)
    v = k.view(T, G, d)
    q = (rms(q, eps) * w[p + "q.norm"]).view(T, H, d)
    k = (rms(k, eps) * w[p + "k.norm"]).view(T, G, d)
    rot = m.get("rot")
    if rot:
        q, k = rotate_part(q, rot["dims"], rot["base"]), rotate_part(k, rot["dims"], rot["base"])
    i = torch.arange(T)
    seen = (i[:, None] >= i[None, :])
    if m.get("mask"):
        seen &= (i[:, None] - i[None, :]) < m["mask"]["size"]
    outs = []
    for head in range(H):
        kh = head // (H // G)
        s = (q[:, head] @ k[:, kh].T) * m["scale"]
        s = s.masked_fill(~seen, -math.inf)
        top = s.max(-1, keepdim=True).values.clamp_min(0.0)
        e = torch.exp(s - top)
        prob = e / (torch.exp(-top) + e.sum(-1, keepdim=True))
        outs.append(prob @ v[:, kh])
    o = torch.stack(outs, 1).reshape(T, H * d) * torch.sigmoid(mm(h, w[p + "g"].T))
    return mm(o, w[p + "o"].T)


def route(h: torch.Tensor, w: dict, p: str, r: dict):
    """Chosen experts [T, top] and their weights.  Choice by sigmoid score plus correction, limited to the best
    groups (a group's score: its two largest choice scores added); weights from the score without correction."""
    E, top = r["experts"], r["top"]
    s = torch.sigmoid(h @ w[p + "router"].to(h.dtype).T)
    choice = s + w[p + "correction"].to(h.dtype)
    groups = r.get("groups")
    if groups:
        n, keep = groups["count"], groups["keep"]
        per = choice.view(-1, n, E // n)
        score = per.topk(min(2, E // n), -1).values.sum(-1)
        best = score.topk(keep, -1).indices
        allowed = torch.zeros_like(score, dtype=torch.bool).scatter_(1, best, True)
        choice = choice.masked_fill(~allowed[:, :, None].expand_as(per).reshape(-1, E), -math.inf)
    chosen = choice.topk(top, -1).indices
    return chosen, s.gather(1, chosen) * r["scale"]


def experts(h: torch.Tensor, w: dict, p: str, mlp: dict) -> torch.Tensor:
    chosen, weight = route(h.to(torch.bfloat16).to(h.dtype) if LOWP is not None else h, w, p, mlp["router"])
    out = torch.zeros_like(h)
    for e in range(mlp["router"]["experts"]):
        rows, place = (chosen == e).nonzero(as_tuple=True)
        if rows.numel() == 0:
            continue
        x = h[rows]
        y = mm(silu(mm(x, w[f"{p}e{e}.gate"].T)) * mm(x, w[f"{p}e{e}.up"].T), w[f"{p}e{e}.down"].T)
        out.index_add_(0, rows, weight[rows, place][:, None] * y)
    return out


MIXERS = {"channel_delta": channel_delta, "attention": window_attention}


def forward(tokens: torch.Tensor, weights: dict, config: dict, dtype=torch.float64, keep_layers: list | None = None) -> torch.Tensor:
    """Logits [T, vocab] of one sequence.  ``keep_layers``: a list that receives the stream after every layer."""
    w = {name: (t.to(dtype) if t.is_floating_point() else t) for name, t in weights.items()}
    eps = config["norm"]["eps"]
    x = w["embed"][tokens] * (config.get("embedding") or {"scale": 1.0})["scale"]
    for i, layer in enumerate(config["layers"]):
        h = rms(x, eps) * w[f"l{i}.norm1"]
        branch = MIXERS[layer["type"]](h, w, f"l{i}.mix.", layer["mixer"], eps)
        if layer.get("mlp") is not None:
            branch = branch + experts(h, w, f"l{i}.mlp.", layer["mlp"])
        x = x + branch
        if keep_layers is not None:
            keep_layers.append(x)
    logits = mm(rms(x, eps) * w["final.norm"], w["head"].T)
    cap = config.get("logit_softcap")
    return cap * torch.tanh(logits / cap) if cap else logits
