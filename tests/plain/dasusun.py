"""A plain, slow implementation of the Dasusun decoder, written from the design's equations.

Whole sequences, no cache, one function per mechanism, PyTorch in one working precision
(float64 for the oracle).  It shares no code with the library under test: it reads a dict of
tensors keyed by the model file's names and the config as a plain dict.

Notation: T tokens, W the model width, H heads; per head ``dn`` unrotated and ``dr`` rotated
query/key dimensions and ``dv`` value dimensions; R the latent size of keys and values.
"""

from __future__ import annotations

import math

import torch

# When set to torch.bfloat16 every matrix product rounds its operands and its result to that type, while
# norms, angles, scores, softmax and the residual sums stay in the working precision: the "standard
# low-precision implementation" that the bfloat16 tests measure the library against.
LOWP: torch.dtype | None = None


def mm(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    if LOWP is None:
        return a @ b
    wide = a.dtype
    return (a.to(LOWP).to(wide) @ b.to(LOWP).to(wide)).to(LOWP).to(wide)


def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps): eps inside the root."""
    return x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps)


def norm_around_zero(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """A layer's norms and the model's last norm: the stored weight is an offset from one."""
    return rms(x, eps) * (1.0 + w)


def norm_plain(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """The norms inside the mixer (on the latents): the weight multiplies as it is stored."""
    return rms(x, eps) * w


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z.pow(3))))


def causal_conv(h: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """h [T, W], w [W, taps]: y_t = sum_j w[:, j] * h_(t - taps + 1 + j), zeros before the start.
    The caller adds the result to h."""
    taps = w.shape[1]
    y = torch.zeros_like(h)
    for j in range(taps):
        back = taps - 1 - j
        if back == 0:
            y = y + w[:, j] * h
        elif back < h.shape[0]:
            y[back:] = y[back:] + w[:, j] * h[:-back]
    return y


def rotary_frequencies(dims: int, base: float, scaling: dict | None, dtype=torch.float64) -> tuple[torch.Tensor, float]:
    """The dims/2 frequencies and the factor on cos and sin.  Without scaling: base^(-2i/dims) and 1."""
    i = torch.arange(dims // 2, dtype=dtype)
    f = base ** (-2.0 * i / dims)
    if not scaling:
        return f, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def turn_dim(turns: float) -> float:
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(turn_dim(float(scaling["fast"]))), 0)
    hi = min(math.ceil(turn_dim(float(scaling["slow"]))), dims - 1)
    ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
    f = f / factor * ramp + f * (1.0 - ramp)
    return f, 0.1 * math.log(factor) + 1.0


def rotate(x: torch.Tensor, positions: torch.Tensor, dims: int, base: float, scaling: dict | None) -> torch.Tensor:
    """x [T, ..., d]: the first ``dims`` entries of the last axis are rotated, entry i paired with i + dims/2;
    the rest passes."""
    f, mag = rotary_frequencies(dims, base, scaling, x.dtype)
    angle = positions.to(x.dtype)[:, None] * f[None, :]
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [dims // 2]
    cos, sin = (angle.cos() * mag).reshape(shape), (angle.sin() * mag).reshape(shape)
    u, v = x[..., :dims // 2], x[..., dims // 2:dims]
    return torch.cat([u * cos - v * sin, v * cos + u * sin, x[..., dims:]], dim=-1)


def latent_attention(h: torch.Tensor, t: dict, m: dict, eps: float, positions: torch.Tensor) -> torch.Tensor:
    """The mixer on its input h [T, W]; ``t`` holds its tensors by their short names, ``m`` its sizes."""
    T = h.shape[0]
    H, dn, dr, dv, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    rot = m["rot"]
    cq = norm_plain(mm(h, t["dq"].T), t["dq.norm"], eps)
    q = mm(cq, t["uq"].T).view(T, H, dn + dr)
    q_n, q_r = q[..., :dn], q[..., dn:]
    kv = mm(h, t["dkv"].T)
    c = norm_plain(kv[:, :R], t["dkv.norm"], eps)
    k_r = kv[:, R:]  # one rotated part for all heads, not normed
    k_n = mm(c, t["uk"].T).view(T, H, dn)
    v = mm(c, t["uv"].T).view(T, H, dv)
    q_r = rotate(q_r, positions, rot["dims"], rot["base"], rot.get("scaling"))
    k_r = rotate(k_r, positions, rot["dims"], rot["base"], rot.get("scaling"))
    scores = (torch.einsum("ihd,jhd->hij", q_n, k_n) + torch.einsum("ihd,jd->hij", q_r, k_r)) * m["scale"]
    i = positions[:, None]
    j = positions[None, :]
    seen = (i - j >= 0)
    mask = m.get("mask")
    if mask:
        seen = seen & (i - j < mask["size"])
    scores = scores.masked_fill(~seen[None], float("-inf"))
    p = torch.softmax(scores, dim=-1)
    if LOWP is not None:
        p = p.to(LOWP).to(h.dtype)
    o = torch.einsum("hij,jhd->ihd", p, v).reshape(T, H * dv)
    if LOWP is not None:
        o = o.to(LOWP).to(h.dtype)
    return mm(o, t["o"].T)


def dense_feed_forward(h: torch.Tensor, t: dict) -> torch.Tensor:
    return mm(gelu_tanh(mm(h, t["up"].T)), t["down"].T)


def layer(x: torch.Tensor, w: dict, prefix: str, spec: dict, config: dict, positions: torch.Tensor) -> torch.Tensor:
    """One layer on its input stream x [T, W]; returns the layer's result (before the depth average)."""
    eps = config["norm"]["eps"]

    def get(name):
        return w[prefix + name].to(x.dtype)

    h = norm_around_zero(x, get("norm1"), eps)
    if config.get("canon"):
        h = h + causal_conv(h, get("canon1"))
    if spec["type"] != "latent_attention":
        raise ValueError(f"no mixer {spec['type']!r} in this design")
    tensors = {n: get("mix." + n) for n in ("dq", "dq.norm", "uq", "dkv", "dkv.norm", "uk", "uv", "o")}
    y = latent_attention(h, tensors, spec["mixer"], eps, positions)
    x = x + get("ls1") * norm_around_zero(y, get("norm1b"), eps)
    if spec.get("mlp"):
        if spec["mlp"]["kind"] != "dense":
            raise ValueError(f"no feed-forward {spec['mlp']['kind']!r} in this design")
        h = norm_around_zero(x, get("norm2"), eps)
        y = dense_feed_forward(h, {"up": get("mlp.up"), "down": get("mlp.down")})
        x = x + get("ls2") * norm_around_zero(y, get("norm2b"), eps)
    return x


def forward(ids: torch.Tensor, w: dict, config: dict, dtype=torch.float64, streams: list | None = None) -> torch.Tensor:
    """Logits [T, vocab] of one whole sequence.  ``streams``, if a list, receives the stream after every layer
    (after the depth average)."""
    positions = torch.arange(ids.shape[0])
    table = w["embed"].to(dtype)
    x = table[ids.long()]
    kept = [x]
    for i, spec in enumerate(config["layers"]):
        kept.append(layer(x, w, f"l{i}.", spec, config, positions))
        mix = w[f"l{i}.dwa"].to(dtype)
        x = sum(mix[j] * kept[j] for j in range(i + 2))
        if streams is not None:
            streams.append(x)
    z = norm_around_zero(x, w["final.norm"].to(dtype), config["norm"]["eps"])
    return mm(z, table.T)
