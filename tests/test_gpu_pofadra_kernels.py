"""The kernels of the delta rule, the routed experts and the wide-norm attention, each alone against the plain
function of the same mechanism, at sizes of their own; with inputs made so that a fault shows where random numbers
would hide it (a state that must survive a change of slot, a key at a window's edge whose score stands out, a sink
that carries most of the weight, groups whose best expert must lose)."""

import math

import pytest
import torch

from tests.plain import pofadra as plain
from tests.test_gpu_kernels import DEV, F, fill_pages, rand, scrambled_pages

pytestmark = pytest.mark.gpu


def i32(values):
    return torch.tensor(values, dtype=torch.int32, device=DEV)


# ------------------------------------------------------------------ the recurrence
@pytest.mark.parametrize("H,G,d,dv", [(4, 2, 24, 40), (2, 2, 64, 16), (3, 1, 132, 36), (5, 5, 8, 8), (2, 1, 128, 128), (1, 1, 256, 33)])
def test_delta_scan_against_the_plain_recurrence_under_every_cut(H, G, d, dv):
    """Three sequences of unequal lengths in scattered slots, cut into a prompt, portions of 2 and 5 tokens and single
    tokens: the 32-bit results are those of the whole prompt bit for bit, and the oracle's within rounding."""
    lens = [37, 1, 18]
    slots = [5, 0, 3]
    data = []
    for i, n in enumerate(lens):
        q = plain.unit(rand(n, G, d, seed=10 + i)) * d**-0.5
        k = plain.unit(rand(n, G, d, seed=20 + i))
        v = rand(n, H, dv, seed=30 + i)
        g = torch.sigmoid(rand(n, H, d, seed=40 + i) + 2.0)
        beta = torch.sigmoid(rand(n, H, seed=50 + i))
        data.append((q, k, v, g, beta))

    def run(cuts):
        state = torch.full((7, H, d, dv), float("nan"), device=DEV)
        state[slots] = 0.0
        done = [0, 0, 0]
        outs = [[], [], []]
        for cut in cuts:  # cut: tokens each sequence brings in this step (0: not in the step)
            live = [i for i in range(3) if cut[i]]
            parts = [[t[done[i]:done[i] + cut[i]] for t in data[i]] for i in live]
            packed = [torch.cat([p[j] for p in parts]).float().contiguous().to(DEV) for j in range(5)]
            starts = [0]
            for i in live:
                starts.append(starts[-1] + cut[i])
            o = F().delta_scan(*packed, state, i32(starts), i32([slots[i] for i in live]), len(live))
            for n, i in enumerate(live):
                outs[i].append(o[starts[n]:starts[n + 1]])
                done[i] += cut[i]
        assert done == lens
        return [torch.cat(o) for o in outs], state

    whole, state_whole = run([lens])
    for i in range(3):
        q, k, v, g, beta = data[i]
        for h in range(H):
            want = plain.delta_recurrence(q[:, h // (H // G)], k[:, h // (H // G)], v[:, h], g[:, h], beta[:, h])
            err = (whole[i][:, h].double().cpu() - want).abs().max().item()
            assert err < 2e-5 * (1 + want.abs().max().item()), f"sequence {i} head {h}: {err:.3e}"
    cuts = [[20, 1, 2], [2, 0, 2], [5, 0, 5], [1, 0, 1], [1, 0, 1]] + [[1, 0, 1]] * 7 + [[1, 0, 0]]
    stepped, state_stepped = run(cuts)
    for i in range(3):
        assert torch.equal(stepped[i], whole[i]), f"sequence {i}: cutting the prompt changed 32-bit results"
    assert torch.equal(state_stepped[slots], state_whole[slots])
    assert torch.isnan(state_whole[[1, 2, 4, 6]]).all()  # no other slot was touched


def test_delta_scan_keeps_what_only_the_state_remembers():
    """A value written at the first token with no decay and never overwritten (later keys are orthogonal to the first) is
    read back 300 tokens later, across many staged groups of tokens, exactly."""
    d, dv, n = 16, 8, 301
    q = torch.zeros(n, 1, d)
    k = torch.zeros(n, 1, d)
    k[0, 0, 3] = 1.0
    for t in range(1, n):
        k[t, 0, 4 + t % 12] = 1.0
    v = rand(n, 1, dv, seed=3).float()
    g = torch.ones(n, 1, d)
    beta = torch.ones(n, 1)
    q[-1, 0, 3] = 1.0
    state = torch.zeros(1, 1, d, dv, device=DEV)
    o = F().delta_scan(q.to(DEV), k.to(DEV), v.to(DEV), g.to(DEV), beta.to(DEV), state, i32([0, n]), i32([0]), 1)
    assert torch.equal(o[-1, 0].cpu(), v[0, 0])
    assert (o[:-1] == 0).all()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,d,dv,taps", [(4, 2, 24, 40, 3), (2, 2, 64, 16, 1), (3, 1, 132, 36, 4), (5, 5, 8, 8, 2)])
def test_delta_prepare_and_conv_roll(dtype, H, G, d, dv, taps):
    """Convolution with its state, SiLU, unit lengths, decays and beta against the plain formulas: a sequence whole, and
    the same sequence in portions of 1, 2 and more tokens (shorter and longer than the convolution reaches back)."""
    n, C = 23, 2 * G * d + H * dv
    proj = rand(n, C + H + 5, seed=1).to(dtype)  # wider than needed: the kernels take a row stride
    low = rand(n, H * (d + dv) + 3, seed=2).float()
    conv_w = rand(C, taps, seed=3, scale=0.5).float()
    a_log, dt_bias = rand(H, seed=4).float(), rand(H * d, seed=5).float()
    x = proj.double()
    act = plain.silu(plain.short_conv(x[:, :C], conv_w.double()))
    want_q = plain.unit(act[:, :G * d].view(n, G, d)) * d**-0.5
    want_k = plain.unit(act[:, G * d:2 * G * d].view(n, G, d))
    want_v = act[:, 2 * G * d:].view(n, H, dv)
    step = torch.nn.functional.softplus(low.double()[:, :H * d] + dt_bias.double()).view(n, H, d)
    want_g = torch.exp(-torch.exp(a_log.double())[None, :, None] * step)
    want_beta = torch.sigmoid(x[:, C:C + H])
    for cuts in ([n], [1, 1, 2, 1, 5, 3, 1, 9]):
        assert sum(cuts) == n
        state = torch.full((4, max(taps - 1, 1), C), float("nan"), device=DEV)
        state[2] = 0.0
        got, at = [], 0
        for c in cuts:
            p, lw = proj[at:at + c].contiguous().to(DEV), low[at:at + c].contiguous().to(DEV)
            pos = i32(list(range(at, at + c)))
            single = c == 1  # a step of one token: the kernel moves the state on itself
            res = F().delta_prepare(p, lw, conv_w.to(DEV), state if taps > 1 else None, a_log.to(DEV), dt_bias.to(DEV), pos,
                                    i32([0] * c), i32([0, c]), i32([2]), H, G, d, dv, taps, roll_single=single)
            if taps > 1 and not single:
                F().conv_roll(p, state, i32([0, c]), i32([2]), 1, C)
            got.append(res)
            at += c
        for j, (want, name) in enumerate([(want_q, "q"), (want_k, "k"), (want_v, "v"), (want_g, "g"), (want_beta, "beta")]):
            have = torch.cat([r[j] for r in got]).double().cpu()
            assert (have - want).abs().max().item() < 3e-6 * (1 + want.abs().max().item()), f"{name} with cuts {cuts}"
        if taps > 1:
            assert (state[2].double().cpu() - x[n - (taps - 1):, :C]).abs().max().item() == 0
            assert torch.isnan(state[[0, 1, 3]]).all()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_head_norm_gate(dtype):
    n, H, dv = 9, 3, 28
    o = rand(n, H, dv, seed=1).float()
    w = rand(dv, seed=2).float()
    gate = rand(n, 50 + H * dv, seed=3).to(dtype)
    want = (plain.rms(o.double(), 1e-5) * w.double() * torch.sigmoid(gate.double()[:, 50:].view(n, H, dv))).view(n, H * dv)
    got = F().head_norm_gate(o.to(DEV), w.to(DEV), gate.to(DEV), 50, 1e-5, dtype).double().cpu()
    assert (got - want).abs().max().item() < (1e-5 if dtype == torch.float32 else 2e-2)


# ------------------------------------------------------------------ routed experts
@pytest.mark.parametrize("E,top,count,keep", [(8, 2, 2, 1), (6, 2, 3, 2), (9, 4, 3, 2), (12, 2, 4, 1), (5, 5, 1, 1), (2, 1, 2, 2), (64, 6, 8, 3), (4, 1, 4, 4)])
def test_route_groups(E, top, count, keep):
    n, width = 200, 72
    h = rand(n, width, seed=1).float()
    w = {"r.router": rand(E, width, seed=2, scale=0.3).float(), "r.correction": rand(E, seed=3, scale=0.4).float()}
    r = {"experts": E, "top": top, "scale": 1.7, "groups": {"count": count, "keep": keep}}
    want_ids, want_w = plain.route(h.double(), w, "r.", r)
    ids, weights = F().route_groups(h.to(DEV), w["r.router"].to(DEV), w["r.correction"].to(DEV), top, count, keep, 1.7)
    assert torch.equal(ids.cpu().long(), want_ids), "other experts were chosen, or in another order"
    assert (weights.double().cpu() - want_w).abs().max().item() < 1e-6


def test_route_groups_the_best_expert_loses_with_its_group():
    """All choice scores are negative: the experts of the kept group must still beat the masked ones (which count as
    minus infinity, not as zero).  Then expert 0 has by far the largest score but a correction sinks its group, the
    other group is kept, and the weights are the scores without the correction."""
    width = 8
    router = torch.zeros(4, width)
    for e in range(4):
        router[e, e] = 1.0
    h = torch.zeros(1, width)
    h[0, :4] = torch.tensor([3.0, -6.0, 0.4, 0.3])
    correction = torch.tensor([-2.0, -2.0, -5.0, -5.0])
    ids, weights = F().route_groups(h.to(DEV), router.to(DEV), correction.to(DEV), 2, 2, 1, 1.0)
    s = torch.sigmoid(h[0, :4])
    want_ids, want_w = plain.route(h.double(), {"r.router": router, "r.correction": correction}, "r.",
                                   {"experts": 4, "top": 2, "scale": 1.0, "groups": {"count": 2, "keep": 1}})
    assert ids.cpu().tolist() == want_ids.tolist() == [[0, 1]]
    correction = torch.tensor([-3.0, -3.0, 0.0, 0.0])
    ids, weights = F().route_groups(h.to(DEV), router.to(DEV), correction.to(DEV), 2, 2, 1, 1.0)
    assert ids.cpu().tolist() == [[2, 3]]
    assert torch.allclose(weights.cpu()[0], s[2:4])  # without the correction


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("width,ff,E,top,n", [(72, 24, 5, 5, 7), (96, 48, 6, 2, 33), (128, 100, 8, 3, 1), (70, 30, 3, 1, 5),
                                              (64, 2048, 9, 8, 2)])  # the last: more than 48 KB of staged activations
def test_experts_pairwise(dtype, width, ff, E, top, n):
    h = rand(n, width, seed=1).to(dtype)
    w = {}
    for e in range(E):
        w[f"m.e{e}.gate"] = rand(ff, width, seed=10 + e, scale=0.2).to(dtype)
        w[f"m.e{e}.up"] = rand(ff, width, seed=30 + e, scale=0.2).to(dtype)
        w[f"m.e{e}.down"] = rand(width, ff, seed=50 + e, scale=0.2).to(dtype)
    gen = torch.Generator().manual_seed(5)
    ids = torch.stack([torch.randperm(E, generator=gen)[:top] for _ in range(n)]).to(torch.int32)
    weights = torch.rand(n, top, generator=gen)
    add = rand(n, width, seed=7).to(dtype)
    want = add.double().clone()
    for t in range(n):
        for kk in range(top):
            e = int(ids[t, kk])
            x = h[t].double()
            y = (plain.silu(w[f"m.e{e}.gate"].double() @ x) * (w[f"m.e{e}.up"].double() @ x))
            if dtype == torch.bfloat16:
                y = y.to(dtype).double()  # the activations between the two products are kept in the run's type
            want[t] += weights[t, kk].double() * (w[f"m.e{e}.down"].double() @ y)
    gate_up = torch.stack([torch.stack([w[f"m.e{e}.gate"], w[f"m.e{e}.up"]]) for e in range(E)]).contiguous().to(DEV)
    down = torch.stack([w[f"m.e{e}.down"] for e in range(E)]).contiguous().to(DEV)
    got = F().experts_pairwise(h.to(DEV), gate_up, down, ids.to(DEV), weights.to(DEV), add.to(DEV))
    assert got.dtype == torch.float32
    assert (got.double().cpu() - want).abs().max().item() < (2e-5 if dtype == torch.float32 else 2e-2) * (1 + want.abs().max().item())
    alone = F().experts_pairwise(h[:1].contiguous().to(DEV), gate_up, down, ids[:1].contiguous().to(DEV), weights[:1].contiguous().to(DEV),
                                 add[:1].contiguous().to(DEV))
    assert torch.equal(alone[0], got[0]), "a token's result depends on the batch"


# ------------------------------------------------------------------ attention: wide norms, sink, window
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n_q,n_kv,d,rot", [(6, 2, 16, 8), (2, 2, 40, 40), (3, 1, 24, 4), (4, 4, 8, 0), (4, 2, 64, 32)])
def test_wide_norm_rope_write(dtype, n_q, n_kv, d, rot):
    from gtar_kimik3_public_b200.parts.rope import RotaryEncoding

    n, past, eps, base = 70, 61, 1e-5, 100.0
    kv, slots, table = scrambled_pages(1, past + n, n_kv, d, dtype, seed=4)
    proj = rand(n, (n_q + n_kv) * d + 11, seed=1).to(dtype)
    w_q, w_k = 1 + 0.2 * rand(n_q * d, seed=2).float(), 1 + 0.2 * rand(n_kv * d, seed=3).float()
    cos = sin = None
    if rot:
        table_ = RotaryEncoding(rot, base, precise=True)
        table_.prepare(past + n, torch.device(DEV))
        cos, sin = table_.cos, table_.sin
    pos = i32(list(range(past, past + n)))
    q = F().wide_norm_rope_write(proj.to(DEV), n_q, n_kv, d, w_q.to(DEV), w_k.to(DEV), eps, cos, sin, rot, pos, i32([0] * n),
                                 slots.to(DEV), kv, past + n - 1)
    x = proj.double()
    qn = (plain.rms(x[:, :n_q * d], eps) * w_q.double()).view(n, n_q, d)
    kn = (plain.rms(x[:, n_q * d:(n_q + n_kv) * d], eps) * w_k.double()).view(n, n_kv, d)
    if rot:
        full_q = torch.zeros(past + n, n_q, d, dtype=torch.float64)
        full_k = torch.zeros(past + n, n_kv, d, dtype=torch.float64)
        full_q[past:], full_k[past:] = qn, kn
        qn, kn = plain.rotate_part(full_q, rot, base)[past:], plain.rotate_part(full_k, rot, base)[past:]
    tol = 2e-5 if dtype == torch.float32 else 3e-2
    assert (q.double().cpu() - qn).abs().max().item() < tol
    for t in (0, 1, 2, 3, n - 1):  # page borders: positions 61 .. 64 straddle one
        p = past + t
        page = int(table[int(slots[0]), p // 64])
        assert (kv.k[page, :, p % 64].double().cpu() - kn[t]).abs().max().item() < tol
        want_v = x[t, n_q * d:(n_q + n_kv) * d].view(n_kv, d)
        assert torch.equal(kv.v[page, :, p % 64].double().cpu(), want_v), "the value must be the key as projected"


def _sink_attention(q, k, v, pos, window, scale):
    """softmax with one more term of score 0 in the denominator; q [n_q, d], k/v [S, n_kv, d]."""
    n_q, n_kv = q.shape[0], k.shape[1]
    lo = max(0, pos - window + 1) if window else 0
    out = []
    for h in range(n_q):
        kh = h // (n_q // n_kv)
        s = (k[lo:pos + 1, kh] @ q[h]) * scale
        e = torch.exp(s - s.max().clamp_min(0))
        out.append(((e / (torch.exp(-s.max().clamp_min(0)) + e.sum()))[:, None] * v[lo:pos + 1, kh]).sum(0))
    return torch.stack(out)


def _attend(kind, q, kv, positions, seqs, slots, lens, scale, window):
    """The three kernels behind one face.  ``q [n, n_q, d]``, one query per listed position."""
    if kind == "exact":
        return F().attention_exact(q, kv, i32(positions), i32(seqs), slots, scale, window, sink=True)
    if kind == "decode":  # one token per sequence
        return F().attention_decode(q, kv, i32(lens), slots, scale, window, n_splits=2, sink=True)
    starts = [0]
    for s in sorted(set(seqs)):
        starts.append(starts[-1] + seqs.count(s))
    return F().attention_prefill(q, kv, i32(starts), i32(lens), slots, max(b - a for a, b in zip(starts, starts[1:])), scale, window,
                                 tensor_cores="tcgen05" if kind == "prefill_tc" else "mma", sink=True)


@pytest.mark.parametrize("kind,dtype,d", [("exact", torch.float32, 24), ("exact", torch.bfloat16, 64), ("prefill", torch.bfloat16, 64),
                                          ("prefill", torch.bfloat16, 128), ("prefill_tc", torch.bfloat16, 128), ("decode", torch.bfloat16, 64),
                                          ("decode", torch.bfloat16, 128)])
def test_attention_with_a_sink_random(kind, dtype, d):
    n_q, n_kv, window, scale = 4, 2, 100, 0.11
    lens = [300, 77]
    kv, slots, table = scrambled_pages(2, 300, n_kv, d, dtype, seed=12)
    ks = [rand(n, n_kv, d, seed=20 + i).to(dtype) for i, n in enumerate(lens)]
    vs = [rand(n, n_kv, d, seed=30 + i).to(dtype) for i, n in enumerate(lens)]
    for i in range(2):
        fill_pages(kv, table, int(slots[i]), ks[i], vs[i])
    new = [1, 1] if kind == "decode" else [220, 77]
    qs = [rand(m, n_q, d, seed=40 + i).to(dtype) for i, m in enumerate(new)]
    positions = [p for i in range(2) for p in range(lens[i] - new[i], lens[i])]
    seqs = [i for i in range(2) for _ in range(new[i])]
    out = _attend(kind, torch.cat(qs).to(DEV), kv, positions, seqs, slots.to(DEV), lens, scale, window).double().cpu()
    assert torch.isfinite(out).all()
    at = 0
    for i in range(2):
        for t in range(new[i]):
            want = _sink_attention(qs[i][t].double(), ks[i].double(), vs[i].double(), lens[i] - new[i] + t, window, scale)
            assert (out[at] - want).abs().max().item() < (2e-5 if dtype == torch.float32 else 2e-2), f"sequence {i} token {t}"
            at += 1


@pytest.mark.parametrize("kind,dtype,d", [("exact", torch.float32, 32), ("prefill", torch.bfloat16, 64), ("decode", torch.bfloat16, 64),
                                          ("prefill", torch.bfloat16, 128), ("prefill_tc", torch.bfloat16, 128), ("decode", torch.bfloat16, 128)])
def test_attention_sink_weight_and_window_edges(kind, dtype, d):
    """One key stands out (score 12.5 against about 0 elsewhere): at the window's last place inside it carries the
    output; a key just outside with a far larger score must not be seen; where every score is strongly negative the
    sink takes nearly all the weight and the output is nearly zero; the same at the first tokens, at page borders, and
    with a key hundreds back when there is no window."""
    n_q, n_kv, n, scale = 2, 1, 400, 0.5
    for window, pos in ((100, 399), (64, 127), (65, 128), (1, 70), (0, 399), (100, 5)):
        kv, slots, table = scrambled_pages(1, n, n_kv, d, dtype, seed=13)
        k = rand(n, n_kv, d, seed=1, scale=0.02)
        v = rand(n, n_kv, d, seed=2)
        q = torch.zeros(1, n_q, d, dtype=torch.float64)
        q[0, :, 0] = 5.0
        inside = max(0, pos - window + 1) if window else 3
        k[inside, 0, 0] = 5.0
        if window and pos - window >= 0:
            k[pos - window, 0, 0] = 40.0  # would take everything if it were visible
        fill_pages(kv, table, int(slots[0]), k.to(dtype), v.to(dtype))
        out = _attend(kind, q.to(dtype).to(DEV), kv, [pos], [0], slots.to(DEV), [pos + 1], scale, window).double().cpu()
        want = _sink_attention(q[0].to(dtype).double(), k.to(dtype).double(), v.to(dtype).double(), pos, window, scale)
        tol = 2e-5 if dtype == torch.float32 else 2e-2
        assert (out[0] - want).abs().max().item() < tol, f"window {window}, position {pos}"
        assert (out[0, 0] - v[inside, 0].to(dtype).double()).abs().max().item() < 0.05, f"window {window}: the key at its edge was not found"
        out = _attend(kind, (-q).to(dtype).to(DEV), kv, [pos], [0], slots.to(DEV), [pos + 1], scale, window).double().cpu()
        want = _sink_attention(-q[0].to(dtype).double(), k.to(dtype).double(), v.to(dtype).double(), pos, window, scale)
        assert (out[0] - want).abs().max().item() < tol
