"""Each mechanism of the Dasusun layers alone, the library's kernel against the plain implementation's function:
the merging of a branch into the stream (norm after the branch, layer scale, depth mix, next norm), the causal
convolution with its state, GELU, the stretched rotation's tables, the preparation of the latents, and attention over
latent rows with inputs made so that ONE key decides the result: far back, at page borders, the last key inside a
window and the first outside it, in prompts and in single-token steps."""

import math

import pytest
import torch

from tests.plain import dasusun as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _f():
    from gtar_kimik3_public_b200.ops import functional as F

    return F


@pytest.mark.parametrize("width,rows", [(96, 5), (97, 4), (1000, 3), (4096, 2)])  # 97: the one-element kernel
@pytest.mark.parametrize("y_dtype", [torch.float32, torch.bfloat16])
def test_branch_merge(width, rows, y_dtype):
    F = _f()
    gen = torch.Generator().manual_seed(width)
    x = torch.randn(rows, width, generator=gen) * 3
    y = (torch.randn(rows, width, generator=gen) * 0.5).to(y_dtype)
    w_y, scale, w_z = (torch.randn(width, generator=gen) * 0.3 for _ in range(3))
    kept = torch.randn(4, rows, width, generator=gen)
    mix = torch.randn(3, generator=gen)
    eps_y, eps_z = 1e-5, 1e-3
    v = x.double() + scale.double() * plain.norm_around_zero(y.double(), w_y.double(), eps_y)
    want_kept = v.clone()
    v = mix[0].double() * kept[0].double() + mix[1].double() * kept[1].double() + mix[2].double() * v
    want_z = plain.norm_around_zero(v, w_z.double(), eps_z)
    kept_d = kept.to(DEV)
    out = torch.empty(rows, width, device=DEV)
    stream, z = F.branch_merge(x.to(DEV), y.to(DEV), (1 + w_y).to(DEV), eps_y, scale.to(DEV), kept=kept_d, n_kept=2,
                               mix=mix.to(DEV), next_weight=(1 + w_z).to(DEV), next_eps=eps_z, next_dtype=torch.float32, x_out=out)
    assert torch.allclose(kept_d[2].double().cpu(), want_kept, atol=2e-5, rtol=1e-5)
    assert torch.equal(kept_d[3].cpu(), kept[3])  # entries after the layer's own are untouched
    assert torch.allclose(stream.double().cpu(), v, atol=5e-5, rtol=1e-5)
    assert torch.allclose(z.double().cpu(), want_z, atol=5e-5, rtol=1e-5)
    # without history, without next norm, in place
    xd = x.to(DEV)
    stream, z = F.branch_merge(xd, y.to(DEV), (1 + w_y).to(DEV), eps_y, None)
    assert z is None and stream.data_ptr() == xd.data_ptr()
    want = x.double() + plain.norm_around_zero(y.double(), w_y.double(), eps_y)
    assert torch.allclose(xd.double().cpu(), want, atol=2e-5, rtol=1e-5)


@pytest.mark.parametrize("taps", [1, 2, 3, 5])
@pytest.mark.parametrize("width", [40, 41])  # four channels a thread, and the one-channel kernel
def test_causal_convolution_with_state_under_every_cut(taps, width):
    """Three sequences of unequal lengths fed in portions (also shorter than the taps) give what each gives whole."""
    F = _f()
    n_slots = 6
    gen = torch.Generator().manual_seed(taps)
    w = torch.randn(width, taps, generator=gen)
    lengths = [11, 1, 7]
    slots = [4, 0, 5]
    inputs = [torch.randn(n, width, generator=gen) for n in lengths]
    want = [a.double() + plain.causal_conv(a.double(), w.double()) for a in inputs]
    state = torch.full((n_slots, max(taps - 1, 1), width), float("nan"), device=DEV)[:, :taps - 1].contiguous()
    for s in slots:
        state[s].zero_()  # what the cache does when it hands a slot out
    got = [[] for _ in lengths]
    done = [0, 0, 0]
    for portion in ([3, 1, 2], [1, 0, 1], [1, 0, 0], [1, 0, 4], [5, 0, 0]):
        live = [i for i in range(3) if portion[i]]
        rows = torch.cat([inputs[i][done[i]:done[i] + portion[i]] for i in live]).to(DEV)
        q = [portion[i] for i in live]
        cu = torch.tensor([0] + list(torch.tensor(q).cumsum(0)), dtype=torch.int32, device=DEV)
        tok_seq = torch.repeat_interleave(torch.arange(len(live)), torch.tensor(q)).int().to(DEV)
        tok_pos = torch.cat([torch.arange(done[i], done[i] + portion[i]) for i in live]).int().to(DEV)
        slot_t = torch.tensor([slots[i] for i in live], dtype=torch.int32, device=DEV)
        single = all(n == 1 for n in q)  # one token each: the convolution's kernel moves the states on itself
        out = F.causal_conv(rows, w.t().contiguous().to(DEV), state if taps > 1 else None, tok_pos, tok_seq, cu, slot_t, torch.float32,
                            update_single_token_state=single and taps > 1)
        if taps > 1 and not single:
            F.conv_state(rows, state, cu, slot_t, len(live))
        at = 0
        for i in live:
            got[i].append(out[at:at + portion[i]].cpu())
            at += portion[i]
            done[i] += portion[i]
    for i in range(3):
        assert torch.allclose(torch.cat(got[i]).double(), want[i], atol=1e-5), f"sequence {i}"
    if taps > 1:
        assert torch.isnan(state[1]).all()  # slots of other sequences are not touched


def test_gelu():
    F = _f()
    z = torch.linspace(-8, 8, 4001)
    assert torch.allclose(F.gelu_tanh(z.to(DEV)).cpu().double(), plain.gelu_tanh(z.double()), atol=1e-6)
    got = F.gelu_tanh(z.bfloat16().to(DEV)).cpu().double()
    assert torch.allclose(got, plain.gelu_tanh(z.bfloat16().double()), atol=0.04, rtol=0.01)


@pytest.mark.parametrize("tokens", [1, 5, 16])
def test_gelu_in_the_few_token_product(tokens):
    """Few tokens: GELU is the product's output stage; the result is GELU of the 32-bit sums, rounded once."""
    from gtar_kimik3_public_b200.ops.linear import linear

    gen = torch.Generator().manual_seed(tokens)
    x = torch.randn(tokens, 256, generator=gen).bfloat16()
    w = (torch.randn(200, 256, generator=gen) * 0.2).bfloat16()
    got = linear(x.to(DEV), w.to(DEV), gelu=True).cpu().double()
    want = plain.gelu_tanh(x.double() @ w.double().T)
    assert got.shape == (tokens, 200)
    assert torch.allclose(got, want, atol=0.03, rtol=0.01)
    assert not torch.allclose(got, x.double() @ w.double().T, atol=0.03, rtol=0.01)  # the activation was applied


@pytest.mark.parametrize("dims,base,scaling", [
    (16, 200000.0, {"factor": 3.0, "original": 1024, "fast": 20.0, "slow": 1.5}),
    (8, 10000.0, {"factor": 4.0, "original": 64, "fast": 16.0, "slow": 2.0}),
    (24, 100.0, {"factor": 1.5, "original": 256, "fast": 24.0, "slow": 0.5}),
    (8, 500.0, None),
])
def test_rotation_tables(dims, base, scaling):
    from gtar_kimik3_public_b200.parts.base import build_part

    if scaling:
        part = build_part("position", "rope_scaled", dim=dims, base=base, **scaling)
    else:
        part = build_part("position", "rope", dim=dims, base=base)
    part.prepare(300, torch.device(DEV))
    f, mag = plain.rotary_frequencies(dims, base, scaling)
    angle = torch.arange(301, dtype=torch.float64)[:, None] * f[None, :]
    assert torch.allclose(part.cos[:301].cpu().double(), angle.cos() * mag, atol=2e-4)
    assert torch.allclose(part.sin[:301].cpu().double(), angle.sin() * mag, atol=2e-4)
    if scaling:
        assert not torch.allclose(f, plain.rotary_frequencies(dims, base, None)[0])  # the stretching does something


def _rows_cache(n_pages, width, dtype, table):
    F = _f()
    rows = torch.full((n_pages, 64, width), float("nan"), dtype=dtype, device=DEV)
    return F.PagedRows(rows, torch.tensor(table, dtype=torch.int32, device=DEV))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_latent_prepare(dtype):
    F = _f()
    q_rank, rank, rot, rot_dims, n = 24, 40, 12, 8, 5
    gen = torch.Generator().manual_seed(1)
    proj = torch.randn(n, q_rank + rank + rot, generator=gen).to(dtype)
    w_q, w_kv = torch.rand(q_rank, generator=gen) + 0.5, torch.rand(rank, generator=gen) + 0.5
    positions = torch.tensor([62, 63, 64, 65, 3])
    seqs = torch.tensor([0, 0, 0, 0, 1], dtype=torch.int32)
    cache = _rows_cache(6, rank + rot, dtype, [[5, 2, 0, 0], [0, 0, 0, 0], [4, 1, 0, 0]])
    slots = torch.tensor([0, 2], dtype=torch.int32, device=DEV)
    f, mag = plain.rotary_frequencies(rot_dims, 1000.0, None)
    angle = torch.arange(128, dtype=torch.float64)[:, None] * f[None, :]
    cos, sin = (angle.cos() * mag).float().to(DEV), (angle.sin() * mag).float().to(DEV)
    c_q = F.latent_prepare(proj.to(DEV), q_rank, rank, rot, rot_dims, w_q.to(DEV), w_kv.to(DEV), 1e-5, cos, sin,
                           positions.int().to(DEV), seqs.to(DEV), slots, cache, 65)
    wide = proj.double()
    tol = dict(atol=1e-5, rtol=1e-5) if dtype == torch.float32 else dict(atol=0.03, rtol=0.01)
    assert torch.allclose(c_q.double().cpu(), plain.norm_plain(wide[:, :q_rank], w_q.double(), 1e-5), **tol)
    want_c = plain.norm_plain(wide[:, q_rank:q_rank + rank], w_kv.double(), 1e-5)
    want_k = plain.rotate(wide[:, q_rank + rank:], positions, rot_dims, 1000.0, None)
    where = [(5, 62), (5, 63), (2, 0), (2, 1), (4, 3)]  # page and place of the five positions
    for t, (page, place) in enumerate(where):
        row = cache.rows[page, place].double().cpu()
        assert torch.allclose(row[:rank], want_c[t], **tol)
        assert torch.allclose(row[rank:], want_k[t], **tol)
    assert torch.isnan(cache.rows[5, 61]).all() and torch.isnan(cache.rows[2, 2]).all()  # nothing else is written


def _attend_plain(q_full, rows, pos, window, scale, rank):
    """One query over rows 0..pos of its sequence: softmax over the visible ones, value = the row's first entries."""
    lo = max(0, pos - window + 1) if window else 0
    keys = rows[lo:pos + 1]
    p = torch.softmax((keys @ q_full) * scale, dim=0)
    return p @ keys[:, :rank]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("window", [0, 1, 37, 64, 65, 200])
@pytest.mark.parametrize("heads,rank,rot", [(3, 48, 8), (5, 64, 16), (20, 128, 32)])
def test_latent_attention_one_key_decides(dtype, window, heads, rank, rot):
    """Every cached row points its own way; each query is made to point at ONE chosen key, with a score far above
    the others, so that the output is that key's latent if the key is visible and something else if it is not.
    Targets: the query's own position, the key before it, the last key inside the window, the first outside, keys at
    page borders, the sequence's first tokens and a key hundreds of positions back.  Once as a prompt's step and
    once token by token (the cache already holding all rows)."""
    from gtar_kimik3_public_b200.ops import attention as attention_ops
    from gtar_kimik3_public_b200.parts.base import StepContext

    F = _f()
    rot_dims, dn = 8, 16  # the sizes with a latent of 64 or 128 go through the tensor-core kernel in bfloat16
    length, slot, scale = 300, 1, 0.25
    gen = torch.Generator().manual_seed(window)
    rows = torch.randn(length, rank + rot, generator=gen)
    rows = (rows / rows.norm(dim=-1, keepdim=True)).to(dtype).float()  # unit rows, as the cache holds them
    pages = [7, 3, 9, 0, 5]
    cache = _rows_cache(10, rank + rot, dtype, [[0] * 5, pages])
    for i, page in enumerate(pages):
        part = rows[i * 64:(i + 1) * 64]
        cache.rows[page, :part.shape[0]] = part.to(dtype).to(DEV)
    f, mag = plain.rotary_frequencies(rot_dims, 10000.0, None)
    angle = torch.arange(length, dtype=torch.float64)[:, None] * f[None, :]
    cos, sin = angle.cos().float().to(DEV), angle.sin().float().to(DEV)

    queries = []  # (position, target key)
    for pos in (0, 1, 36, 37, 63, 64, 65, 127, 128, 199, 200, 255, 256, 299):
        targets = {pos, max(pos - 1, 0), 0, 1, 63 if pos >= 63 else 0, 64 if pos >= 64 else 0, max(pos - 250, 0)}
        if window:
            targets |= {max(pos - window + 1, 0), max(pos - window, 0)}
        queries += [(pos, j) for j in sorted(targets) if j <= pos]
    # the query: 80 times the target row in the carried part; its own rotated part is made so that, once rotated to
    # its position, it is 80 times the target's (already rotated) key part
    carried = torch.zeros(len(queries), heads, rank)
    raw = torch.zeros(len(queries), heads, dn + rot)
    for n, (pos, j) in enumerate(queries):
        for h in range(heads):
            gain = 80.0 + 8 * h
            carried[n, h] = gain * rows[j, :rank]
            turned_back = plain.rotate(rows[j, rank:].double()[None], torch.tensor([-pos]), rot_dims, 10000.0, None)[0]
            raw[n, h, dn:] = (gain * turned_back).float()
    carried, raw = carried.to(dtype), raw.to(dtype)
    want = torch.zeros(len(queries), heads, rank, dtype=torch.float64)
    for n, (pos, j) in enumerate(queries):
        for h in range(heads):
            own = plain.rotate(raw[n, h, dn:].double()[None], torch.tensor([pos]), rot_dims, 10000.0, None)[0]
            q_full = torch.cat([carried[n, h].double(), own])
            want[n, h] = _attend_plain(q_full, rows.double(), pos, window, scale, rank)
        visible = pos - j < window if window else True
        hit = torch.allclose(want[n, 0], rows[j, :rank].double(), atol=0.05)
        assert hit == visible, f"the test's own inputs do not single out key {j} for position {pos}"

    def run(indices):
        n = len(indices)
        pos = torch.tensor([queries[i][0] for i in indices], dtype=torch.int32, device=DEV)
        ctx = StepContext(
            n_tokens=n, n_seqs=1, dtype=dtype, tokens=pos, tok_pos=pos, tok_seq=torch.zeros(n, dtype=torch.int32, device=DEV),
            cu_q=torch.tensor([0, n], dtype=torch.int32, device=DEV), slots=torch.tensor([slot], dtype=torch.int32, device=DEV),
            kv_len=torch.tensor([length], dtype=torch.int32, device=DEV), want_rows=pos[:0], max_q_len=n, max_kv_len=length,
            max_position=length - 1, all_single=n == 1)
        out = torch.empty(n, heads, rank, dtype=dtype, device=DEV)
        idx = torch.tensor(indices)
        attention_ops.latent_attention(carried[idx].to(DEV), raw[idx].to(DEV).contiguous(), dn, rot, rot_dims, cos, sin, cache, ctx,
                                       scale, window, out)
        return out.double().cpu()

    tol = dict(atol=2e-5) if dtype == torch.float32 else dict(atol=0.02)
    together = run(list(range(len(queries))))
    assert torch.allclose(together, want, **tol)
    for n in range(0, len(queries), 7):  # a sample of them as single-token steps
        assert torch.allclose(run([n])[0], want[n], **tol), f"position {queries[n][0]} target {queries[n][1]} alone"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("tokens", [1, 7, 16, 40])
@pytest.mark.parametrize("heads,n,k,pad", [(3, 40, 24, 8), (5, 17, 13, 3), (16, 64, 128, 32)])
def test_per_head_products_on_strided_views(dtype, tokens, heads, n, k, pad):
    """One product per head on operands that lie side by side in a token's row, written into a strided view: few tokens take
    the small-product kernel, many the batched product, float32 the FP32-pipe kernel; all against the plain sum."""
    F = _f()
    gen = torch.Generator().manual_seed(tokens * 100 + heads)
    rows = torch.randn(tokens, heads, k + pad, generator=gen).to(dtype)       # a head's operand is the first k of its part
    w = (torch.randn(heads, n, k, generator=gen) * 0.3).to(dtype)
    out = torch.full((tokens, heads * n), float("nan"), dtype=dtype, device=DEV)
    F.linear_batched(rows.to(DEV)[:, :, :k].transpose(0, 1), w.to(DEV), out.view(tokens, heads, n).transpose(0, 1))
    want = torch.einsum("thk,hnk->thn", rows[:, :, :k].double(), w.double()).reshape(tokens, heads * n)
    tol = dict(atol=1e-4, rtol=1e-5) if dtype == torch.float32 else dict(atol=0.05, rtol=0.01)
    assert torch.allclose(out.double().cpu(), want, **tol)
