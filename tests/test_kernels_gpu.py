"""Each CUDA kernel alone against its plain statement (tests/kernel_refs.py), at sizes other
than the engine's: widths that are no power of two, odd head counts, ragged batches."""
import math

import pytest
import torch

import kernel_refs as ref

pytestmark = pytest.mark.gpu
DEV = "cuda"
TOL = {torch.float32: 2e-5, torch.bfloat16: 1.2e-2}     # relative to the largest reference value


def ops():
    from neurogrid_b200.csrc import ops as o
    return o


def close(got, want, dtype, scale=1.0):
    err = float((got.double() - want.double()).abs().max() / want.double().abs().max().clamp_min(1e-30))
    assert err < TOL[dtype] * scale, f"relative error {err:.3e}"


def rnd(*shape, dtype=torch.float32, seed=0, std=1.0):
    g = torch.Generator(device="cpu").manual_seed(seed)
    return (torch.randn(*shape, generator=g) * std).to(dtype).to(DEV)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,V,N", [(80, 301, 7), (2048, 1000, 33)])
def test_embed(dtype, H, V, N):
    table = rnd(V, H, dtype=dtype)
    tok = torch.randint(0, V, (N,), dtype=torch.int32, device=DEV)
    out, out_r = torch.empty(N, H, device=DEV), torch.empty(N, H, device=DEV)
    st, st_r = torch.zeros(1, dtype=torch.int32, device=DEV), torch.zeros(1, dtype=torch.int32, device=DEV)
    ops().embed(table, tok, out, st)
    ref.embed(table, tok, out_r, st_r)
    assert torch.equal(out, out_r) and int(st) == 0
    tok[2] = V + 5                                   # outside the table: zeros and a status bit, no fault
    ops().embed(table, tok, out, st)
    assert int(st) == 1 and float(out[2].abs().max()) == 0.0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,N", [(80, 5), (1000, 19), (2048, 64), (6000, 3)])
def test_add_rmsnorm(dtype, H, N):
    h = rnd(N, H, seed=1)
    delta = rnd(N, H, dtype=dtype, seed=2)
    w = 1 + 0.1 * rnd(H, seed=3)
    for d in (delta, None):
        h1, h2 = h.clone(), h.clone()
        o1, o2 = torch.empty(N, H, dtype=dtype, device=DEV), torch.empty(N, H, dtype=dtype, device=DEV)
        ops().add_rmsnorm(h1, d, w, o1, 1e-5)
        ref.add_rmsnorm(h2, d, w, o2, 1e-5)
        close(o1, o2, dtype)
        close(h1, h2, torch.float32)
    rows = torch.tensor([N - 1, 0, N // 2], dtype=torch.int32, device=DEV)
    h1, h2 = h.clone(), h.clone()
    o1, o2 = torch.empty(3, H, dtype=dtype, device=DEV), torch.empty(3, H, dtype=dtype, device=DEV)
    ops().add_rmsnorm(h1, delta, w, o1, 1e-6, rows)
    ref.add_rmsnorm(h2, delta, w, o2, 1e-6, rows)
    close(o1, o2, dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("I,N", [(200, 3), (4608, 17)])
def test_swiglu(dtype, I, N):
    gu = rnd(N, 2 * I, dtype=dtype, std=2.0)
    o1, o2 = torch.empty(N, I, dtype=dtype, device=DEV), torch.empty(N, I, dtype=dtype, device=DEV)
    ops().swiglu(gu, o1)
    ref.swiglu(gu, o2)
    close(o1, o2, dtype)


@pytest.mark.parametrize("M,N,K", [(1, 301, 80), (7, 64, 96), (130, 200, 333), (65, 129, 17)])
def test_gemm_f32(M, N, K):
    a, w, b = rnd(M, K, seed=1), rnd(N, K, seed=2), rnd(N, seed=3)
    for bias in (None, b):
        o1, o2 = torch.empty(M, N, device=DEV), torch.empty(M, N, device=DEV)
        ops().gemm_f32(a, w, bias, o1)
        ref.gemm_f32(a, w, bias, o2)
        close(o1, o2, torch.float32)
    # a row's result does not depend on the rest of the batch
    o3 = torch.empty(1, N, device=DEV)
    ops().gemm_f32(a[M // 2:M // 2 + 1].contiguous(), w, None, o3)
    o4 = torch.empty(M, N, device=DEV)
    ops().gemm_f32(a, w, None, o4)
    assert torch.equal(o3[0], o4[M // 2])


def _ragged(q_lens, ctx):
    cu = [0]
    for q in q_lens:
        cu.append(cu[-1] + q)
    t = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
    return t(cu), t(ctx), cu[-1]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("L,H,bias", [(2, 80, True), (3, 2048, False), (4, 96, True), (8, 200, False)])
def test_shortconv(dtype, L, H, bias):
    q_lens = [1, 70, 2, 33, 1, 3]
    ctx = [5, 0, 1, 40, 0, 2]
    cu, cb, N = _ragged(q_lens, ctx)
    slots = torch.tensor([3, 0, 5, 1, 6, 2], dtype=torch.int32, device=DEV)
    p = rnd(N, 3 * H, dtype=dtype, seed=4)
    w = rnd(H, L, seed=5, std=0.3)
    b = rnd(H, seed=6, std=0.1) if bias else None
    st1 = rnd(8, L - 1, H, seed=7)                      # stale content: must be masked where position < 0
    st2 = st1.clone()
    o1, o2 = torch.zeros(N, H, dtype=dtype, device=DEV), torch.zeros(N, H, dtype=dtype, device=DEV)
    ops().shortconv(p, w, b, st1, o1, cu, cb, slots, len(q_lens), max(q_lens))
    ref.shortconv(p, w, b, st2, o2, cu, cb, slots, len(q_lens), max(q_lens))
    close(o1, o2, dtype)
    close(st1, st2, torch.float32)
    assert torch.equal(st1[4], st2[4]) and torch.equal(st1[7], st2[7])    # untouched slots stay


@pytest.mark.parametrize("L,H,bias", [(3, 2048, False), (2, 200, True), (4, 96, True), (5, 264, False)])
def test_shortconv_long_portions(L, H, bias):
    """Long bfloat16 portions take the kernel with 16-byte accesses: tiles of 8 tokens, portions
    that are shorter than the conv, longer than a tile, and that continue a sequence."""
    dtype = torch.bfloat16
    q_lens = [300, 1, 70, 2, 67, 9, 3]
    ctx = [0, 5, 1, 0, 40, 2, 1]
    cu, cb, N = _ragged(q_lens, ctx)
    slots = torch.tensor([3, 0, 5, 1, 6, 2, 7], dtype=torch.int32, device=DEV)
    p = rnd(N, 3 * H, dtype=dtype, seed=14)
    w = rnd(H, L, seed=15, std=0.3)
    b = rnd(H, seed=16, std=0.1) if bias else None
    st1 = rnd(9, L - 1, H, seed=17)
    st2 = st1.clone()
    o1, o2 = torch.zeros(N, H, dtype=dtype, device=DEV), torch.zeros(N, H, dtype=dtype, device=DEV)
    ops().shortconv(p, w, b, st1, o1, cu, cb, slots, len(q_lens), max(q_lens))
    ref.shortconv(p, w, b, st2, o2, cu, cb, slots, len(q_lens), max(q_lens))
    close(o1, o2, dtype)
    close(st1, st2, torch.float32)
    assert torch.equal(st1[4], st2[4]) and torch.equal(st1[8], st2[8])


def _paged_setup(dtype, n_kv, hd, ps, q_lens, ctx, seed=0, num_pages=64):
    """Random pages, block tables with shuffled page ids, positions and row->entry maps."""
    g = torch.Generator().manual_seed(seed)
    R = len(q_lens)
    stride = max(-(-(c + q) // ps) for c, q in zip(ctx, q_lens)) + 1
    perm = torch.randperm(num_pages, generator=g).tolist()
    table = torch.full((R, stride), -1, dtype=torch.int32)
    for e in range(R):
        for j in range(-(-(ctx[e] + q_lens[e]) // ps)):
            table[e, j] = perm.pop()
    pos, re = [], []
    for e in range(R):
        pos += list(range(ctx[e], ctx[e] + q_lens[e]))
        re += [e] * q_lens[e]
    k = rnd(num_pages, n_kv, ps, hd, dtype=dtype, seed=seed + 1)
    v = rnd(num_pages, n_kv, ps, hd, dtype=dtype, seed=seed + 2)
    t = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
    return k, v, table.to(DEV), t(pos), t(re)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nH,nKV,hd,ps,half,norm", [(4, 2, 16, 16, False, True), (3, 1, 32, 8, True, True),
                                                     (6, 3, 48, 32, False, False), (5, 5, 256, 16, True, True),
                                                     (8, 2, 80, 4, False, True)])
def test_rope_cache(dtype, nH, nKV, hd, ps, half, norm):
    q_lens, ctx = [3, 1, 20, 1], [0, 37, 5, 200]
    k1, v1, table, pos, re = _paged_setup(dtype, nKV, hd, ps, q_lens, ctx, num_pages=128)
    re[1] = -1                                                  # a padding row
    k2, v2 = k1.clone(), v1.clone()
    N = sum(q_lens)
    qkv = rnd(N, (nH + 2 * nKV) * hd, dtype=dtype, seed=9)
    qw = (1 + 0.1 * rnd(hd, seed=10)) if norm else None
    kw = (1 + 0.1 * rnd(hd, seed=11)) if norm else None
    inv = (10000.0 ** (-2.0 * torch.arange(hd // 2, dtype=torch.float64) / hd)).float().to(DEV)
    st = torch.zeros(1, dtype=torch.int32, device=DEV)
    for inv_freq in (inv, None):
        q1 = torch.empty(N, nH * hd, dtype=dtype, device=DEV)
        q2 = torch.empty_like(q1)
        ops().rope_cache(qkv, q1, qw, kw, inv_freq, half, 1.0, k1, v1, table, pos, re, nH, nKV, hd, 1e-5, st)
        ref.rope_cache(qkv, q2, qw, kw, inv_freq, half, 1.0, k2, v2, table, pos, re, nH, nKV, hd, 1e-5, st)
        close(q1, q2, dtype)
        close(k1, k2, dtype)
        assert torch.equal(v1, v2)
    assert int(st) == 0
    # a layer that only reads another layer's cache: q alone, no pages
    qonly = qkv[:, : nH * hd].contiguous()
    q1, q2 = torch.empty(N, nH * hd, dtype=dtype, device=DEV), torch.empty(N, nH * hd, dtype=dtype, device=DEV)
    ops().rope_cache(qonly, q1, qw, None, inv, half, 2.0, None, None, table, pos, re, nH, 0, hd, 1e-5, st)
    ref.rope_cache(qonly, q2, qw, None, inv, half, 2.0, None, None, table, pos, re, nH, 0, hd, 1e-5, st)
    close(q1, q2, dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nH,nKV,hd,ps,half", [(32, 8, 64, 16, False), (32, 8, 64, 16, True), (5, 2, 64, 8, True),
                                               (3, 3, 64, 32, True), (5, 5, 48, 8, True), (6, 3, 80, 32, False),
                                               (3, 1, 256, 16, False)])
def test_rope_cache_many_rows(dtype, nH, nKV, hd, ps, half):
    """Many rows: several heads per warp and pass, two-element accesses for adjacent pairs."""
    q_lens, ctx = [290, 1, 40, 1], [3, 37, 0, 200]
    k1, v1, table, pos, re = _paged_setup(dtype, nKV, hd, ps, q_lens, ctx, num_pages=128, seed=5)
    re[290] = -1
    k2, v2 = k1.clone(), v1.clone()
    N = sum(q_lens)
    qkv = rnd(N, (nH + 2 * nKV) * hd, dtype=dtype, seed=19)
    qw, kw = 1 + 0.1 * rnd(hd, seed=20), 1 + 0.1 * rnd(hd, seed=21)
    inv = (10000.0 ** (-2.0 * torch.arange(hd // 2, dtype=torch.float64) / hd)).float().to(DEV)
    st = torch.zeros(1, dtype=torch.int32, device=DEV)
    q1 = torch.empty(N, nH * hd, dtype=dtype, device=DEV)
    q2 = torch.empty_like(q1)
    ops().rope_cache(qkv, q1, qw, kw, inv, half, 1.0, k1, v1, table, pos, re, nH, nKV, hd, 1e-6, st)
    ref.rope_cache(qkv, q2, qw, kw, inv, half, 1.0, k2, v2, table, pos, re, nH, nKV, hd, 1e-6, st)
    close(q1, q2, dtype)
    close(k1, k2, dtype)
    assert torch.equal(v1, v2) and int(st) == 0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nH,nKV,hd,ps,window", [(4, 2, 16, 16, None), (3, 1, 32, 8, None), (6, 3, 48, 32, 20),
                                                  (5, 5, 256, 16, None), (8, 2, 80, 4, 7)])
def test_attention_generic(dtype, nH, nKV, hd, ps, window):
    q_lens, ctx = [3, 1, 40, 1, 2], [0, 37, 5, 300, 63]
    k, v, table, pos, re = _paged_setup(dtype, nKV, hd, ps, q_lens, ctx, num_pages=128)
    N = sum(q_lens)
    q = rnd(N, nH * hd, dtype=dtype, seed=12)
    o1, o2 = torch.empty_like(q), torch.empty_like(q)
    ops().attention_generic(q, k, v, table, pos, re, o1, nH, window, 1 / math.sqrt(hd))
    ref.attention_generic(q, k, v, table, pos, re, o2, nH, window, 1 / math.sqrt(hd))
    close(o1, o2, dtype)


def test_attention_finds_a_far_key():
    """One key among hundreds, on another page, carries a score that stands out: the output
    must be its value row.  Random pages elsewhere would hide a wrong page or a wrong slot."""
    nH, nKV, hd, ps = 4, 2, 32, 16
    ctx, far = 611, 77
    k, v, table, pos, re = _paged_setup(torch.float32, nKV, hd, ps, [1], [ctx], num_pages=64, seed=3)
    q = rnd(1, nH * hd, seed=13)
    page, slot = int(table[0, far // ps]), far % ps
    for h in range(nKV):
        k[page, h, slot] = 50.0 * q[0].view(nH, hd)[h * 2]       # aligned with the first head of each group
    out = torch.empty_like(q)
    ops().attention_generic(q, k, v, table, pos, re, out, nH, None, 1 / math.sqrt(hd))
    for h in (0, 2):
        assert torch.allclose(out.view(nH, hd)[h], v[page, h // 2, slot], atol=1e-4)


@pytest.mark.parametrize("V", [301, 65536])
def test_sampling(V):
    W = 6
    logits = rnd(W, V, seed=20, std=3.0)
    logits[1, 17] = logits[1, 200] = logits[1].max() + 1          # a tie: the first index wins
    out = torch.empty(W, dtype=torch.int32, device=DEV)
    ops().sample(logits, None, None, None, out, None)
    assert out.tolist() == torch.argmax(logits, -1).tolist() and out[1] == 17
    temp = torch.tensor([0.0, 0.8, 1.0, 0.3, 1.5, 0.7], device=DEV)
    top_p = torch.tensor([1.0, 1.0, 0.9, 0.5, 1.0, 0.05], device=DEV)
    scratch = torch.empty(W, V, device=DEV)
    for seed in range(8):
        u = torch.rand(W, generator=torch.Generator().manual_seed(seed)).to(DEV)
        ops().sample(logits, temp, top_p, u, out, scratch)
        assert int(out[0]) == int(torch.argmax(logits[0]))
        for r in range(1, W):
            # the draw must fall where the float64 CDF of the kept set puts u, up to float32 rounding
            lg = logits[r].double()
            e = torch.exp((lg - lg.max()) / float(temp[r]))
            p = float(top_p[r])
            if p < 1:
                vals = torch.sort(e, descending=True).values
                cs = torch.cumsum(vals, 0)
                cut = int(torch.nonzero(cs >= p * e.sum())[0])
                kept = e >= vals[cut] * (1 - 1e-6)
                assert bool(kept[int(out[r])])
                e = torch.where(e >= vals[cut], e, torch.zeros_like(e))
            c = torch.cumsum(e, 0) / e.sum()
            i = int(out[r])
            lo = float(c[i - 1]) if i > 0 else 0.0
            assert lo - 1e-4 <= float(u[r]) <= float(c[i]) + 1e-4, (r, i, float(u[r]), lo, float(c[i]))


def _cu(q_lens, ctx):
    cu = [0]
    for n in q_lens:
        cu.append(cu[-1] + n)
    t = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
    return t(cu), t(ctx)


@pytest.mark.parametrize("nH,nKV,hd,ps,window", [(4, 2, 16, 16, None), (3, 1, 32, 8, None), (6, 3, 48, 32, 20),
                                                  (32, 8, 64, 16, None), (8, 2, 80, 4, 70), (4, 1, 128, 16, None),
                                                  (2, 2, 256, 16, None), (16, 1, 64, 64, None)])
def test_attn_prefill_bf16(nH, nKV, hd, ps, window):
    """Portions that start at a page edge, inside a page, at position 0; longer than one
    64-row block; a single-token entry that the kernel handles or leaves alone."""
    q_lens, ctx = [3, 1, 150, 64, 2, 65], [0, 37, 5, 64, 63, 131]
    k, v, table, pos, re = _paged_setup(torch.bfloat16, nKV, hd, ps, q_lens, ctx, num_pages=512 // min(ps, 16) + 64)
    cu, cb = _cu(q_lens, ctx)
    q = rnd(sum(q_lens), nH * hd, dtype=torch.bfloat16, seed=12)
    want = torch.empty_like(q)
    ref.attention_generic(q, k, v, table, pos, re, want, nH, window, 1 / math.sqrt(hd))
    got = torch.zeros_like(q)
    ops().attn_prefill_bf16(q, k, v, table, cu, cb, got, len(q_lens), max(q_lens), nH, window, 1 / math.sqrt(hd), False)
    close(got, want, torch.bfloat16)
    got2 = torch.full_like(q, 7.0)
    ops().attn_prefill_bf16(q, k, v, table, cu, cb, got2, len(q_lens), max(q_lens), nH, window, 1 / math.sqrt(hd), True)
    assert float((got2[3] - 7.0).abs().max()) == 0.0             # row 3 is the single-token entry: untouched
    keep = [i for i in range(sum(q_lens)) if i != 3]
    close(got2[keep], want[keep], torch.bfloat16)


@pytest.mark.parametrize("nH,nKV,hd,ps,window", [(4, 2, 16, 16, None), (3, 1, 32, 8, None), (6, 3, 48, 32, 20),
                                                  (32, 8, 64, 16, None), (8, 2, 80, 4, 70), (4, 1, 128, 16, None),
                                                  (2, 2, 256, 16, None), (16, 1, 64, 64, None), (32, 2, 64, 16, 300)])
@pytest.mark.parametrize("n_splits", [1, 3, 8])
def test_attn_decode_bf16(nH, nKV, hd, ps, window, n_splits):
    """Single-token entries at the first position, at page edges and deep in a context, beside
    a longer entry that the kernel must leave alone; any number of splits gives the same."""
    q_lens, ctx = [1, 1, 5, 1, 1, 1], [0, 15, 3, 16, 777, 255]
    k, v, table, pos, re = _paged_setup(torch.bfloat16, nKV, hd, ps, q_lens, ctx, num_pages=1200 // ps + 16)
    cu, cb = _cu(q_lens, ctx)
    q = rnd(sum(q_lens), nH * hd, dtype=torch.bfloat16, seed=13)
    want = torch.empty_like(q)
    ref.attention_generic(q, k, v, table, pos, re, want, nH, window, 1 / math.sqrt(hd))
    got = torch.full_like(q, 7.0)
    n_scr = ops().attn_decode_scratch_floats(sum(q_lens), nH, hd, n_splits)
    scratch = torch.full((max(n_scr, 1),), float("nan"), device=DEV)
    ops().attn_decode_bf16(q, k, v, table, cu, cb, got, scratch, len(q_lens), nH, window, 1 / math.sqrt(hd),
                           n_splits, 778)
    multi = [2, 3, 4, 5, 6]
    assert float((got[multi] - 7.0).abs().max()) == 0.0
    keep = [i for i in range(sum(q_lens)) if i not in multi]
    close(got[keep], want[keep], torch.bfloat16)


def test_attn_bf16_finds_a_far_key_and_respects_the_window_edge():
    nH, nKV, hd, ps = 8, 2, 64, 16
    ctx_len, far = 1500, 333
    for single in (True, False):
        q_lens = [1] if single else [2]
        ctx = [ctx_len] if single else [ctx_len - 1]
        k, v, table, pos, re = _paged_setup(torch.bfloat16, nKV, hd, ps, q_lens, ctx, num_pages=128, seed=5)
        k *= 0.1
        cu, cb = _cu(q_lens, ctx)
        q = rnd(sum(q_lens), nH * hd, dtype=torch.bfloat16, seed=14)
        page, slot = int(table[0, far // ps]), far % ps
        last = sum(q_lens) - 1
        for h in range(nKV):
            k[page, h, slot] = (6.0 * q[last].view(nH, hd)[h * 4].float()).bfloat16()
        for window, hit in ((None, True), (ctx_len - far + 1, True), (ctx_len - far, False)):
            out = torch.zeros_like(q)
            if single:
                scratch = torch.empty(ops().attn_decode_scratch_floats(1, nH, hd, 4), device=DEV)
                ops().attn_decode_bf16(q, k, v, table, cu, cb, out, scratch, 1, nH, window, 1 / math.sqrt(hd), 4, ctx_len + 1)
            else:
                ops().attn_prefill_bf16(q, k, v, table, cu, cb, out, 1, 2, nH, window, 1 / math.sqrt(hd), False)
            for h in (0, 4):
                d = float((out[last].view(nH, hd)[h].float() - v[page, h // 4, slot].float()).abs().max())
                assert (d < 0.05) == hit, (single, window, h, d)


# ----------------------------------------------------------------------------- tcgen05 products
def _mm_ref(x, w, bias=None):
    r = x.double() @ w.double().T
    return r + bias.double() if bias is not None else r


@pytest.mark.parametrize("M,N,K", [(1, 128, 64), (8, 192, 96), (16, 301, 200), (33, 2048, 2048), (64, 256, 8192),
                                   (130, 384, 72), (300, 1000, 520), (2048, 512, 1024)])
def test_gemm_sm100(M, N, K):
    x = rnd(M, K, dtype=torch.bfloat16, seed=1)
    w = rnd(N, K, dtype=torch.bfloat16, seed=2, std=0.05)
    b = rnd(N, dtype=torch.bfloat16, seed=3)
    want = _mm_ref(x, w)
    out = torch.full((M, N), 7.0, dtype=torch.bfloat16, device=DEV)
    ops().gemm_sm100(x, w, None, out)
    close(out, want, torch.bfloat16)
    ops().gemm_sm100(x, w, b, out)
    close(out, _mm_ref(x, w, b), torch.bfloat16)
    o32 = torch.empty(M, N, device=DEV)
    ops().gemm_sm100(x, w, None, o32)
    close(o32, want, torch.float32, scale=50)                 # float32 sums of bf16 products, other order
    for splits in (2, 5):
        s = ops().gemm_splits(K, splits)
        part = torch.full((s, M, N), float("nan"), device=DEV)
        ops().gemm_sm100(x, w, None, part, splits=splits)
        close(part.double().sum(0), want, torch.float32, scale=50)
    for tile in (16, 32, 64, 128, 256):
        ops().gemm_sm100(x, w, None, out, token_tile=tile)
        close(out, want, torch.bfloat16)
    assert ops().gemm_status(DEV) == 0


@pytest.mark.parametrize("M,I,K", [(1, 192, 64), (8, 8192, 2048), (40, 200, 96), (257, 384, 520)])
def test_gemm_swiglu_sm100(M, I, K):
    x = rnd(M, K, dtype=torch.bfloat16, seed=1)
    w = rnd(2 * I, K, dtype=torch.bfloat16, seed=2, std=0.08)
    gu = _mm_ref(x, w).to(torch.bfloat16)
    want = torch.empty(M, I, dtype=torch.bfloat16, device=DEV)
    ref.swiglu(gu, want)
    out = torch.empty(M, I, dtype=torch.bfloat16, device=DEV)
    ops().gemm_swiglu_sm100(x, w, out)
    close(out, want, torch.bfloat16)
    assert ops().gemm_status(DEV) == 0


def test_add_rmsnorm_sums_partials_in_order():
    N, H, S = 5, 2048, 4
    h = rnd(N, H, seed=1)
    parts = rnd(S, N, H, seed=2)
    w = 1 + 0.1 * rnd(H, seed=3)
    for dtype in (torch.float32, torch.bfloat16):
        h1, h2 = h.clone(), h.clone()
        o1, o2 = torch.empty(N, H, dtype=dtype, device=DEV), torch.empty(N, H, dtype=dtype, device=DEV)
        ops().add_rmsnorm(h1, parts, w, o1, 1e-5)
        ref.add_rmsnorm(h2, parts, w, o2, 1e-5)
        close(o1, o2, dtype)
        close(h1, h2, torch.float32)
    h1 = h.clone()
    ops().residual_add(h1, parts)
    close(h1, h.double() + parts.double().sum(0), torch.float32)


def test_consumers_add_partial_sums():
    """The conv and rope kernels take a float32 stack of split-K partial sums in place of their
    input and give what they give for the summed, rounded input."""
    S, H, L = 3, 96, 3
    q_lens, ctx = [1, 4, 1], [5, 0, 2]
    cu, cb, N = _ragged(q_lens, ctx)
    slots = torch.tensor([0, 1, 2], dtype=torch.int32, device=DEV)
    parts = rnd(S, N, 3 * H, seed=4)
    whole = parts.double().sum(0).to(torch.bfloat16)
    w = rnd(H, L, seed=5, std=0.3)
    st1, st2 = torch.zeros(4, L - 1, H, device=DEV), torch.zeros(4, L - 1, H, device=DEV)
    o1, o2 = torch.zeros(N, H, dtype=torch.bfloat16, device=DEV), torch.zeros(N, H, dtype=torch.bfloat16, device=DEV)
    ops().shortconv(parts, w, None, st1, o1, cu, cb, slots, 3, 4)
    ops().shortconv(whole, w, None, st2, o2, cu, cb, slots, 3, 4)
    close(o1, o2, torch.bfloat16, scale=0.5)
    close(st1, st2, torch.float32, scale=100)
    nH, nKV, hd, ps = 4, 2, 32, 8
    k1, v1, table, pos, re = _paged_setup(torch.bfloat16, nKV, hd, ps, q_lens, ctx)
    k2, v2 = k1.clone(), v1.clone()
    parts = rnd(S, N, (nH + 2 * nKV) * hd, seed=6)
    whole = parts.double().sum(0).to(torch.bfloat16)
    qw = 1 + 0.1 * rnd(hd, seed=7)
    inv = (10000.0 ** (-2.0 * torch.arange(hd // 2, dtype=torch.float64) / hd)).float().to(DEV)
    stt = torch.zeros(1, dtype=torch.int32, device=DEV)
    q1 = torch.empty(N, nH * hd, dtype=torch.bfloat16, device=DEV)
    q2 = torch.empty_like(q1)
    ops().rope_cache(parts, q1, qw, qw, inv, False, 1.0, k1, v1, table, pos, re, nH, nKV, hd, 1e-5, stt)
    ops().rope_cache(whole, q2, qw, qw, inv, False, 1.0, k2, v2, table, pos, re, nH, nKV, hd, 1e-5, stt)
    assert torch.equal(q1, q2) and torch.equal(k1, k2) and torch.equal(v1, v2)


@pytest.mark.parametrize("nH,nKV,ps,window", [(4, 2, 16, None), (32, 8, 16, None), (3, 1, 8, None), (16, 1, 64, None),
                                               (8, 2, 32, 70), (8, 8, 16, 300)])
def test_attn_prefill_sm100(nH, nKV, ps, window):
    """The tcgen05 prefill kernel: portions that start at a page edge, inside a page, at 0;
    shorter and longer than one 128-row block; a single-token entry handled or left alone."""
    hd = 64
    q_lens, ctx = [3, 1, 150, 128, 2, 129, 400], [0, 37, 5, 64, 63, 131, 77]
    k, v, table, pos, re = _paged_setup(torch.bfloat16, nKV, hd, ps, q_lens, ctx, num_pages=1400 // ps + 64)
    cu, cb = _cu(q_lens, ctx)
    q = rnd(sum(q_lens), nH * hd, dtype=torch.bfloat16, seed=12)
    want = torch.empty_like(q)
    ref.attention_generic(q, k, v, table, pos, re, want, nH, window, 1 / math.sqrt(hd))
    got = torch.zeros_like(q)
    ops().attn_prefill_sm100(q, k, v, table, cu, cb, got, len(q_lens), max(q_lens), nH, window, 1 / math.sqrt(hd), False)
    assert ops().gemm_status(DEV) == 0
    close(got, want, torch.bfloat16)
    got2 = torch.full_like(q, 7.0)
    ops().attn_prefill_sm100(q, k, v, table, cu, cb, got2, len(q_lens), max(q_lens), nH, window, 1 / math.sqrt(hd), True)
    assert float((got2[3] - 7.0).abs().max()) == 0.0
    keep = [i for i in range(sum(q_lens)) if i != 3]
    close(got2[keep], want[keep], torch.bfloat16)


@pytest.mark.parametrize("n_splits,window", [(2, None), (3, None), (4, None), (2, 2500), (4, 300)])
def test_attn_prefill_sm100_cut_into_runs_of_keys(n_splits, window):
    """The same kernel with the keys of every block cut into runs that a second kernel merges: a
    long context (every run has tiles), contexts too short to cut (the first run does all, the
    others write empty records), a single-token entry handled or left alone, a far key that only
    one run sees."""
    nH, nKV, hd, ps = 8, 2, 64, 16
    q_lens, ctx = [200, 1, 130, 3], [4300, 2100, 0, 1000]
    k, v, table, pos, re = _paged_setup(torch.bfloat16, nKV, hd, ps, q_lens, ctx, num_pages=8000 // ps + 64, seed=3)
    k *= 0.3
    cu, cb = _cu(q_lens, ctx)
    q = rnd(sum(q_lens), nH * hd, dtype=torch.bfloat16, seed=12)
    far = 777                                                # one key that the last row of entry 0 cannot miss
    page, slot = int(table[0, far // ps]), far % ps
    k[page, 0, slot] = (5.0 * q[199].view(nH, hd)[0].float()).bfloat16()
    want = torch.empty_like(q)
    ref.attention_generic(q, k, v, table, pos, re, want, nH, window, 1 / math.sqrt(hd))
    floats = ops().attn_prefill_scratch_floats(q.shape[0], nH, hd, n_splits)
    scratch = torch.full((floats,), float("nan"), device=DEV)
    for skip_single in (False, True):
        got = torch.full_like(q, 7.0)
        ops().attn_prefill_sm100(q, k, v, table, cu, cb, got, len(q_lens), max(q_lens), nH, window, 1 / math.sqrt(hd),
                                 skip_single, None, scratch, n_splits)
        assert ops().gemm_status(DEV) == 0
        keep = [i for i in range(sum(q_lens)) if not (skip_single and i == 200)]
        close(got[keep], want[keep], torch.bfloat16)
        if skip_single:
            assert float((got[200] - 7.0).abs().max()) == 0.0
    if window is None:
        d = float((got[199].view(nH, hd)[0].float() - v[page, 0, slot].float()).abs().max())
        assert d < 0.05, d
    with pytest.raises(Exception):
        ops().attn_prefill_sm100(q, k, v, table, cu, cb, got, len(q_lens), max(q_lens), nH, window, 1 / math.sqrt(hd),
                                 False, None, scratch[:10], n_splits)


def test_attn_prefill_sm100_finds_a_far_key_and_respects_the_window_edge():
    nH, nKV, hd, ps = 8, 2, 64, 16
    ctx_len, far = 1500, 333
    q_lens, ctx = [130], [ctx_len - 129]                        # the last row sits at position ctx_len
    k, v, table, pos, re = _paged_setup(torch.bfloat16, nKV, hd, ps, q_lens, ctx, num_pages=128, seed=5)
    k *= 0.1
    cu, cb = _cu(q_lens, ctx)
    q = rnd(130, nH * hd, dtype=torch.bfloat16, seed=14)
    page, slot = int(table[0, far // ps]), far % ps
    for h in range(nKV):
        k[page, h, slot] = (6.0 * q[129].view(nH, hd)[h * 4].float()).bfloat16()
    for window, hit in ((None, True), (ctx_len - far + 1, True), (ctx_len - far, False)):
        out = torch.zeros_like(q)
        ops().attn_prefill_sm100(q, k, v, table, cu, cb, out, 1, 130, nH, window, 1 / math.sqrt(hd), False)
        for h in (0, 4):
            d = float((out[129].view(nH, hd)[h].float() - v[page, h // 4, slot].float()).abs().max())
            assert (d < 0.05) == hit, (window, h, d)


@pytest.mark.parametrize("M,N,K", [(5, 77, 100), (200, 301, 36), (70, 128, 64)])
def test_linear_routes_every_shape(M, N, K):
    """`ops.linear` in bfloat16: the tcgen05 kernel where it takes the operands (few rows, K a
    multiple of 8), the library otherwise; bias and float32 output either way."""
    x = rnd(M, K, dtype=torch.bfloat16, seed=1)
    w = rnd(N, K, dtype=torch.bfloat16, seed=2, std=0.1)
    b = rnd(N, dtype=torch.bfloat16, seed=3)
    out = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
    ops().linear(x, w, None, out)
    close(out, _mm_ref(x, w), torch.bfloat16)
    ops().linear(x, w, b, out)
    close(out, _mm_ref(x, w, b), torch.bfloat16)
    o32 = torch.empty(M, N, device=DEV)
    ops().linear(x, w, None, o32)
    close(o32, _mm_ref(x, w), torch.float32, scale=50)


@pytest.mark.parametrize("M,N,K", [(1, 128, 64), (8, 2048, 8192), (16, 2048, 2048), (3, 301, 200)])
def test_gemm_adds_into_the_residual_stream(M, N, K):
    x = rnd(M, K, dtype=torch.bfloat16, seed=1)
    w = rnd(N, K, dtype=torch.bfloat16, seed=2, std=0.05)
    h = rnd(M, N, seed=3)
    want = h.double() + _mm_ref(x, w)
    from neurogrid_b200.parts.base import Workspace
    assert ops().linear_to_residual(x, w, None, Workspace(64, DEV), "t", residual=h) is None
    close(h, want, torch.float32, scale=100)
    assert ops().gemm_status(DEV) == 0


def test_tensor_core_kernels_repeat_bit_for_bit():
    """The same launch thirty times gives the same bits: a race between the producer, the MMA
    issuer and the softmax or epilogue warps would show as a difference between runs."""
    nH, nKV, hd, ps = 32, 8, 64, 16
    q_lens, ctx = [1500, 700, 1], [40, 0, 900]
    k, v, table, pos, re = _paged_setup(torch.bfloat16, nKV, hd, ps, q_lens, ctx, num_pages=256)
    cu, cb = _cu(q_lens, ctx)
    q = rnd(sum(q_lens), nH * hd, dtype=torch.bfloat16, seed=12)
    first = None
    for i in range(30):
        out = torch.zeros_like(q)
        ops().attn_prefill_sm100(q, k, v, table, cu, cb, out, len(q_lens), max(q_lens), nH, None, 0.125, False)
        if first is None:
            first = out.clone()
        assert torch.equal(out, first), f"attention run {i} differs"
    x = rnd(40, 2048, dtype=torch.bfloat16, seed=1)
    w = rnd(4096, 2048, dtype=torch.bfloat16, seed=2, std=0.05)
    first = None
    for i in range(30):
        o = torch.empty(40, 2048, dtype=torch.bfloat16, device=DEV)
        ops().gemm_swiglu_sm100(x, w, o)
        part = torch.empty(ops().gemm_splits(2048, 4), 40, 4096, device=DEV)
        ops().gemm_sm100(x, w, None, part, splits=4)
        if first is None:
            first = (o.clone(), part.clone())
        assert torch.equal(o, first[0]) and torch.equal(part, first[1]), f"product run {i} differs"
    assert ops().gemm_status(DEV) == 0


def test_residual_add_epilogue_spread_is_bounded():
    """The epilogue that adds a split-K product into the float32 stream (red.global.add) fixes no
    order for its additions, so runs may differ in the last bits, and by no more: thirty runs from
    the same start stay within 1e-6 of the stream's scale of each other."""
    from neurogrid_b200.parts.base import Workspace
    ws = Workspace(64, DEV)
    for M, N, K in ((8, 2048, 8192), (40, 2048, 2048), (3, 304, 200)):
        x = rnd(M, K, dtype=torch.bfloat16, seed=1)
        w = rnd(N, K, dtype=torch.bfloat16, seed=2, std=0.05)
        h0 = rnd(M, N, seed=3, std=3.0)
        want = h0.double() + _mm_ref(x, w)
        scale = float(want.abs().max())
        lo = hi = None
        for _ in range(30):
            h = h0.clone()
            assert ops().linear_to_residual(x, w, None, ws, "t", residual=h) is None
            lo = h.clone() if lo is None else torch.minimum(lo, h)
            hi = h.clone() if hi is None else torch.maximum(hi, h)
        assert float((hi - lo).max()) <= 1e-6 * scale, (M, N, K, float((hi - lo).max()), scale)
        close(hi, want, torch.float32, scale=100)
    assert ops().gemm_status(DEV) == 0
