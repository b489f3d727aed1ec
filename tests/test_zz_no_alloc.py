"""The allocation-free decode-attention entry point, called through its exported C symbol.

Some users of the library cannot hand a kernel scratch memory: a host that links the C ABI
without an allocator, a server that gave all device memory away at start-up, a loop where
cudaMalloc must never run.  ``ng_attn_decode_bf16_noalloc`` keeps the split scratch inside the
library for them.  Here its output is checked against the plain statement of the attention
(``kernel_refs.attention_generic``, float64) and against the ordinary entry point (scratch from
the caller) on the same inputs, twice in a row: the second call runs on whatever the first left
in the shared array, with other splits and contexts, so stale content would show.  The steps
hold a prompt portion between the single-token entries, so rows outnumber entries and a row
index exceeds the number of entries.  That no device memory is taken is read from the driver's
own count of free memory (``cudaMemGetInfo``), which sees a cudaMalloc by anyone.
This file is collected last on purpose; it also passes alone in a fresh process.
"""
import ctypes
import math

import pytest
import torch

import kernel_refs

pytestmark = pytest.mark.gpu
HD, NH, NKV, PS = 64, 8, 2, 16
C = ctypes


def _case(seed, q_lens, ctx_lens, num_pages=256):
    """Entry e brings q_lens[e] rows after ctx_lens[e] cached tokens."""
    g = torch.Generator().manual_seed(seed)
    R, N = len(ctx_lens), sum(q_lens)
    k = torch.randn(num_pages, NKV, PS, HD, generator=g).bfloat16().cuda()
    v = torch.randn(num_pages, NKV, PS, HD, generator=g).bfloat16().cuda()
    q = torch.randn(N, NH * HD, generator=g).bfloat16().cuda()
    stride = max(-(-(c + n) // PS) for c, n in zip(ctx_lens, q_lens))
    perm = torch.randperm(num_pages, generator=g).tolist()
    table = torch.full((R, stride), -1, dtype=torch.int32)
    pos, row_entry, cu = [], [], [0]
    for e, (c, n) in enumerate(zip(ctx_lens, q_lens)):
        for j in range(-(-(c + n) // PS)):
            table[e, j] = perm.pop()
        pos += list(range(c, c + n))
        row_entry += [e] * n
        cu.append(cu[-1] + n)
    t = lambda x: torch.tensor(x, dtype=torch.int32).cuda()
    return q, k, v, table.cuda(), t(cu), t(ctx_lens), t(pos), t(row_entry)


def _bind(lib):
    fn = lib.ng_attn_decode_bf16_noalloc
    fn.restype = C.c_int
    fn.argtypes = [C.c_void_p] * 4 + [C.c_int] + [C.c_void_p] * 3 + [C.c_int] * 8 + [C.c_float, C.c_int, C.c_int,
                                                                                   C.c_void_p]
    lib.ng_attn_decode_noalloc_max_floats.restype = C.c_int
    return fn


def test_no_alloc_entry_matches_the_plain_statement_twice():
    from neurogrid_b200.csrc import build, ops
    lib = build.load("attention_bf16", {"NG_HEAD_DIM": HD})
    fn = _bind(lib)
    cap = lib.ng_attn_decode_noalloc_max_floats()
    assert cap == 1 << 20
    stream = torch.cuda.current_stream().cuda_stream
    scale = 1 / math.sqrt(HD)
    cases = ((1, [1, 1, 5, 1, 1, 1], [0, 15, 40, 700, 255, 1033], 6),      # a 5-token portion between the singles
             (2, [1, 9, 1, 1, 1], [90, 3, 2047, 3, 511], 3))
    for seed, q_lens, ctx_lens, splits in cases:
        q, k, v, table, cu, cb, pos, row_entry = _case(seed, q_lens, ctx_lens)
        R, N = len(ctx_lens), sum(q_lens)
        single = torch.tensor([r for e in range(R) if q_lens[e] == 1 for r in [int(cu[e])]], device="cuda")
        assert int(single.max()) >= R                          # a row index beyond the number of entries
        max_ctx = max(c + 1 for c, n in zip(ctx_lens, q_lens) if n == 1)
        # the plain statement, float64 inside
        plain = torch.zeros_like(q)
        kernel_refs.attention_generic(q, k, v, table, pos, row_entry, plain, NH, None, scale)
        # the ordinary entry point with the caller's scratch
        want = torch.full_like(q, 7.0)
        scratch = torch.empty(ops.attn_decode_scratch_floats(N, NH, HD, splits), device="cuda")
        ops.attn_decode_bf16(q, k, v, table, cu, cb, want, scratch, R, NH, None, scale, splits, max_ctx)
        got = torch.full_like(q, 7.0)
        torch.cuda.synchronize()
        free_before, _ = torch.cuda.mem_get_info()
        rc = fn(q.data_ptr(), k.data_ptr(), v.data_ptr(), table.data_ptr(), table.shape[1], cu.data_ptr(),
                cb.data_ptr(), got.data_ptr(), N, R, NH, NKV, HD, PS, k.shape[0], 0, scale, splits, max_ctx, stream)
        assert rc == 0
        torch.cuda.synchronize()
        free_after, _ = torch.cuda.mem_get_info()
        assert free_after >= free_before                       # the driver saw no allocation, by anyone
        err = float((got[single].float() - plain[single].float()).abs().max() / plain[single].float().abs().max())
        assert err < 1.2e-2, err                               # the tolerance of the bfloat16 kernel tests
        assert torch.equal(got[single], want[single])          # and the ordinary entry's bits
        multi = torch.tensor([r for r in range(N) if r not in set(single.tolist())], device="cuda")
        assert float((got[multi].float() - 7.0).abs().max()) == 0.0   # rows of the portion are not this kernel's
        # told fewer rows than the step holds, the entry point skips the entries beyond them and
        # writes nothing outside what it was told of
        short = torch.full_like(q, 7.0)
        n_told = int(single[-2]) + 1
        rc = fn(q.data_ptr(), k.data_ptr(), v.data_ptr(), table.data_ptr(), table.shape[1], cu.data_ptr(),
                cb.data_ptr(), short.data_ptr(), n_told, R, NH, NKV, HD, PS, k.shape[0], 0, scale, splits, max_ctx,
                stream)
        torch.cuda.synchronize()
        assert rc == 0
        assert torch.equal(short[single[:-1]], want[single[:-1]])
        assert float((short[n_told:].float() - 7.0).abs().max()) == 0.0
    # a call that needs more scratch than the library holds is refused and launches nothing
    q, k, v, table, cu, cb, _, _ = _case(3, [1] * 64, [100] * 64, num_pages=512)
    big_splits = cap // (64 * NH * (HD + 2)) + 1
    out = torch.full_like(q, 3.0)
    rc = fn(q.data_ptr(), k.data_ptr(), v.data_ptr(), table.data_ptr(), table.shape[1], cu.data_ptr(),
            cb.data_ptr(), out.data_ptr(), 64, 64, NH, NKV, HD, PS, k.shape[0], 0, scale, big_splits, 101, stream)
    torch.cuda.synchronize()
    assert rc == 4 and float((out.float() - 3.0).abs().max()) == 0.0
