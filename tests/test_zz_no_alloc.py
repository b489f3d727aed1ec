"""The allocation-free decode-attention entry point, called through its exported C symbol.

Some users of the library cannot hand a kernel scratch memory: a host that links the C ABI
without an allocator, a server that gave all device memory away at start-up, a loop where
cudaMalloc must never run.  ``ng_attn_decode_bf16_noalloc`` keeps the split scratch inside the
library for them.  Here it is checked against the ordinary entry point (scratch from the
caller) on the same inputs, twice in a row: the second call runs on whatever the first left
in the shared array, with other splits and contexts, so stale content would show.
This file is collected last on purpose; it also passes alone in a fresh process.
"""
import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu
HD, NH, NKV, PS = 64, 8, 2, 16
C = ctypes


def _case(seed, ctx_lens, num_pages=256):
    g = torch.Generator().manual_seed(seed)
    R = len(ctx_lens)
    k = torch.randn(num_pages, NKV, PS, HD, generator=g).bfloat16().cuda()
    v = torch.randn(num_pages, NKV, PS, HD, generator=g).bfloat16().cuda()
    q = torch.randn(R, NH * HD, generator=g).bfloat16().cuda()
    stride = max(-(-(c + 1) // PS) for c in ctx_lens)
    perm = torch.randperm(num_pages, generator=g).tolist()
    table = torch.full((R, stride), -1, dtype=torch.int32)
    for e, c in enumerate(ctx_lens):
        for j in range(-(-(c + 1) // PS)):
            table[e, j] = perm.pop()
    cu = torch.arange(R + 1, dtype=torch.int32).cuda()
    cb = torch.tensor(ctx_lens, dtype=torch.int32).cuda()
    return q, k, v, table.cuda(), cu, cb


def test_no_alloc_entry_matches_the_ordinary_one_twice():
    from neurogrid_b200.csrc import build, ops
    lib = build.load("attention_bf16", {"NG_HEAD_DIM": HD})
    fn = lib.ng_attn_decode_bf16_noalloc
    fn.restype = C.c_int
    fn.argtypes = [C.c_void_p] * 4 + [C.c_int] + [C.c_void_p] * 3 + [C.c_int] * 8 + [C.c_float, C.c_int, C.c_int,
                                                                                   C.c_void_p]
    lib.ng_attn_decode_noalloc_max_floats.restype = C.c_int
    cap = lib.ng_attn_decode_noalloc_max_floats()
    assert cap == 1 << 20
    stream = torch.cuda.current_stream().cuda_stream
    scale = 1 / math.sqrt(HD)
    for seed, ctx_lens, splits in ((1, [0, 15, 700, 255, 1033], 6), (2, [90, 2047, 3, 511], 3)):
        q, k, v, table, cu, cb = _case(seed, ctx_lens)
        R = len(ctx_lens)
        want = torch.zeros_like(q)
        scratch = torch.empty(ops.attn_decode_scratch_floats(R, NH, HD, splits), device="cuda")
        ops.attn_decode_bf16(q, k, v, table, cu, cb, want, scratch, R, NH, None, scale, splits, max(ctx_lens) + 1)
        got = torch.zeros_like(q)
        before = torch.cuda.memory_allocated()
        rc = fn(q.data_ptr(), k.data_ptr(), v.data_ptr(), table.data_ptr(), table.shape[1], cu.data_ptr(),
                cb.data_ptr(), got.data_ptr(), R, R, NH, NKV, HD, PS, k.shape[0], 0, scale, splits,
                max(ctx_lens) + 1, stream)
        assert rc == 0
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        err = float((got.float() - want.float()).abs().max() / want.float().abs().max())
        assert err < 1.2e-2, err                              # the tolerance of the bfloat16 kernel tests
        assert torch.equal(got, want)                         # same kernels, same order: in fact identical
    # a call that needs more scratch than the library holds is refused and launches nothing
    q, k, v, table, cu, cb = _case(3, [100] * 64, num_pages=512)
    big_splits = cap // (64 * NH * (HD + 2)) + 1
    out = torch.full_like(q, 3.0)
    rc = fn(q.data_ptr(), k.data_ptr(), v.data_ptr(), table.data_ptr(), table.shape[1], cu.data_ptr(),
            cb.data_ptr(), out.data_ptr(), 64, 64, NH, NKV, HD, PS, k.shape[0], 0, scale, big_splits, 101, stream)
    torch.cuda.synchronize()
    assert rc == 4 and float((out.float() - 3.0).abs().max()) == 0.0
