"""The persistent chain kernel (norms, tensor-core products and one-token convolutions of a
decode step inside one launch) against the same operations launched one by one."""
import pytest
import torch

import kernel_refs as ref
from test_kernels_gpu import _ragged, close, rnd

pytestmark = pytest.mark.gpu
DEV = "cuda"
BF = torch.bfloat16


def ops():
    from neurogrid_b200.csrc import ops as o
    return o


@pytest.fixture(autouse=True)
def _chains_on(monkeypatch):
    """The chain kernel is an option that is off by default: these tests switch it on."""
    monkeypatch.setattr(ops(), "CHAIN", True)


class _WS:
    """The few workspace calls the recorded launchers make."""
    max_rows = 64

    def __init__(self):
        self.bufs = {}

    def buf(self, name, n, cols, dtype):
        return self.bufs.setdefault((name, n, cols, dtype), torch.zeros(n, cols, dtype=dtype, device=DEV))

    def flat(self, name, numel, dtype, reserve=0):
        return self.bufs.setdefault((name, numel, dtype), torch.zeros(max(numel, 1), dtype=dtype, device=DEV))


@pytest.mark.parametrize("M,N,K", [(1, 256, 128), (8, 6144, 2048), (13, 1000, 264), (16, 40000, 512),
                                   (33, 2048, 2048), (64, 520, 1032)])
def test_single_products(M, N, K):
    """Every epilogue as a chain of one operation; N = 40000 gives a block several tiles."""
    o = ops()
    x = rnd(M, K, dtype=BF, seed=1)
    w = rnd(N, K, dtype=BF, seed=2, std=0.05)
    want = x.double() @ w.double().T
    with o.chain_scope(DEV, M) as ch:
        assert ch is not None
        out32 = torch.zeros(M, N, device=DEV)
        o.gemm_sm100(x, w, None, out32)
    assert ch.launches == 1
    close(out32, want, torch.float32, scale=50)
    with o.chain_scope(DEV, M):
        out16 = torch.zeros(M, N, dtype=BF, device=DEV)
        o.gemm_sm100(x, w, None, out16)
    close(out16, want, BF)
    # split-K partial sums and the residual add
    ws = _WS()
    h = rnd(M, N, seed=3)
    h0 = h.clone()
    with o.chain_scope(DEV, M):
        parts = o.linear_to_residual(x, w, None, ws, "p")
        assert o.linear_to_residual(x, w, None, ws, "q", residual=h) is None
    got = parts.double().sum(0) if parts.dim() == 3 else parts.double()
    close(got, want, BF if parts.dim() == 2 else torch.float32, scale=1 if parts.dim() == 2 else 50)
    close(h - h0, want, torch.float32, scale=50)
    assert o.gemm_status(DEV) == 0


@pytest.mark.parametrize("M,I,K", [(3, 192, 128), (8, 8192, 2048), (40, 1000, 520)])
def test_swiglu_product(M, I, K):
    o = ops()
    x = rnd(M, K, dtype=BF, seed=4)
    w = rnd(2 * I, K, dtype=BF, seed=5, std=0.05)
    with o.chain_scope(DEV, M):
        out = torch.zeros(M, I, dtype=BF, device=DEV)
        o.gemm_swiglu_sm100(x, w, out)
    gu = (x.double() @ w.double().T).to(BF)
    want = torch.zeros(M, I, dtype=BF, device=DEV)
    ref.swiglu(gu, want)
    close(out, want, BF, scale=1.5)


def _conv_layer(o, ws, h, x_buf, wts, state, cu, cb, slots, n_entries, eps):
    """norm -> in_proj -> conv -> out_proj (+= h) -> norm -> gate/up -> down (+= h)."""
    n1, w_in, w_conv, b_conv, w_out, n2, w_gu, w_down = wts
    M, H = h.shape
    o.add_rmsnorm(h, None, n1, x_buf, eps)
    p = o.linear_to_residual(x_buf, w_in, None, ws, "conv_in")
    g = ws.buf("gated", M, H, BF)
    o.shortconv(p, w_conv, b_conv, state, g, cu, cb, slots, n_entries, 1)
    assert o.linear_to_residual(g, w_out, None, ws, "mix", residual=h) is None
    o.add_rmsnorm(h, None, n2, x_buf, eps)
    act = ws.buf("act", M, w_down.shape[1], BF)
    o.gemm_swiglu_sm100(x_buf, w_gu, act)
    assert o.linear_to_residual(act, w_down, None, ws, "ffn", residual=h) is None


@pytest.mark.parametrize("M,H,I,L,bias", [(8, 2048, 8192, 3, False), (5, 264, 520, 4, True), (1, 96, 192, 2, False),
                                          (30, 512, 1024, 3, True)])
def test_conv_layer_chain_equals_separate_launches(M, H, I, L, bias, monkeypatch):
    """Two layers in one chain: every kind of operation, barriers between them, padding
    entries, state slots, against the same launchers run one by one."""
    o = ops()
    q_lens = [1] * (M - 1) + [0]                 # the last entry is padding: it brings nothing
    ctx = [5, 0, 1, 40, 2, 7, 9, 3][: M] + [3] * max(0, M - 8)
    cu, cb, _ = _ragged(q_lens, ctx)
    slots = torch.arange(M, dtype=torch.int32, device=DEV).flip(0).contiguous()

    def weights(seed):
        return (1 + 0.1 * rnd(H, seed=seed), rnd(3 * H, H, dtype=BF, seed=seed + 1, std=0.03),
                rnd(H, L, seed=seed + 2, std=0.3), rnd(H, seed=seed + 3, std=0.1) if bias else None,
                rnd(H, H, dtype=BF, seed=seed + 4, std=0.03), 1 + 0.1 * rnd(H, seed=seed + 5),
                rnd(2 * I, H, dtype=BF, seed=seed + 6, std=0.03), rnd(H, I, dtype=BF, seed=seed + 7, std=0.03))

    layers = [weights(10), weights(30)]
    results = []
    for chained in (False, True, True):
        h = rnd(M, H, seed=50)
        states = [rnd(M + 1, L - 1, H, seed=60 + i) for i in range(2)]
        ws, x_buf = _WS(), torch.zeros(M, H, dtype=BF, device=DEV)
        scope = o.chain_scope(DEV, M) if chained else __import__("contextlib").nullcontext()
        with scope as ch:
            for wts, st in zip(layers, states):
                _conv_layer(o, ws, h, x_buf, wts, st, cu, cb, slots, M, 1e-5)
        if chained:
            assert ch.launches == 1
        torch.cuda.synchronize()
        results.append((h.clone(), [s.clone() for s in states]))
    assert o.gemm_status(DEV) == 0
    (h0, s0), (h1, s1), (h2, s2) = results
    # the residual adds are atomic (their order is not fixed): close, not equal
    scale = float(h0.abs().max())
    assert float((h1 - h0).abs().max()) < 2e-2 * scale
    assert float((h2 - h1).abs().max()) < 2e-2 * scale
    for a, b in zip(s0, s1):
        assert float((a - b).abs().max()) <= 2e-2 * float(a.abs().max())
        assert torch.equal(a[M], b[M])                              # a slot no entry names stays


def test_final_norm_gathers_rows_and_head_follows():
    o = ops()
    M, H, V = 8, 264, 3001
    h = rnd(M, H, seed=1)
    w = 1 + 0.1 * rnd(H, seed=2)
    head = rnd(V, H, dtype=BF, seed=3, std=0.05)
    rows = torch.tensor([6, 0, 3], dtype=torch.int32, device=DEV)
    x = torch.zeros(3, H, dtype=BF, device=DEV)
    logits = torch.zeros(3, V, device=DEV)
    with o.chain_scope(DEV, M) as ch:
        o.add_rmsnorm(h, None, w, x, 1e-6, rows)
        o.linear(x, head, None, logits)
    assert ch.launches == 1
    want_x = torch.zeros_like(x)
    ref.add_rmsnorm(h.clone(), None, w, want_x, 1e-6, rows)
    close(x, want_x, BF)
    close(logits, x.double() @ head.double().T, torch.float32, scale=50)


@pytest.mark.parametrize("name", ["A", "B"])
def test_decode_steps_through_chains_match_separate_kernels(model_dirs, name, monkeypatch):
    """A model's decode steps (eager first, then as a captured graph) with the chains on and off."""
    from helpers import make_runner, rel_err
    from neurogrid_b200.engine import StepEntry
    from tiny_configs import PAGE_SIZE
    o = ops()
    prompts = {"a": list(range(3, 40)), "b": list(range(50, 61)), "c": [7]}
    out = {}
    for chained in (False, True):
        monkeypatch.setattr(o, "CHAIN", chained)
        runner = make_runner(model_dirs[name], dtype=BF, device="cuda", page_size=PAGE_SIZE[name], num_pages=64,
                             max_requests=4, max_seq_len=128)
        for r, p in prompts.items():
            runner.step([StepEntry(r, p, [])])
        rows = []
        for i in range(12):
            rows.append(runner.step([StepEntry(r, [(11 * i + 5 * j) % 200], [0]) for j, r in enumerate(prompts)]).clone())
        runner.check_status()
        assert runner.stats()["graph_replays"] > 0
        out[chained] = torch.cat(rows)
    assert rel_err(out[True], out[False]) < 2e-2
