"""Each part alone, built through the registry from its spec, against the plain functions,
at sizes and options the LFM2 configurations do not use (window, no q/k norm, biases, a
softmax scale, width != heads * head_dim, scaled rotary positions)."""
import math

import pytest
import torch

import plain_lfm2 as plain
from helpers import make_ctx, rel_err
from neurogrid_b200.config import AttentionSpec, NoPositionSpec, RMSNormSpec, RopeSpec, ShortConvSpec, SwiGLUSpec
from neurogrid_b200.parts import PagedView, SlotView, build
from neurogrid_b200.weights import draw

pytestmark = pytest.mark.gpu
DEV = "cuda"
TOL = {torch.float32: 1e-4, torch.bfloat16: 2e-2}


def _bound(category, spec, dtype, seed=0, **kw):
    part = build(category, spec, dtype=dtype, device=DEV, **kw)
    w = draw(part.tensors(), seed)                        # bfloat16 on the CPU, as a model folder holds them
    part.bind(w)
    return part, {k: v.double() for k, v in w.items()}


def _x(T, H, dtype, seed=1):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(T, H, generator=g).to(torch.bfloat16).to(dtype).to(DEV)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rmsnorm_part_with_residual_sum(dtype):
    part, w = _bound("norm", RMSNormSpec(200, 3e-6), dtype)
    h = _x(9, 200, torch.float32)
    d = _x(9, 200, dtype, seed=2)
    out = torch.empty(9, 200, dtype=dtype, device=DEV)
    h0 = h.clone()
    part.forward(h, d, out)
    want = plain.rmsnorm(h0.double().cpu() + d.double().cpu(), w["weight"], 3e-6)
    assert rel_err(out, want) < TOL[dtype] and rel_err(h, h0.double() + d.double()) < 1e-6


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_swiglu_part(dtype):
    part, w = _bound("ffn", SwiGLUSpec(80, 200), dtype)
    x = _x(13, 80, dtype)
    y = part.forward(x, make_ctx([13], [0], [0], dtype=dtype))
    want = plain.swiglu(x.double().cpu(), w["gate_proj.weight"], w["up_proj.weight"], w["down_proj.weight"],
                        rb=dtype == torch.bfloat16)
    assert rel_err(y, want) < TOL[dtype]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("L,bias", [(2, False), (4, True), (7, True)])
def test_shortconv_part_whole_and_cut(dtype, L, bias):
    H, T = 80, 61
    part, w = _bound("mixer", ShortConvSpec(H, L, bias), dtype)
    x = _x(T, H, dtype)
    want = plain.short_conv(x.double().cpu(), w["in_proj.weight"], w.get("in_proj.bias"), w["conv.weight"],
                            w.get("conv.bias"), w["out_proj.weight"], w.get("out_proj.bias"),
                            rb=dtype == torch.bfloat16)
    state = torch.randn(3, L - 1, H, device=DEV)                  # stale slot content must not matter
    whole = part.forward(x, make_ctx([T], [0], [1], dtype=dtype), SlotView(state)).clone()
    assert rel_err(whole, want) < TOL[dtype]
    state2 = torch.randn(3, L - 1, H, device=DEV)
    got, at = [], 0
    for n in (1, 2, 1, 30, 3, 24):
        got.append(part.forward(x[at:at + n].contiguous(), make_ctx([n], [at], [2], dtype=dtype),
                                SlotView(state2)).clone())
        at += n
    assert rel_err(torch.cat(got), want) < TOL[dtype]
    assert torch.allclose(state[1], state2[2], atol=1e-5)          # both slots end with the same last inputs


def _attend(part, x, cuts, dtype, n_kv, hd, ps=8, pages=32):
    k = torch.randn(pages, n_kv, ps, hd, device=DEV).to(dtype)     # stale pages
    v = torch.randn(pages, n_kv, ps, hd, device=DEV).to(dtype)
    perm = torch.randperm(pages).tolist()
    table = torch.full((1, pages), -1, dtype=torch.int32)
    for j in range(-(-x.shape[0] // ps)):
        table[0, j] = perm[j]
    view = PagedView(k, v, table.to(DEV))
    out, at = [], 0
    for n in cuts:
        out.append(part.forward(x[at:at + n].contiguous(), make_ctx([n], [at], [0], dtype=dtype), view).clone())
        at += n
    return torch.cat(out)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("window,qk_norm,pairing", [(None, True, "adjacent"), (9, False, "half"), (1, True, "half")])
def test_attention_part_whole_and_cut(dtype, window, qk_norm, pairing):
    H, nH, nKV, hd, T = 72, 6, 2, 16, 45                           # heads * head_dim = 96 != width
    spec = AttentionSpec(H, nH, nKV, hd, RopeSpec(hd, 5000.0, pairing), qk_norm=qk_norm, qk_norm_eps=2e-6,
                         window=window)
    part, w = _bound("mixer", spec, dtype)
    x = _x(T, H, dtype)
    want = plain.attention(x.double().cpu(), w["q_proj.weight"], w["k_proj.weight"], w["v_proj.weight"],
                           w["o_proj.weight"], w.get("q_norm.weight"), w.get("k_norm.weight"), n_heads=nH,
                           n_kv=nKV, hd=hd, eps=2e-6, theta=5000.0, pairing=pairing, window=window,
                           rb=dtype == torch.bfloat16)
    assert rel_err(_attend(part, x, [T], dtype, nKV, hd), want) < TOL[dtype]
    assert rel_err(_attend(part, x, [2, 1, 17, 1, 1, 20, 3], dtype, nKV, hd), want) < TOL[dtype]


def test_attention_options_no_position_scale_and_bias():
    """No position encoding, a softmax scale of its own, projection biases."""
    H, nH, nKV, hd, T = 64, 4, 4, 16, 20
    spec = AttentionSpec(H, nH, nKV, hd, NoPositionSpec(), softmax_scale=0.37, bias=True)
    part, w = _bound("mixer", spec, torch.float32)
    x = _x(T, H, torch.float32)
    xs = x.double().cpu()
    q = (xs @ w["q_proj.weight"].T + w["q_proj.bias"]).reshape(T, nH, hd)
    k = (xs @ w["k_proj.weight"].T + w["k_proj.bias"]).reshape(T, nKV, hd)
    v = (xs @ w["v_proj.weight"].T + w["v_proj.bias"]).reshape(T, nKV, hd)
    mask = torch.triu(torch.ones(T, T, dtype=torch.bool), 1)
    o = torch.stack([torch.softmax(((q[:, h] @ k[:, h].T) * 0.37).masked_fill(mask, -1e300), -1) @ v[:, h]
                     for h in range(nH)], 1).reshape(T, -1)
    want = o @ w["o_proj.weight"].T + w["o_proj.bias"]
    assert rel_err(_attend(part, x, [T], torch.float32, nKV, hd), want) < 1e-4
    assert rel_err(_attend(part, x, [7, 13], torch.float32, nKV, hd), want) < 1e-4


def test_rope_position_scale():
    """Scaled positions: angle = (pos / scale) * inv_freq."""
    from neurogrid_b200.csrc import ops
    hd, nH = 32, 2
    pos_part = build("position", RopeSpec(hd, 10000.0, "adjacent", scale=4.0), device=DEV)
    pa = pos_part.kernel_args()
    inv, half, scale = pa.inv_freq, pa.half_pairing, pa.pos_scale
    assert scale == 4.0 and not half
    T = 12
    q = _x(T, nH * hd, torch.float32)
    ctx = make_ctx([T], [100], [0], dtype=torch.float32)
    out = torch.empty_like(q)
    ops.rope_cache(q, out, None, None, inv, half, scale, None, None, torch.zeros(1, 1, dtype=torch.int32, device=DEV),
                   ctx.positions, ctx.row_entry, nH, 0, hd, 1e-6, ctx.status)
    want = plain.rope(q.double().cpu().reshape(T, nH, hd), torch.arange(100, 100 + T), 10000.0, "adjacent", scale=4.0)
    assert rel_err(out, want.reshape(T, -1)) < 1e-5


def test_window_edge_is_exact():
    """The key just outside the window carries a score that would dominate: it must not count;
    the key just inside must."""
    from neurogrid_b200.csrc import ops
    nH, nKV, hd, ps, W = 2, 1, 32, 8, 11
    pos = 57
    k = torch.randn(16, nKV, ps, hd, device=DEV) * 0.1
    v = torch.randn(16, nKV, ps, hd, device=DEV)
    table = torch.arange(16, dtype=torch.int32, device=DEV).flip(0).reshape(1, 16).contiguous()
    q = torch.randn(1, nH * hd, device=DEV)
    ctx = make_ctx([1], [pos], [0], dtype=torch.float32)
    outside, inside = pos - W, pos - W + 1

    def put(p, scale):
        k[int(table[0, p // ps]), 0, p % ps] = scale * q[0, :hd]

    out = torch.empty_like(q)
    put(outside, 40.0)
    ops.attention_generic(q, k, v, table, ctx.positions, ctx.row_entry, out, nH, W, 1 / math.sqrt(hd))
    far = v[int(table[0, outside // ps]), 0, outside % ps]
    assert float((out[0, :hd] - far).abs().max()) > 0.1            # not captured by the outside key
    put(outside, 0.0)
    put(inside, 40.0)
    ops.attention_generic(q, k, v, table, ctx.positions, ctx.row_entry, out, nH, W, 1 / math.sqrt(hd))
    near = v[int(table[0, inside // ps]), 0, inside % ps]
    assert torch.allclose(out[0, :hd], near, atol=1e-3)
