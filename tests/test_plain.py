"""The plain implementation checked against itself: hand-computed cases, properties the
formulas must have, and a second, independently structured formulation (token by token with
an explicit cache and conv state) that must give the same logits as the whole-sequence one."""
import math

import pytest
import torch

import plain_lfm2 as plain

F = torch.float64


def test_short_conv_taps_by_hand():
    """H = 1, L = 3, identity projections: c[t] = w0 u[t-2] + w1 u[t-1] + w2 u[t] with zeros
    before the sequence; out = C * c, u = B * x."""
    w_in = torch.tensor([[2.0], [3.0], [5.0]], dtype=F)            # B = 2n, C = 3n, x = 5n
    w_conv = torch.tensor([[[0.1, 0.2, 0.4]]], dtype=F)
    w_out = torch.tensor([[1.0]], dtype=F)
    n = torch.tensor([[1.0], [2.0], [3.0], [4.0]], dtype=F)
    u = [10.0 * v * v for v in (1, 2, 3, 4)]                      # B*x = 10 n^2
    c = [0.4 * u[0], 0.2 * u[0] + 0.4 * u[1], 0.1 * u[0] + 0.2 * u[1] + 0.4 * u[2], 0.1 * u[1] + 0.2 * u[2] + 0.4 * u[3]]
    want = torch.tensor([[3.0 * v * cc] for v, cc in zip((1, 2, 3, 4), c)], dtype=F)
    got = plain.short_conv(n, w_in, None, w_conv, None, w_out, None)
    assert torch.allclose(got, want)
    # biases: in_proj bias shifts B, C, x; conv bias is added before the C gate; out bias after
    got_b = plain.short_conv(n, w_in, torch.tensor([0.0, 1.0, 0.0], dtype=F), w_conv, torch.tensor([0.5], dtype=F),
                             w_out, torch.tensor([7.0], dtype=F))
    want_b = torch.tensor([[(3.0 * v + 1.0) * (cc + 0.5) + 7.0] for v, cc in zip((1, 2, 3, 4), c)], dtype=F)
    assert torch.allclose(got_b, want_b)


def test_rope_pairings_and_properties():
    T, nh, hd = 5, 2, 8
    g = torch.Generator().manual_seed(0)
    x = torch.randn(T, nh, hd, generator=g, dtype=F)
    pos = torch.tensor([0, 1, 7, 100, 1000])
    for pairing in ("adjacent", "half"):
        y = plain.rope(x, pos, 10000.0, pairing)
        assert torch.allclose(y[0], x[0])                                         # position 0: identity
        assert torch.allclose(y.norm(dim=-1), x.norm(dim=-1))                     # a rotation
    # by hand: pair 0 of the adjacent pairing turns by the angle pos * theta^0 = pos
    y = plain.rope(x, pos, 10000.0, "adjacent")
    c, s = math.cos(7.0), math.sin(7.0)
    assert torch.allclose(y[2, 0, 0], x[2, 0, 0] * c - x[2, 0, 1] * s)
    assert torch.allclose(y[2, 0, 1], x[2, 0, 0] * s + x[2, 0, 1] * c)
    # the half pairing is the adjacent one on permuted dims
    perm = torch.tensor([0, 2, 4, 6, 1, 3, 5, 7])
    assert torch.allclose(plain.rope(x[..., perm], pos, 10000.0, "half"), y[..., perm])
    # scores depend on the distance only
    q, k = x[:1].expand(T, nh, hd), x[1:2].expand(T, nh, hd)
    a = (plain.rope(q, torch.tensor([3] * T), 1e4, "adjacent") * plain.rope(k, torch.tensor([1] * T), 1e4, "adjacent")).sum(-1)
    b = (plain.rope(q, torch.tensor([103] * T), 1e4, "adjacent") * plain.rope(k, torch.tensor([101] * T), 1e4, "adjacent")).sum(-1)
    assert torch.allclose(a, b)


def test_rmsnorm_and_swiglu_by_hand():
    x = torch.tensor([[3.0, 4.0]], dtype=F)
    assert torch.allclose(plain.rmsnorm(x, torch.tensor([1.0, 2.0], dtype=F), 0.0),
                          torch.tensor([[3.0 / math.sqrt(12.5), 8.0 / math.sqrt(12.5)]], dtype=F))
    n = torch.tensor([[1.0, -2.0]], dtype=F)
    w1 = torch.tensor([[1.0, 0.0]], dtype=F); w3 = torch.tensor([[0.0, 1.0]], dtype=F); w2 = torch.tensor([[2.0], [0.5]], dtype=F)
    silu1 = 1.0 / (1.0 + math.exp(-1.0))
    assert torch.allclose(plain.swiglu(n, w1, w3, w2), torch.tensor([[2.0 * silu1 * -2.0, 0.5 * silu1 * -2.0]], dtype=F))


def test_ffn_width_rule():
    assert plain.ffn_width(dict(block_ff_dim=12288, block_auto_adjust_ff_dim=True, block_multiple_of=256)) == 8192
    assert plain.ffn_width(dict(block_ff_dim=288, block_auto_adjust_ff_dim=True, block_multiple_of=64)) == 192
    assert plain.ffn_width(dict(block_ff_dim=256, block_auto_adjust_ff_dim=False)) == 256
    assert plain.ffn_width(dict(intermediate_size=100)) == 100


def _incremental(cfg, w, tokens):
    """The same model token by token: explicit key/value lists and conv inputs carried along."""
    H = cfg["hidden_size"]
    eps = cfg.get("norm_eps", cfg.get("rms_norm_eps"))
    nh, nkv = cfg["num_attention_heads"], cfg["num_key_value_heads"]
    hd = cfg.get("head_dim") or H // nh
    L = cfg["conv_L_cache"]
    pairing = cfg.get("rope_pairing", "half")
    kv = {i: ([], []) for i, t in enumerate(cfg["layer_types"]) if t == "full_attention"}
    tail = {i: [torch.zeros(H, dtype=F)] * (L - 1) for i, t in enumerate(cfg["layer_types"]) if t == "conv"}
    out = []
    for pos, tok in enumerate(tokens):
        h = w["model.embed_tokens.weight"][tok]
        for i, kind in enumerate(cfg["layer_types"]):
            p = f"model.layers.{i}."
            n = plain.rmsnorm(h, w[p + "operator_norm.weight"], eps)
            if kind == "conv":
                pr = w[p + "conv.in_proj.weight"] @ n + (w.get(p + "conv.in_proj.bias", 0))
                Bg, Cg, x = pr[:H], pr[H:2 * H], pr[2 * H:]
                hist = tail[i] + [Bg * x]
                wc = w[p + "conv.conv.weight"].reshape(H, L)
                c = sum(wc[:, k] * hist[k] for k in range(L)) + w.get(p + "conv.conv.bias", 0)
                tail[i] = hist[1:]
                m = w[p + "conv.out_proj.weight"] @ (Cg * c) + w.get(p + "conv.out_proj.bias", 0)
            else:
                q = (w[p + "self_attn.q_proj.weight"] @ n).reshape(nh, hd)
                k = (w[p + "self_attn.k_proj.weight"] @ n).reshape(nkv, hd)
                v = (w[p + "self_attn.v_proj.weight"] @ n).reshape(nkv, hd)
                q = plain.rmsnorm(q, w[p + "self_attn.q_layernorm.weight"], eps)
                k = plain.rmsnorm(k, w[p + "self_attn.k_layernorm.weight"], eps)
                pp = torch.tensor([pos])
                q = plain.rope(q[None], pp, cfg["rope_theta"], pairing)[0]
                k = plain.rope(k[None], pp, cfg["rope_theta"], pairing)[0]
                kv[i][0].append(k); kv[i][1].append(v)
                K, V = torch.stack(kv[i][0]), torch.stack(kv[i][1])          # [t, nkv, hd]
                o = torch.empty(nh, hd, dtype=F)
                for hh in range(nh):
                    g = hh // (nh // nkv)
                    sc = (K[:, g] @ q[hh]) / math.sqrt(hd)
                    o[hh] = torch.softmax(sc, 0) @ V[:, g]
                m = w[p + "self_attn.out_proj.weight"] @ o.reshape(-1)
            h = h + m
            n = plain.rmsnorm(h, w[p + "ffn_norm.weight"], eps)
            g1 = w[p + "feed_forward.w1.weight"] @ n
            h = h + w[p + "feed_forward.w2.weight"] @ (g1 / (1 + torch.exp(-g1)) * (w[p + "feed_forward.w3.weight"] @ n))
        n = plain.rmsnorm(h, w["model.embedding_norm.weight"], eps)
        out.append(w.get("lm_head.weight", w["model.embed_tokens.weight"]) @ n)
    return torch.stack(out)


@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_whole_sequence_equals_token_by_token(model_dirs, name):
    cfg, w = plain.load_plain(model_dirs[name])
    g = torch.Generator().manual_seed(3)
    toks = torch.randint(0, cfg["vocab_size"], (23,), generator=g).tolist()
    a = plain.forward(cfg, w, toks)
    b = _incremental(cfg, w, toks)
    assert float((a - b).abs().max() / a.abs().max()) < 1e-12


def test_sampler_mirror():
    lg = torch.tensor([0.0, 1.0, 2.0, 3.0], dtype=F)
    p = plain.sample_probs(lg, 1.0, 1.0)
    assert torch.allclose(p, torch.softmax(lg, 0)) and abs(float(p.sum()) - 1) < 1e-12
    p9 = plain.sample_probs(lg, 1.0, 0.9)                       # 0.64 + 0.24 = 0.88 < 0.9: three tokens stay
    assert float(p9[0]) == 0.0 and abs(float(p9.sum()) - 1) < 1e-12 and float(p9[1]) > 0
    p5 = plain.sample_probs(lg, 1.0, 0.5)                       # the best token alone reaches 0.5
    assert p5.tolist() == [0.0, 0.0, 0.0, 1.0]
    assert plain.sample_from(p, 0.0) == 0 and plain.sample_from(p, 0.999999) == 3
    cold = plain.sample_probs(lg, 0.05, 1.0)
    assert float(cold[3]) > 0.999
