"""A plain, slow implementation of the LFM2 decoder: whole sequences, no cache, float64.

It is written from the reference's formulas; each function cites the reference lines it restates.
The reference's LFM2 math lives in CUDA files and cuBLAS calls (its non-CUDA build is a stub,
gpu/bindings/gpu_stub.go:17), so it cannot be imported or run on a CPU; it was run once on a GPU
instead, through its own library's stock entry points, on the Tiny A model, and
``tests/test_golden_reference.py`` holds this file to the logits it returned
(``tests/golden/reference_tiny_a.npz``, made by ``tests/golden/make_reference_golden.py``).  Nothing here is shared with the
product: the config is parsed here, weights are read with the ``safetensors`` package, and
every part is one function over a whole sequence.

``round_bf16=True`` rounds to bfloat16 at the places where the engine's bfloat16 path
stores an activation (matrix-product outputs, norm outputs, the gated conv output, q, the
cached k and v, the attention output, the SwiGLU product); sums, norms, softmax, angles and
the residual stream stay wide, as in the engine.
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional, Sequence

import torch

F = torch.float64


def _r(t: torch.Tensor, on: bool) -> torch.Tensor:
    return t.to(torch.bfloat16).to(F) if on else t


# ----------------------------------------------------------------------------- config
def ffn_width(cfg: dict) -> int:
    """cmd/neurogrid/main.go:831-841: 2/3 of block_ff_dim rounded up to a multiple (256 there;
    the key block_multiple_of here), applied when block_auto_adjust_ff_dim is set."""
    ff = cfg.get("block_ff_dim", cfg.get("intermediate_size"))
    if not cfg.get("block_auto_adjust_ff_dim", False):
        return ff
    d = int(2 * ff / 3)
    d = int(cfg.get("block_ffn_dim_multiplier", 1.0) * d)
    m = cfg["block_multiple_of"]
    return ((d + m - 1) // m) * m


def load_plain(model_dir: str):
    from safetensors.torch import load_file
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    w = {k: v.to(F) for k, v in load_file(os.path.join(model_dir, "model.safetensors")).items()}
    return cfg, w


# ----------------------------------------------------------------------------- parts
def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """gpu/cuda/bf16_utils.cu:57-93: y = x * rsqrt(mean(x^2) + eps) * w (weight direct, no 1+w)."""
    return x * torch.rsqrt((x * x).mean(-1, keepdim=True) + eps) * w


def rope(x: torch.Tensor, positions: torch.Tensor, theta: float, pairing: str, scale: float = 1.0) -> torch.Tensor:
    """gpu/cuda/bf16_utils.cu:330-378: inv_freq_i = theta^(-2i/hd), angle = pos * inv_freq_i,
    x1' = x1 cos - x2 sin, x2' = x1 sin + x2 cos; pairs (2i, 2i+1) ("adjacent", style 1, the
    reference engine's choice for this family, pkg/model/model_config.go:93-99) or (i, i + hd/2)
    ("half", style 0, the checkpoint format's, which the reference's golden data comes from:
    scripts/generate_golden_lfm2.py:37-93).
    x: [T, heads, hd]."""
    hd = x.shape[-1]
    i = torch.arange(hd // 2, dtype=F)
    inv_freq = theta ** (-2.0 * i / hd)
    ang = (positions.to(F) / scale)[:, None] * inv_freq[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    out = torch.empty_like(x)
    if pairing == "adjacent":
        x1, x2 = x[..., 0::2], x[..., 1::2]
        out[..., 0::2] = x1 * c - x2 * s
        out[..., 1::2] = x1 * s + x2 * c
    else:
        x1, x2 = x[..., : hd // 2], x[..., hd // 2:]
        out[..., : hd // 2] = x1 * c - x2 * s
        out[..., hd // 2:] = x1 * s + x2 * c
    return out


def short_conv(n: torch.Tensor, w_in, b_in, w_conv, b_conv, w_out, b_out, rb: bool = False) -> torch.Tensor:
    """gpu/engine/conv_layer.cu:222-250,325: p = n W_in^T; B, C, x = p[:, :H], p[:, H:2H], p[:, 2H:];
    u = B*x; causal depthwise conv (gpu/cuda/conv.cu:52-66: c[t] = sum_k w[d,k] u[t-(L-1)+k], zero
    before the sequence); g = C*c; out = g W_out^T.  Biases (absent in the reference) are added
    to each of the three parametrised parts, the conv's before the C gate.  n: [T, H]."""
    T, H = n.shape
    L = w_conv.shape[-1]
    p = n @ w_in.T
    if b_in is not None:
        p = p + b_in
    p = _r(p, rb)
    Bg, Cg, x = p[:, :H], p[:, H:2 * H], p[:, 2 * H:]
    u = Bg * x
    wc = w_conv.reshape(H, L)
    c = torch.zeros(T, H, dtype=F)
    for t in range(T):
        for k in range(L):
            src = t - (L - 1) + k
            if src >= 0:
                c[t] += wc[:, k] * u[src]
    if b_conv is not None:
        c = c + b_conv
    g = _r(Cg * c, rb)
    out = g @ w_out.T
    if b_out is not None:
        out = out + b_out
    return _r(out, rb)


def attention(n: torch.Tensor, wq, wk, wv, wo, q_norm_w, k_norm_w, *, n_heads: int, n_kv: int, hd: int,
              eps: float, theta: float, pairing: str, positions: Optional[torch.Tensor] = None,
              window: Optional[int] = None, rb: bool = False) -> torch.Tensor:
    """gpu/engine/layer.cu:1665-1731: q, k, v projections; per-head RMSNorm over hd on q and k
    (weights shared by the heads, layer.cu:1323-1366); rotation; scores q.k / sqrt(hd) with keys
    after the query masked, softmax, weighted sum of v (gpu/cuda/paged_attention.cu:278-387);
    query head h reads KV head h // (n_heads / n_kv); output projection.  n: [T, H]."""
    T = n.shape[0]
    pos = torch.arange(T) if positions is None else positions
    q = _r(n @ wq.T, rb).reshape(T, n_heads, hd)
    k = _r(n @ wk.T, rb).reshape(T, n_kv, hd)
    v = _r(n @ wv.T, rb).reshape(T, n_kv, hd)
    if q_norm_w is not None:
        q = rmsnorm(q, q_norm_w, eps)
        k = rmsnorm(k, k_norm_w, eps)
    q = _r(rope(q, pos, theta, pairing), rb)
    k = _r(rope(k, pos, theta, pairing), rb)
    out = torch.zeros(T, n_heads, hd, dtype=F)
    group = n_heads // n_kv
    for h in range(n_heads):
        kh = h // group
        s = (q[:, h] @ k[:, kh].T) / math.sqrt(hd)
        qi, ki = pos[:, None], pos[None, :]
        mask = ki > qi
        if window is not None:
            mask = mask | (ki <= qi - window)
        s = s.masked_fill(mask, float("-inf"))
        out[:, h] = torch.softmax(s, dim=-1) @ v[:, kh]
    out = _r(out.reshape(T, n_heads * hd), rb)
    return _r(out @ wo.T, rb)


def swiglu(n: torch.Tensor, w1, w3, w2, rb: bool = False) -> torch.Tensor:
    """gpu/engine/conv_layer.cu:334-338, layer.cu:1751-1761: (silu(n W1^T) * (n W3^T)) W2^T,
    silu(z) = z / (1 + exp(-z))."""
    g, u = _r(n @ w1.T, rb), _r(n @ w3.T, rb)
    a = _r(g / (1.0 + torch.exp(-g)) * u, rb)
    return _r(a @ w2.T, rb)


# ----------------------------------------------------------------------------- whole model
def forward(cfg: dict, w: Dict[str, torch.Tensor], tokens: Sequence[int], round_bf16: bool = False,
            rows: Optional[Sequence[int]] = None) -> torch.Tensor:
    """Logits [T, V] for one whole sequence (or of the positions ``rows`` only: the head of a
    large vocabulary is most of the work).  Layer skeleton r = x + mixer(norm(x)),
    y = r + ffn(norm(r)) (gpu/engine/conv_layer.cu:220,328-341; layer.cu:1662-1765); final
    norm model.embedding_norm then the head, tied to the embedding unless lm_head.weight exists
    (pkg/inference/engine_gpu.go:73-88, pkg/model/loader.go:591-600).  A ``sliding_window`` key
    (no LFM2 configuration has one; the tests' windowed toy model does) limits every attention
    layer to that many keys, the query's own included."""
    rb = round_bf16
    H = cfg["hidden_size"]
    eps = cfg.get("norm_eps", cfg.get("rms_norm_eps"))
    n_heads, n_kv = cfg["num_attention_heads"], cfg["num_key_value_heads"]
    hd = cfg.get("head_dim") or H // n_heads
    tok = torch.as_tensor(list(tokens), dtype=torch.long)
    h = w["model.embed_tokens.weight"][tok]                      # pkg/model/loader.go:586-588
    for i, kind in enumerate(cfg["layer_types"]):
        p = f"model.layers.{i}."
        n = _r(rmsnorm(h, w[p + "operator_norm.weight"], eps), rb)
        if kind == "conv":
            m = short_conv(n, w[p + "conv.in_proj.weight"], w.get(p + "conv.in_proj.bias"),
                           w[p + "conv.conv.weight"], w.get(p + "conv.conv.bias"),
                           w[p + "conv.out_proj.weight"], w.get(p + "conv.out_proj.bias"), rb)
        else:
            m = attention(n, w[p + "self_attn.q_proj.weight"], w[p + "self_attn.k_proj.weight"],
                          w[p + "self_attn.v_proj.weight"], w[p + "self_attn.out_proj.weight"],
                          w[p + "self_attn.q_layernorm.weight"], w[p + "self_attn.k_layernorm.weight"],
                          n_heads=n_heads, n_kv=n_kv, hd=hd, eps=eps, theta=cfg["rope_theta"],
                          pairing=cfg.get("rope_pairing", "half"), window=cfg.get("sliding_window"), rb=rb)
        h = h + m
        n = _r(rmsnorm(h, w[p + "ffn_norm.weight"], eps), rb)
        h = h + swiglu(n, w[p + "feed_forward.w1.weight"], w[p + "feed_forward.w3.weight"],
                       w[p + "feed_forward.w2.weight"], rb)
    if rows is not None:
        h = h[torch.as_tensor(list(rows), dtype=torch.long)]
    n = _r(rmsnorm(h, w["model.embedding_norm.weight"], eps), rb)
    head = w.get("lm_head.weight", w["model.embed_tokens.weight"])
    return n @ head.T


def generate_greedy(cfg, w, prompt: Sequence[int], n_new: int, round_bf16: bool = False) -> List[int]:
    """Argmax decoding, first index on ties (pkg/inference/sampler.go:58-73); the whole
    sequence is recomputed for every token."""
    seq = list(prompt)
    for _ in range(n_new):
        seq.append(int(torch.argmax(forward(cfg, w, seq, round_bf16)[-1]).item()))
    return seq[len(prompt):]


# ----------------------------------------------------------------------------- sampling
def sample_probs(logits: torch.Tensor, temperature: float, top_p: float) -> torch.Tensor:
    """pkg/inference/sampler.go:25-51,114-149: softmax(logits / T); for 0 < top_p < 1 keep the
    most probable tokens through the first cumulative sum >= top_p, renormalise."""
    p = torch.softmax(logits.to(F) / temperature, dim=-1)
    if 0.0 < top_p < 1.0:
        sp, idx = torch.sort(p, descending=True, stable=True)
        cut = int(torch.nonzero(torch.cumsum(sp, 0) >= top_p)[0].item()) if (torch.cumsum(sp, 0) >= top_p).any() \
            else len(sp) - 1
        keep = torch.zeros_like(p)
        keep[idx[: cut + 1]] = sp[: cut + 1]
        p = keep / keep.sum()
    return p


def sample_from(p: torch.Tensor, u: float) -> int:
    """pkg/inference/sampler.go:170-189: the first index whose cumulative probability exceeds u."""
    c = torch.cumsum(p, 0)
    hit = torch.nonzero(u < c)
    return int(hit[0].item()) if len(hit) else len(p) - 1
