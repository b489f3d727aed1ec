"""Plain PyTorch statements of what each CUDA launcher computes, with the launchers' signatures.

Used two ways: the GPU tests compare every kernel with its function here, and the CPU tests
install these functions in place of the launchers (``install(monkeypatch)``) so that the host
side of the engine (batch packing, cache, scheduling) can be exercised where there is no GPU.
They are test code only: the product has no CPU path.
Math is float64 inside; outputs are rounded once to the output tensor's dtype.
"""
from __future__ import annotations

import math

import torch

D = torch.float64


def embed(table, tokens, out, status, accumulate=False):
    tok = tokens.long()
    bad = (tok < 0) | (tok >= table.shape[0])
    if bad.any():
        status |= 4 if accumulate else 1
    rows = table[tok.clamp(0, table.shape[0] - 1)].to(torch.float32)
    rows[bad] = 0
    out.copy_(out + rows if accumulate else rows)


def gather_tokens(dst, src, idx):
    m = idx >= 0
    dst[m] = src[idx[m].long()]


def add_rmsnorm(h, delta, weight, out, eps, rows=None):
    idx = torch.arange(out.shape[0], device=h.device) if rows is None else rows.long()
    if delta is not None:
        if delta.dim() == 3:                                  # a stack of float32 partial sums
            delta = delta.to(D).sum(0)
        h[idx] = (h[idx].to(D) + delta[idx].to(D)).to(torch.float32)
    x = h[idx].to(D)
    y = x * torch.rsqrt((x * x).mean(-1, keepdim=True) + eps) * weight.to(D)
    out.copy_(y.to(out.dtype))


def residual_add(h, delta):
    if delta.dim() == 3:
        delta = delta.to(D).sum(0)
    h.copy_((h.to(D) + delta.to(D)).to(torch.float32))


def swiglu(gate_up, out):
    I = out.shape[1]
    g, u = gate_up[:, :I].to(D), gate_up[:, I:].to(D)
    out.copy_((g / (1 + torch.exp(-g)) * u).to(out.dtype))


def gemm_f32(a, w, bias, out):
    r = a.to(D) @ w.to(D).T
    if bias is not None:
        r = r + bias.to(D)
    out.copy_(r.to(out.dtype))


def linear(x, weight, bias, out):
    gemm_f32(x, weight, bias, out)


def shortconv(p, weight, bias, state, out, cu_q, ctx_before, slots, n_entries, max_q):
    H = out.shape[1]
    L = weight.shape[1]
    if p.dim() == 3:                                          # float32 partial sums, rounded where the product would be
        p = p.to(D).sum(0).to(out.dtype)
    cu = cu_q.tolist()
    for e in range(n_entries):
        q0, q1 = cu[e], cu[e + 1]
        if q1 == q0:
            continue
        ctx, slot = int(ctx_before[e]), int(slots[e])
        rows = p[q0:q1].to(D)
        Bg, Cg, x = rows[:, :H], rows[:, H:2 * H], rows[:, 2 * H:]
        u_new = Bg * x
        old = state[slot].to(D).clone()                       # [L-1, H], positions ctx-(L-1)..ctx-1
        for j in range(L - 1):
            if ctx - (L - 1) + j < 0:
                old[j] = 0
        u = torch.cat([old, u_new])                           # index i <-> chunk index i-(L-1)
        c = torch.zeros(q1 - q0, H, dtype=D, device=p.device)
        for k in range(L):
            c += weight[:, k].to(D) * u[k:k + (q1 - q0)]
        if bias is not None:
            c = c + bias.to(D)
        out[q0:q1] = (Cg * c).to(out.dtype)
        state[slot] = u[-(L - 1):].to(torch.float32)


def rope_cache(qkv, q_out, q_weight, k_weight, inv_freq, half_pairing, pos_scale, k_pages, v_pages, table,
               positions, row_entry, n_heads, n_kv_heads, head_dim, eps, status):
    if qkv.dim() == 3:
        qkv = qkv.to(D).sum(0).to(q_out.dtype)
    n = qkv.shape[0]
    hd = head_dim
    x = qkv.to(D)
    q = x[:, : n_heads * hd].reshape(n, n_heads, hd)
    k = x[:, n_heads * hd:(n_heads + n_kv_heads) * hd].reshape(n, n_kv_heads, hd)
    v = x[:, (n_heads + n_kv_heads) * hd:].reshape(n, n_kv_heads, hd)

    def norm(t, w):
        return t * torch.rsqrt((t * t).mean(-1, keepdim=True) + eps) * w.to(D)

    def rot(t):
        if inv_freq is None:
            return t
        ang = ((positions.to(torch.float32) / pos_scale)[:, None] * inv_freq[None, :]).to(D)   # float32 angle
        c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
        o = torch.empty_like(t)
        if half_pairing:
            a, b = t[..., : hd // 2], t[..., hd // 2:]
            o[..., : hd // 2], o[..., hd // 2:] = a * c - b * s, a * s + b * c
        else:
            a, b = t[..., 0::2], t[..., 1::2]
            o[..., 0::2], o[..., 1::2] = a * c - b * s, a * s + b * c
        return o

    if q_weight is not None:
        q = norm(q, q_weight)
        if n_kv_heads:
            k = norm(k, k_weight)
    q, k = rot(q), (rot(k) if n_kv_heads else k)
    valid = row_entry >= 0
    qo = q.reshape(n, -1).to(q_out.dtype)
    qo[~valid] = 0
    q_out.copy_(qo)
    if n_kv_heads:
        ps = k_pages.shape[2]
        for r in range(n):
            if not bool(valid[r]):
                continue
            pos = int(positions[r])
            page = int(table[int(row_entry[r]), pos // ps])
            if page < 0 or page >= k_pages.shape[0]:
                status |= 2
                continue
            k_pages[page, :, pos % ps] = k[r].to(k_pages.dtype)
            v_pages[page, :, pos % ps] = v[r].to(v_pages.dtype)


def attention_generic(q, k_pages, v_pages, table, positions, row_entry, out, n_heads, window, scale, slopes=None):
    n = q.shape[0]
    P, n_kv, ps, hd = k_pages.shape
    group = n_heads // n_kv
    for r in range(n):
        e = int(row_entry[r])
        if e < 0:
            out[r] = 0
            continue
        pos = int(positions[r])
        lo = max(0, pos - window + 1) if window else 0
        kp = torch.arange(lo, pos + 1, device=q.device)
        pages = table[e, kp // ps].long()
        K = k_pages[pages, :, kp % ps].to(D)             # [keys, n_kv, hd]
        Vv = v_pages[pages, :, kp % ps].to(D)
        qr = q[r].to(D).reshape(n_heads, hd)
        o = torch.empty(n_heads, hd, dtype=D, device=q.device)
        for h in range(n_heads):
            s = (K[:, h // group] @ qr[h]) * scale
            if slopes is not None:
                s = s - float(slopes[h]) * (pos - kp).to(D)
            o[h] = torch.softmax(s, 0) @ Vv[:, h // group]
        out[r] = o.reshape(-1).to(out.dtype)


def sample(logits, temperature, top_p, uniform, out, scratch):
    W, V = logits.shape
    for r in range(W):
        lg = logits[r].to(D)
        t = float(temperature[r]) if temperature is not None else 0.0
        if not t > 0:
            out[r] = int(torch.argmax(lg))
            continue
        e = torch.exp((lg - lg.max()) / t)
        p = float(top_p[r]) if top_p is not None else 1.0
        if 0 < p < 1:
            vals = torch.sort(e, descending=True).values
            cs = torch.cumsum(vals, 0)
            cut = int(torch.nonzero(cs >= p * e.sum())[0]) if (cs >= p * e.sum()).any() else V - 1
            e = torch.where(e >= vals[cut], e, torch.zeros_like(e))
        c = torch.cumsum(e, 0)
        target = float(uniform[r]) * float(c[-1])
        hit = torch.nonzero(target < c)
        out[r] = int(hit[0]) if len(hit) else int(torch.argmax(lg))


_NAMES = ["gather_tokens", "embed", "add_rmsnorm", "residual_add", "swiglu", "gemm_f32", "linear", "shortconv", "rope_cache",
          "attention_generic", "sample"]


def install(monkeypatch):
    """Replace the launchers of ``neurogrid_b200.csrc.ops`` with the functions above."""
    from neurogrid_b200.csrc import ops
    for n in _NAMES:
        monkeypatch.setattr(ops, n, globals()[n])


def _rows_of(cu_q, single: bool):
    cu = cu_q.tolist()
    rows, entries = [], []
    for e in range(len(cu) - 1):
        n = cu[e + 1] - cu[e]
        if (n == 1) == single and n > 0:
            rows += list(range(cu[e], cu[e + 1]))
            entries += [e] * n
    return rows, entries


def _attend_rows(q, k_pages, v_pages, table, cu_q, ctx_before, out, n_heads, window, scale, single, slopes=None):
    rows, entries = _rows_of(cu_q, single)
    cu = cu_q.tolist()
    n = q.shape[0]
    pos = torch.zeros(n, dtype=torch.int32, device=q.device)
    re = torch.full((n,), -1, dtype=torch.int32, device=q.device)
    for r, e in zip(rows, entries):
        pos[r] = int(ctx_before[e]) + (r - cu[e])
        re[r] = e
    tmp = out.clone()
    attention_generic(q, k_pages, v_pages, table, pos, re, tmp, n_heads, window, scale, slopes)
    for r in rows:
        out[r] = tmp[r]


def attn_prefill_bf16(q, k_pages, v_pages, table, cu_q, ctx_before, out, n_entries, max_q, n_heads, window, scale,
                      skip_single, slopes=None):
    _attend_rows(q, k_pages, v_pages, table, cu_q, ctx_before, out, n_heads, window, scale, False, slopes)
    if not skip_single:
        _attend_rows(q, k_pages, v_pages, table, cu_q, ctx_before, out, n_heads, window, scale, True, slopes)


def attn_decode_bf16(q, k_pages, v_pages, table, cu_q, ctx_before, out, scratch, n_entries, n_heads, window, scale,
                     n_splits, max_ctx, slopes=None):
    _attend_rows(q, k_pages, v_pages, table, cu_q, ctx_before, out, n_heads, window, scale, True, slopes)


def attn_prefill_sm100(q, k_pages, v_pages, table, cu_q, ctx_before, out, n_entries, max_q, n_heads, window, scale,
                       skip_single, slopes=None, scratch=None, n_splits=1):
    attn_prefill_bf16(q, k_pages, v_pages, table, cu_q, ctx_before, out, n_entries, max_q, n_heads, window, scale,
                      skip_single, slopes)


_NAMES += ["attn_prefill_bf16", "attn_decode_bf16", "attn_prefill_sm100"]
# ops.linear_to_residual is host logic over ops.linear: it is not replaced
