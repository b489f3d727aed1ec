"""Grouped-query attention over paged keys and values."""
from __future__ import annotations

import math

import torch

from ..cache.manager import PagedNeed
from ..csrc import ops
from ..weights.decl import TensorDecl
from . import registry
from .base import PositionArgs
from .registry import register


@register("mixer", "attention")
class Attention:
    """q, k, v projections (stacked into one product at bind time) -> optional per-head
    RMSNorm of q and k -> position encoding -> k, v into the layer's pages -> softmax(q k^T
    * scale) v over the visible keys (all earlier ones, or a window) -> output projection.
    Query head h reads KV head h // (n_heads / n_kv_heads).

    Reference: gpu/engine/layer.cu:1665-1731 (order: norm, rotation, cache), scale and mask
    gpu/cuda/paged_attention.cu:278-387, gpu/cuda/attention.cu:369-500.  ``owns_cache`` False
    builds a layer that only reads another layer's keys and values: it has no k/v weights.
    """

    graph_safe = True      # launches depend on device data and on launch-time constants only

    def __init__(self, spec, *, dtype, device, owns_cache=True):
        self.spec, self.dtype, self.device, self.owns_cache = spec, dtype, device, owns_cache
        self.position = registry.build("position", spec.position, device=device)
        self.scale = spec.softmax_scale if spec.softmax_scale is not None else 1.0 / math.sqrt(spec.head_dim)
        self.w_qkv = self.b_qkv = self.w_o = self.b_o = self.q_norm = self.k_norm = None

    def _proj_names(self):
        return ("q", "k", "v") if self.owns_cache else ("q",)

    def tensors(self):
        s, n = self.spec, self.spec.names
        rows = {"q": s.n_heads * s.head_dim, "k": s.n_kv_heads * s.head_dim, "v": s.n_kv_heads * s.head_dim}
        d = {f"{n[p]}.weight": TensorDecl((rows[p], s.hidden)) for p in self._proj_names()}
        d[f"{n['o']}.weight"] = TensorDecl((s.hidden, s.n_heads * s.head_dim))
        if s.bias:
            for p in self._proj_names():
                d[f"{n[p]}.bias"] = TensorDecl((rows[p],), "bias")
            d[f"{n['o']}.bias"] = TensorDecl((s.hidden,), "bias")
        if s.qk_norm:
            d[f"{n['q_norm']}.weight"] = TensorDecl((s.head_dim,), "norm")
            if self.owns_cache:
                d[f"{n['k_norm']}.weight"] = TensorDecl((s.head_dim,), "norm")
        return d

    def bind(self, t):
        s, n = self.spec, self.spec.names
        kw = dict(device=self.device, dtype=self.dtype)
        f32 = dict(device=self.device, dtype=torch.float32)
        self.w_qkv = torch.cat([t[f"{n[p]}.weight"].to(**kw) for p in self._proj_names()]).contiguous()
        self.w_o = t[f"{n['o']}.weight"].to(**kw).contiguous()
        if s.bias:
            self.b_qkv = torch.cat([t[f"{n[p]}.bias"].to(**kw) for p in self._proj_names()]).contiguous()
            self.b_o = t[f"{n['o']}.bias"].to(**kw).contiguous()
        if s.qk_norm:
            self.q_norm = t[f"{n['q_norm']}.weight"].to(**f32).contiguous()
            if self.owns_cache:
                self.k_norm = t[f"{n['k_norm']}.weight"].to(**f32).contiguous()

    def cache_need(self):
        return PagedNeed(self.spec.n_kv_heads, self.spec.head_dim, self.spec.window)

    def scratch_bytes_per_row(self):
        """Workspace per row of a step besides the products' outputs: the records of the portion kernel's runs."""
        s = self.spec
        if self.dtype != torch.bfloat16 or s.head_dim != 64:
            return 0
        return 4 * ops.attn_prefill_scratch_floats(1, s.n_heads, s.head_dim, PREFILL_MAX_SPLITS)

    def kernels(self):
        s = self.spec
        jobs = [_product_library(self.dtype), ("rope_cache", {"NG_ROPE_PAIRS": ops.rope_pairs(s.head_dim)})]
        if self.dtype == torch.bfloat16 and s.n_heads // s.n_kv_heads <= 16:
            jobs.append(("attention_bf16", {"NG_HEAD_DIM": s.head_dim}))
            if s.head_dim == 64:                             # the tcgen05 kernel for portions (pages of 8..64 tokens)
                jobs.append(("attention_sm100", None))
        else:
            jobs.append(("attention_generic", None))
        return jobs

    def forward(self, x, ctx, cache):
        s = self.spec
        n = x.shape[0]
        writes = cache.writes
        if writes and not self.owns_cache:
            raise RuntimeError("an attention layer without k/v weights cannot write a cache")
        n_kv = s.n_kv_heads if self.owns_cache else 0
        qkv = ops.linear_to_residual(x, self.w_qkv, self.b_qkv, ctx.ws, "attn_qkv")
        q = ctx.ws.buf("attn_q", n, s.n_heads * s.head_dim, self.dtype)
        pa = PositionArgs.of(self.position.kernel_args())
        inv_freq, half, pos_scale = pa.inv_freq, pa.half_pairing, pa.pos_scale
        if self.owns_cache and not writes:
            # has k/v weights but this run reads another cache: q path only
            if qkv.dim() == 3:
                qkv = qkv.sum(0).to(self.dtype)
            qkv_q = ctx.ws.buf("attn_qonly", n, s.n_heads * s.head_dim, self.dtype)
            qkv_q.copy_(qkv[:, : s.n_heads * s.head_dim])
            qkv, n_kv = qkv_q, 0
        ops.rope_cache(qkv, q, self.q_norm, self.k_norm, inv_freq, half, pos_scale,
                       cache.k_pages if n_kv else None, cache.v_pages if n_kv else None, cache.table,
                       ctx.positions, ctx.row_entry, s.n_heads, n_kv, s.head_dim, s.qk_norm_eps, ctx.status)
        a = ctx.ws.buf("attn_out", n, s.n_heads * s.head_dim, self.dtype)
        self.attend(q, cache, ctx, a, pa.score_slopes)
        return ops.linear_to_residual(a, self.w_o, self.b_o, ctx.ws, "mixer_out", residual=ctx.residual)

    def attend(self, q, cache, ctx, out, slopes=None):
        """float32: the order-fixed kernel.  bfloat16: tensor-core kernels, one for portions
        and one (split over the context) for entries that bring a single token.  ``slopes``: the
        position encoding's score bias per head, if it has one."""
        s = self.spec
        if self.dtype != torch.bfloat16 or s.n_heads // s.n_kv_heads > 16:
            ops.attention_generic(q, cache.k_pages, cache.v_pages, cache.table, ctx.positions, ctx.row_entry, out,
                                  s.n_heads, s.window, self.scale, slopes)
            return
        singles = [c + 1 for c, n in zip(ctx.ctx_lens, ctx.q_lens) if n == 1]
        has_multi = any(n > 1 for n in ctx.q_lens)
        if ctx.fixed_launches:                       # a graph that serves every mix of its size: both kernels, always
            has_multi, singles = ctx.max_q > 1, singles or [1]
        if has_multi:
            if ops.attn_prefill_sm100_takes(s.head_dim, cache.k_pages.shape[2]):
                # a launch's graph is kept per class of context (`prefill_ctx`), so the cut of the keys is as fixed as the graph
                if ctx.prefill_ctx:                  # a graph for a class of steps: planned for one portion of max_q rows
                    span, tiles = ctx.prefill_ctx, -(-ctx.max_q // 128)
                else:
                    span = max(c + n for c, n in zip(ctx.ctx_lens, ctx.q_lens) if n > 1)
                    tiles = sum(-(-n // 128) for n in ctx.q_lens if n > 1 or not singles)
                n_splits = prefill_splits(tiles * s.n_heads, min(span, s.window) if s.window else span, self.device)
                floats = ops.attn_prefill_scratch_floats(q.shape[0], s.n_heads, s.head_dim, n_splits)
                scratch = None
                if floats or ctx.ws.fixed:
                    bound = ops.attn_prefill_scratch_floats(ctx.ws.max_rows, s.n_heads, s.head_dim, PREFILL_MAX_SPLITS)
                    scratch = ctx.ws.flat("attn_prefill_scratch", floats, torch.float32, reserve=bound)
                ops.attn_prefill_sm100(q, cache.k_pages, cache.v_pages, cache.table, ctx.cu_q, ctx.ctx_before, out,
                                       ctx.n_entries, ctx.max_q, s.n_heads, s.window, self.scale, bool(singles), slopes,
                                       scratch, n_splits)
            else:
                ops.attn_prefill_bf16(q, cache.k_pages, cache.v_pages, cache.table, ctx.cu_q, ctx.ctx_before, out,
                                      ctx.n_entries, ctx.max_q, s.n_heads, s.window, self.scale, bool(singles), slopes)
        if singles:
            max_ctx = ctx.decode_max_ctx or max(singles)
            n_splits = decode_splits(ctx.decode_batch or len(singles), s.n_kv_heads, max_ctx, s.window, self.device)
            floats = ops.attn_decode_scratch_floats(q.shape[0], s.n_heads, s.head_dim, n_splits)
            scratch = None
            if floats or ctx.ws.fixed:
                # upper bound over every batch size: splits <= 3 * SMs / (rows * n_kv_heads) + 1, or 2, or
                # what the longest context a request can have asks (one per 2,048 keys)
                per_row = max(2, -(-(cache.table.shape[1] * cache.k_pages.shape[2]) // 2048))
                bound = (3 * sm_count(self.device) // s.n_kv_heads + per_row * ctx.ws.max_rows + 2) * s.n_heads * (s.head_dim + 2)
                scratch = ctx.ws.flat("attn_split_scratch", floats, torch.float32, reserve=bound)
            ops.attn_decode_bf16(q, cache.k_pages, cache.v_pages, cache.table, ctx.cu_q, ctx.ctx_before, out,
                                 scratch, ctx.n_entries, s.n_heads, s.window, self.scale, n_splits, max_ctx, slopes)


def _product_library(dtype):
    return ("gemm_sm100", None) if dtype == torch.bfloat16 else ("gemm_f32", None)


_SM_COUNT = {}


def sm_count(device) -> int:
    key = str(device)
    if key not in _SM_COUNT:
        _SM_COUNT[key] = torch.cuda.get_device_properties(device).multi_processor_count
    return _SM_COUNT[key]


PREFILL_MAX_SPLITS = 4
PREFILL_SPLIT_MIN_CTX = 8192        # keys a portion sees before its blocks are worth cutting (the merge costs a pass)


def prefill_splits(n_blocks: int, span: int, device) -> int:
    """Runs the keys of every block of the portion kernel are cut into.  The kernel keeps two
    blocks on an SM; `n_blocks` blocks of about equal length take ceil(n_blocks / slots) rounds,
    the last of them partly empty (24 heads x 16 row tiles = 384 blocks on 296 slots: 1.3 rounds
    cost 2).  Cutting each block into 2..4 runs makes the rounds finer.  Worth it only where the
    blocks are long (`span` keys: the merge of the runs is one more pass over the output in
    float32) and few (many rounds are even enough), and where the filling improves by a tenth."""
    if span < PREFILL_SPLIT_MIN_CTX or n_blocks <= 0:
        return 1
    slots = 2 * sm_count(device)

    def filling(blocks):
        return blocks / (slots * -(-blocks // slots))

    best, best_f = 1, filling(n_blocks)
    for n in range(2, PREFILL_MAX_SPLITS + 1):
        if span // (64 * n) < 16:                # the kernel does not cut runs shorter than 16 tiles
            break
        f = filling(n_blocks * n) - 0.02 * (n - 1)
        if f > best_f + 0.08:
            best, best_f = n, f
    return best


def decode_splits(n_single: int, n_kv_heads: int, max_ctx: int, window, device) -> int:
    """Splits of the context for the single-token entries: about three blocks per SM, at least
    two when the context is long (a lone block per (entry, KV head) leaves the tail of the
    launch unbalanced), no split longer than 2,048 keys and none shorter than 256.
    Measured on a B200 over batch 1..64 and contexts 600..32,000 (32 / 8 heads of 64): within
    about 10 % of the best split count of each shape, except where the number of blocks falls
    just above a whole number of waves."""
    span = min(window, max_ctx) if window else max_ctx
    pairs = max(1, n_single * n_kv_heads)
    want = max(-(-3 * sm_count(device) // pairs), 2 if span >= 1024 else 1, -(-span // 2048))
    return max(1, min(want, span // 256))
