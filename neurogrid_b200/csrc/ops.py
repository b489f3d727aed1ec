"""Python faces of the CUDA launchers: tensors in, one kernel launch out.

Every function checks devices, dtypes and layout, passes raw pointers and the current
stream to the C launcher, and raises on a refused size.  There is no CPU path: a tensor
that is not on a CUDA device is an error, and so is a missing compiler or library.
Shapes in the docstrings use N = rows (tokens) of the step, R = entries (requests) of the
step, H = model width.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

from . import build

_c_int, _c_float, _c_void_p, _c_ll = ctypes.c_int, ctypes.c_float, ctypes.c_void_p, ctypes.c_longlong

_ERR = {1: "a size the kernel does not take", 2: "the launch failed", 3: "a dtype the kernel does not take"}


class KernelError(RuntimeError):
    pass


def _check(rc: int, what: str) -> None:
    if rc != 0:
        detail = ""
        if rc == 2:
            detail = f" ({torch.cuda.get_device_name()}: the kernels are built for sm_100a only)"
        raise KernelError(f"{what}: {_ERR.get(rc, rc)}{detail}")


def _ptr(t: Optional[torch.Tensor], what: str = "tensor") -> Optional[int]:
    if t is None:
        return None
    if not t.is_cuda:
        raise KernelError(f"{what} is on {t.device}: neurogrid_b200 kernels run on a CUDA device only "
                          "(there is no CPU path)")
    if not t.is_contiguous():
        raise KernelError(f"{what} must be contiguous")
    return t.data_ptr()


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_current_device = getattr(torch._C, "_cuda_getDevice", None)


def _stream() -> int:
    """The current stream's handle (the capture stream while a graph is being captured).  Asked
    from the C layer directly: a step launches a hundred kernels and more, and building a
    stream object for each costs as much as the launch."""
    if _raw_stream is not None and _current_device is not None:
        return _raw_stream(_current_device())
    return torch.cuda.current_stream().cuda_stream


def _act_flag(t: torch.Tensor, what: str) -> int:
    if t.dtype == torch.bfloat16:
        return 1
    if t.dtype == torch.float32:
        return 0
    raise KernelError(f"{what} has dtype {t.dtype}; the kernels take float32 or bfloat16")


def _f32(t: Optional[torch.Tensor], what: str):
    if t is not None and t.dtype != torch.float32:
        raise KernelError(f"{what} must be float32, got {t.dtype}")
    return t


def _i32(t: Optional[torch.Tensor], what: str):
    if t is not None and t.dtype != torch.int32:
        raise KernelError(f"{what} must be int32, got {t.dtype}")
    return t


_fn_cache = {}


def _fn(lib_name: str, symbol: str, argtypes, defines=None):
    key = (lib_name, symbol, tuple(sorted((defines or {}).items())))
    f = _fn_cache.get(key)
    if f is None:
        f = getattr(build.load(lib_name, defines), symbol)
        f.argtypes = argtypes
        f.restype = _c_int
        _fn_cache[key] = f
    return f


# ----------------------------------------------------------------------------- elementwise
def embed(table: torch.Tensor, tokens: torch.Tensor, out: torch.Tensor, status: torch.Tensor,
          accumulate: bool = False) -> None:
    """out[N,H] (float32) = table[tokens]; a token outside the table gives zeros and a status bit.
    ``accumulate``: out += table[tokens] instead (``tokens`` are then positions into a table of
    learned positions; one outside the table sets the bad-position bit)."""
    n, H = out.shape
    V = table.shape[0]
    f = _fn("elementwise", "ng_embed", [_c_void_p, _c_int, _c_void_p, _c_void_p, _c_int, _c_int, _c_int,
                                       _c_void_p, _c_int, _c_int, _c_void_p])
    _f32(out, "embed out"), _i32(tokens, "tokens"), _i32(status, "status")
    _check(f(_ptr(table, "embedding table"), _act_flag(table, "embedding table"), _ptr(tokens), _ptr(out),
             n, H, V, _ptr(status), int(accumulate), 4 if accumulate else 1, _stream()), "embed")


def _partials(delta: Optional[torch.Tensor], h: torch.Tensor, act: int):
    """(delta_f32, n_partials, stride): ``delta`` is [N,H] of the activation dtype, or a stack
    [S,N,H] of float32 partial sums (split-K products) that are added in ascending order."""
    if delta is None:
        return 0, 1, 0
    if delta.dim() == 3:
        if delta.dtype != torch.float32 or delta.shape[1:] != h.shape:
            raise KernelError("a stack of partial sums must be float32 [S, N, H]")
        return 1, delta.shape[0], delta.shape[1] * delta.shape[2]
    if delta.shape != h.shape or _act_flag(delta, "delta") != act:
        raise KernelError("delta must have the residual stream's shape and the activation dtype")
    return (1 if delta.dtype == torch.float32 else 0), 1, 0


def gather_tokens(dst: torch.Tensor, src: torch.Tensor, idx: torch.Tensor) -> None:
    """dst[i] = src[idx[i]] where idx[i] >= 0 (int32 all): device-sampled tokens into a step's tokens."""
    _i32(dst, "dst"), _i32(src, "src"), _i32(idx, "idx")
    f = _fn("elementwise", "ng_gather_i32", [_c_void_p, _c_void_p, _c_void_p, _c_int, _c_void_p])
    _check(f(_ptr(dst), _ptr(src), _ptr(idx), dst.numel(), _stream()), "gather_tokens")


def add_rmsnorm(h: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, out: torch.Tensor,
                eps: float, rows: Optional[torch.Tensor] = None) -> None:
    """h[N,H] float32 (+= delta if given); out[i] = rmsnorm(h[rows[i] if rows else i]) * weight.
    ``delta`` may be a float32 stack [S,N,H] of partial sums."""
    n_out, H = out.shape
    act = _act_flag(out, "norm out")
    _f32(h, "residual stream"), _f32(weight, "norm weight"), _i32(rows, "rows")
    d32, n_part, stride = _partials(delta, h, act)
    f = _fn("elementwise", "ng_add_rmsnorm", [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int,
                                             _c_int, _c_float, _c_int, _c_int, _c_int, _c_ll, _c_void_p])
    _check(f(_ptr(h), _ptr(delta), _ptr(weight), _ptr(out), _ptr(rows), n_out, H, float(eps), act, d32, n_part,
             stride, _stream()), "add_rmsnorm")


def residual_add(h: torch.Tensor, delta: torch.Tensor) -> None:
    """h (float32) += delta (or the sum of a float32 stack [S,N,H])."""
    _f32(h, "residual stream")
    n_part = delta.shape[0] if delta.dim() == 3 else 1
    f = _fn("elementwise", "ng_residual_add", [_c_void_p, _c_void_p, _c_ll, _c_int, _c_int, _c_void_p])
    _check(f(_ptr(h), _ptr(delta), h.numel(), int(delta.dtype == torch.bfloat16), n_part, _stream()), "residual_add")


def swiglu(gate_up: torch.Tensor, out: torch.Tensor) -> None:
    """out[N,I] = silu(gate_up[:, :I]) * gate_up[:, I:]."""
    n, I = out.shape
    if gate_up.shape != (n, 2 * I) or gate_up.dtype != out.dtype:
        raise KernelError(f"swiglu: gate_up {tuple(gate_up.shape)} does not match out {tuple(out.shape)}")
    f = _fn("elementwise", "ng_swiglu", [_c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_void_p])
    _check(f(_ptr(gate_up), _ptr(out), n, I, _act_flag(out, "swiglu out"), _stream()), "swiglu")


# ----------------------------------------------------------------------------- float32 product
def gemm_f32(a: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor) -> None:
    """out[M,N] = a[M,K] @ w[N,K]^T (+ bias), float32 throughout, FFMA only."""
    M, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K or out.shape != (M, N):
        raise KernelError(f"gemm_f32: a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)} do not fit")
    _f32(a, "a"), _f32(w, "w"), _f32(bias, "bias"), _f32(out, "out")
    f = _fn("gemm_f32", "ng_gemm_f32", [_c_void_p] * 4 + [_c_int] * 6 + [_c_void_p])
    _check(f(_ptr(a), _ptr(w), _ptr(bias), _ptr(out), M, N, K, K, K, N, _stream()), "gemm_f32")


# ----------------------------------------------------------------------------- short convolution
def shortconv(p: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], state: torch.Tensor,
              out: torch.Tensor, cu_q: torch.Tensor, ctx_before: torch.Tensor, slots: torch.Tensor,
              n_entries: int, max_q: int) -> None:
    """p[N,3H] = B|C|x (or a float32 stack [S,N,3H] of partial sums); out[N,H] = C * conv(B*x);
    state[slots, L-1, H] float32 carries B*x."""
    n, H = out.shape
    L = weight.shape[1]
    n_part, stride = _stack(p, (n, 3 * H), out.dtype, "shortconv input")
    if weight.shape[0] != H or state.shape[1:] != (L - 1, H):
        raise KernelError("shortconv: shapes do not fit")
    _f32(weight, "conv weight"), _f32(bias, "conv bias"), _f32(state, "conv state")
    _i32(cu_q, "cu_q"), _i32(ctx_before, "ctx_before"), _i32(slots, "slots")
    if not 2 <= L <= 8:
        raise KernelError(f"shortconv: width {L} is outside [2, 8]")
    f = _fn("shortconv", "ng_shortconv", [_c_void_p] * 8 + [_c_int] * 6 + [_c_ll, _c_void_p], {"NG_CONV_L": L})
    _check(f(_ptr(p), _ptr(weight), _ptr(bias), _ptr(state), _ptr(out), _ptr(cu_q), _ptr(ctx_before),
             _ptr(slots), n_entries, max_q, H, L, _act_flag(out, "conv out"), n_part, stride, _stream()), "shortconv")


def _stack(t: torch.Tensor, shape, act_dtype, what: str):
    """(n_partials, stride) of an input that is [*shape] in the activation dtype or a float32
    stack [S, *shape] of partial sums."""
    if t.dim() == len(shape) + 1:
        if t.dtype != torch.float32 or tuple(t.shape[1:]) != tuple(shape):
            raise KernelError(f"{what}: a stack of partial sums must be float32 [S, {', '.join(map(str, shape))}]")
        n = 1
        for d in shape:
            n *= d
        return t.shape[0], n
    if tuple(t.shape) != tuple(shape) or t.dtype != act_dtype:
        raise KernelError(f"{what}: expected {tuple(shape)} {act_dtype}, got {tuple(t.shape)} {t.dtype}")
    return 1, 0


# ----------------------------------------------------------------------------- attention
def rope_pairs(head_dim: int) -> int:
    """The rope kernel's specialisation for a head size: pairs of a head that one lane handles."""
    if head_dim <= 0 or head_dim % 2 or head_dim > 256:
        raise KernelError(f"rope_cache: head size {head_dim} is not an even number up to 256")
    return 1 if head_dim <= 64 else 2 if head_dim <= 128 else 4


def rope_cache(qkv: torch.Tensor, q_out: torch.Tensor, q_weight: Optional[torch.Tensor],
               k_weight: Optional[torch.Tensor], inv_freq: Optional[torch.Tensor], half_pairing: bool,
               pos_scale: float, k_pages: Optional[torch.Tensor], v_pages: Optional[torch.Tensor],
               table: torch.Tensor, positions: torch.Tensor, row_entry: torch.Tensor, n_heads: int,
               n_kv_heads: int, head_dim: int, eps: float, status: torch.Tensor) -> None:
    """Per-head norm of q and k, rotation, q -> q_out[N, nH*hd], k and v -> pages[P, nKV, page, hd].

    ``n_kv_heads`` 0 (with no pages) handles a layer that only reads another layer's cache.
    """
    n = q_out.shape[0]
    if q_out.shape != (n, n_heads * head_dim):
        raise KernelError("rope_cache: shapes do not fit")
    n_part, stride = _stack(qkv, (n, (n_heads + 2 * n_kv_heads) * head_dim), q_out.dtype, "rope_cache input")
    act = _act_flag(q_out, "q_out")
    page_size = num_pages = 1
    if n_kv_heads:
        if k_pages.dtype != q_out.dtype or k_pages.shape != v_pages.shape or k_pages.shape[1] != n_kv_heads \
                or k_pages.shape[3] != head_dim:
            raise KernelError("rope_cache: pages do not fit the projection")
        num_pages, page_size = k_pages.shape[0], k_pages.shape[2]
    _f32(q_weight, "q norm weight"), _f32(k_weight, "k norm weight"), _f32(inv_freq, "inv_freq")
    _i32(table, "table"), _i32(positions, "positions"), _i32(row_entry, "row_entry"), _i32(status, "status")
    f = _fn("rope_cache", "ng_rope_cache",
            [_c_void_p] * 5 + [_c_int, _c_float] + [_c_void_p] * 3 + [_c_int] + [_c_void_p] * 2 + [_c_int] * 6
            + [_c_float, _c_void_p, _c_int, _c_int, _c_ll, _c_void_p], {"NG_ROPE_PAIRS": rope_pairs(head_dim)})
    _check(f(_ptr(qkv), _ptr(q_out), _ptr(q_weight), _ptr(k_weight), _ptr(inv_freq), int(half_pairing),
             float(pos_scale), _ptr(k_pages), _ptr(v_pages), _ptr(table), table.shape[1], _ptr(positions),
             _ptr(row_entry), n, n_heads, n_kv_heads, head_dim, page_size, num_pages, float(eps), _ptr(status),
             act, n_part, stride, _stream()), "rope_cache")


def attention_generic(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, table: torch.Tensor,
                      positions: torch.Tensor, row_entry: torch.Tensor, out: torch.Tensor, n_heads: int,
                      window: Optional[int], scale: float, slopes: Optional[torch.Tensor] = None) -> None:
    """out[N, nH*hd] = softmax(q k^T * scale - bias, keys max(0,pos-window+1)..pos) v over the pages;
    bias = slopes[head] * (query position - key position) when ``slopes`` (float32 [nH]) is given."""
    n = q.shape[0]
    num_pages, n_kv, page_size, hd = k_pages.shape
    if q.shape != (n, n_heads * hd) or out.shape != q.shape or q.dtype != k_pages.dtype or out.dtype != q.dtype:
        raise KernelError("attention: shapes or dtypes do not fit")
    _i32(table, "table"), _i32(positions, "positions"), _i32(row_entry, "row_entry")
    f = _fn("attention_generic", "ng_attention_generic",
            [_c_void_p] * 4 + [_c_int] + [_c_void_p] * 3 + [_c_int] * 7 + [_c_float, _c_void_p, _c_int, _c_void_p])
    _check(f(_ptr(q), _ptr(k_pages), _ptr(v_pages), _ptr(table), table.shape[1], _ptr(positions),
             _ptr(row_entry), _ptr(out), n, n_heads, n_kv, hd, page_size, num_pages, int(window or 0),
             float(scale), _slopes(slopes, n_heads), _act_flag(q, "q"), _stream()), "attention_generic")


def _slopes(slopes: Optional[torch.Tensor], n_heads: int) -> Optional[int]:
    if slopes is None:
        return None
    if slopes.dtype != torch.float32 or slopes.numel() != n_heads:
        raise KernelError(f"score slopes must be float32 [{n_heads}]")
    return _ptr(slopes, "score slopes")


def attn_prefill_bf16(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, table: torch.Tensor,
                      cu_q: torch.Tensor, ctx_before: torch.Tensor, out: torch.Tensor, n_entries: int, max_q: int,
                      n_heads: int, window: Optional[int], scale: float, skip_single: bool,
                      slopes: Optional[torch.Tensor] = None) -> None:
    """Tensor-core flash attention of the step's portions (bfloat16); entries of one token are
    left to the decode kernel when ``skip_single``."""
    num_pages, n_kv, page_size, hd = k_pages.shape
    if q.dtype != torch.bfloat16 or k_pages.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
        raise KernelError("attn_prefill_bf16 takes bfloat16 tensors")
    if q.shape[1] != n_heads * hd or out.shape != q.shape or v_pages.shape != k_pages.shape:
        raise KernelError("attn_prefill_bf16: shapes do not fit")
    _i32(table, "table"), _i32(cu_q, "cu_q"), _i32(ctx_before, "ctx_before")
    f = _fn("attention_bf16", "ng_attn_prefill_bf16",
            [_c_void_p] * 4 + [_c_int] + [_c_void_p] * 3 + [_c_int] * 8 + [_c_float, _c_int, _c_void_p, _c_void_p],
            {"NG_HEAD_DIM": hd})
    _check(f(_ptr(q), _ptr(k_pages), _ptr(v_pages), _ptr(table), table.shape[1], _ptr(cu_q), _ptr(ctx_before),
             _ptr(out), n_entries, max_q, n_heads, n_kv, hd, page_size, num_pages, int(window or 0), float(scale),
             int(skip_single), _slopes(slopes, n_heads), _stream()), "attn_prefill_bf16")


ATTN_BACKEND = os.environ.get("NEUROGRID_B200_ATTN", "sm100")     # "sm100": tcgen05 prefill kernel; "mma": mma.sync


def attn_prefill_sm100_takes(head_dim: int, page_size: int) -> bool:
    """Whether the tcgen05 prefill kernel takes this shape (else the mma.sync kernel runs)."""
    return ATTN_BACKEND == "sm100" and head_dim == 64 and page_size in (8, 16, 32, 64)


def attn_prefill_scratch_floats(n_rows: int, n_heads: int, head_dim: int, n_splits: int) -> int:
    """float32 values the tcgen05 prefill kernel needs when it cuts the keys into ``n_splits`` runs."""
    return n_rows * n_heads * n_splits * (head_dim + 2) if n_splits > 1 else 0


def attn_prefill_sm100(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, table: torch.Tensor,
                       cu_q: torch.Tensor, ctx_before: torch.Tensor, out: torch.Tensor, n_entries: int, max_q: int,
                       n_heads: int, window: Optional[int], scale: float, skip_single: bool,
                       slopes: Optional[torch.Tensor] = None, scratch: Optional[torch.Tensor] = None,
                       n_splits: int = 1) -> None:
    """Flash attention of the step's portions on tcgen05/TMA/TMEM (bfloat16, head size 64).
    ``n_splits`` > 1: the keys of every block of rows are cut into that many runs, each a block of
    its own, merged by a second kernel through ``scratch`` (``attn_prefill_scratch_floats`` float32
    values); for long contexts whose blocks would fill the GPU unevenly."""
    num_pages, n_kv, page_size, hd = k_pages.shape
    if q.dtype != torch.bfloat16 or k_pages.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
        raise KernelError("attn_prefill_sm100 takes bfloat16 tensors")
    if q.shape[1] != n_heads * hd or out.shape != q.shape or v_pages.shape != k_pages.shape:
        raise KernelError("attn_prefill_sm100: shapes do not fit")
    need = attn_prefill_scratch_floats(q.shape[0], n_heads, hd, n_splits)
    if need and (scratch is None or scratch.numel() < need or scratch.dtype != torch.float32):
        raise KernelError(f"attn_prefill_sm100 needs {need} float32 values of scratch")
    _i32(table, "table"), _i32(cu_q, "cu_q"), _i32(ctx_before, "ctx_before")
    f = _fn("attention_sm100", "ng_attn_prefill_sm100",
            [_c_void_p] * 4 + [_c_int] + [_c_void_p] * 3 + [_c_int] * 9 + [_c_float, _c_int, _c_void_p, _c_void_p, _c_int,
                                                                             _c_void_p, _c_void_p])
    _check(f(_ptr(q), _ptr(k_pages), _ptr(v_pages), _ptr(table), table.shape[1], _ptr(cu_q), _ptr(ctx_before),
             _ptr(out), q.shape[0], n_entries, max_q, n_heads, n_kv, hd, page_size, num_pages, int(window or 0),
             float(scale), int(skip_single), _slopes(slopes, n_heads), _ptr(scratch) if need else None, int(n_splits),
             _ptr(_gemm_status(q.device)), _stream()),
           "attn_prefill_sm100")


def attn_decode_scratch_floats(n_rows: int, n_heads: int, head_dim: int, n_splits: int) -> int:
    return n_rows * n_heads * n_splits * (head_dim + 2) if n_splits > 1 else 0


def attn_decode_bf16(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, table: torch.Tensor,
                     cu_q: torch.Tensor, ctx_before: torch.Tensor, out: torch.Tensor,
                     scratch: Optional[torch.Tensor], n_entries: int, n_heads: int, window: Optional[int],
                     scale: float, n_splits: int, max_ctx: int, slopes: Optional[torch.Tensor] = None) -> None:
    """Split-context attention of the entries that bring one token (bfloat16).  ``max_ctx`` bounds
    the keys any entry sees (its tokens after the step); ``scratch`` holds
    ``attn_decode_scratch_floats`` float32 values when ``n_splits`` > 1."""
    num_pages, n_kv, page_size, hd = k_pages.shape
    if q.dtype != torch.bfloat16 or k_pages.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
        raise KernelError("attn_decode_bf16 takes bfloat16 tensors")
    if q.shape[1] != n_heads * hd or out.shape != q.shape or v_pages.shape != k_pages.shape:
        raise KernelError("attn_decode_bf16: shapes do not fit")
    need = attn_decode_scratch_floats(q.shape[0], n_heads, hd, n_splits)
    if need and (scratch is None or scratch.numel() < need or scratch.dtype != torch.float32):
        raise KernelError(f"attn_decode_bf16 needs {need} float32 values of scratch")
    _i32(table, "table"), _i32(cu_q, "cu_q"), _i32(ctx_before, "ctx_before")
    f = _fn("attention_bf16", "ng_attn_decode_bf16",
            [_c_void_p] * 4 + [_c_int] + [_c_void_p] * 4 + [_c_int] * 7 + [_c_float, _c_int, _c_int, _c_void_p, _c_void_p],
            {"NG_HEAD_DIM": hd})
    _check(f(_ptr(q), _ptr(k_pages), _ptr(v_pages), _ptr(table), table.shape[1], _ptr(cu_q), _ptr(ctx_before),
             _ptr(out), _ptr(scratch), n_entries, n_heads, n_kv, hd, page_size, num_pages, int(window or 0),
             float(scale), int(n_splits), int(max_ctx), _slopes(slopes, n_heads), _stream()), "attn_decode_bf16")


# ----------------------------------------------------------------------------- sampling
def sample(logits: torch.Tensor, temperature: Optional[torch.Tensor], top_p: Optional[torch.Tensor],
           uniform: Optional[torch.Tensor], out: torch.Tensor, scratch: Optional[torch.Tensor]) -> None:
    """out[W] int32: argmax where temperature <= 0 (or None), else a draw; scratch[W,V] float32."""
    W, V = logits.shape
    _f32(logits, "logits"), _f32(temperature, "temperature"), _f32(top_p, "top_p"), _f32(uniform, "uniform")
    _i32(out, "sample out"), _f32(scratch, "sample scratch")
    if temperature is not None and (uniform is None or scratch is None or scratch.numel() < W * V):
        raise KernelError("sample: a draw needs uniform numbers and W*V floats of scratch")
    f = _fn("sampling", "ng_sample", [_c_void_p, _c_int, _c_int] + [_c_void_p] * 6)
    _check(f(_ptr(logits), W, V, _ptr(temperature), _ptr(top_p), _ptr(uniform), _ptr(out), _ptr(scratch),
             _stream()), "sample")


# ----------------------------------------------------------------------------- tensor-core products
_GEMM_ARGS = [_c_void_p] * 4 + [_c_int] * 9 + [_c_void_p, _c_void_p]
# Steps of at most FUSE_MAX_ROWS rows (bfloat16, tcgen05 backend) add the products that end a
# mixer or a feed-forward straight into the float32 residual stream (red.global.add in the
# epilogue): the norm kernel that follows has no partial sums to read.  Measured on the decode
# graph of the 1.2B shape: batch 8 0.887 -> 0.852 ms, batch 64 1.329 -> 1.233 ms.
FUSE_MAX_ROWS = int(os.environ.get("NEUROGRID_B200_FUSE_ROWS", "64"))
FUSE_RED = os.environ.get("NEUROGRID_B200_FUSE_RED", "1") == "1"
GEMM_BACKEND = os.environ.get("NEUROGRID_B200_GEMM", "sm100")     # "sm100": tcgen05 kernel; "cublas": vendor library
# Rows up to which the tcgen05 kernel is used.  It streams weights at memory speed, which is the
# whole job when a step has few rows; for long portions the vendor library's product is still
# faster than this one-tile-per-block kernel, so it stands there.
SM100_MAX_ROWS = int(os.environ.get("NEUROGRID_B200_GEMM_MAX_ROWS", "64"))
_status_word = {}


def _gemm_status(device) -> torch.Tensor:
    t = _status_word.get(device)
    if t is None:
        t = _status_word[device] = torch.zeros(1, dtype=torch.int32, device=device)
    return t


def gemm_status(device) -> int:
    """Error bits the tcgen05 kernels recorded on ``device`` (8 = a bounded wait ran out); clears them."""
    t = _status_word.get(torch.device(device))
    if t is None:
        return 0
    own = int(t.item())
    if own:
        t.zero_()
    return own


def gemm_sm100_ok(x: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether the tcgen05 kernel is used for these operands (else the library's product)."""
    return (GEMM_BACKEND == "sm100" and x.shape[0] <= SM100_MAX_ROWS and gemm_sm100_takes(x, w))


def gemm_sm100_takes(x: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether the tcgen05 kernel can take these operands at all."""
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.is_cuda and x.dim() == 2
            and x.shape[1] % 8 == 0 and x.is_contiguous() and w.is_contiguous()
            and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def gemm_sm100(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor, *,
               splits: int = 1, token_tile: int = 0) -> None:
    """out = x @ w^T on tcgen05/TMA.  out bf16 [M,N] (+ bias), or float32 [M,N], or float32
    [S,M,N] partial sums over S = splits of K (``gemm_splits`` tells S for a K)."""
    M, K = x.shape
    N = w.shape[0]
    if out.dtype == torch.bfloat16:
        epi, s_eff = 0, 1
        if out.shape != (M, N) or splits != 1:
            raise KernelError("gemm_sm100: bf16 output is [M, N] without splits")
    else:
        epi = 1
        s_eff = gemm_splits(K, splits)
        if bias is not None or tuple(out.shape) not in (((M, N),) if s_eff == 1 else ()) + ((s_eff, M, N),):
            raise KernelError(f"gemm_sm100: float32 output must be [{s_eff}, {M}, {N}] (no bias)")
    f = _fn("gemm_sm100", "ng_gemm_sm100", _GEMM_ARGS)
    _check(f(_ptr(x), _ptr(w), _ptr(bias), _ptr(out), M, N, K, N, N, epi, s_eff, 0, token_tile,
             _ptr(_gemm_status(x.device)), _stream()), "gemm_sm100")


def gemm_splits(K: int, splits: int) -> int:
    total = -(-K // 64)
    splits = max(1, min(splits, total))
    per = -(-total // splits)
    return -(-total // per)


def gemm_swiglu_sm100(x: torch.Tensor, w_gate_up: torch.Tensor, out: torch.Tensor, *, token_tile: int = 0) -> None:
    """out[M,I] = silu(x wg^T) * (x wu^T) with w_gate_up = [wg (I rows); wu (I rows)]: the gate is
    applied in the product's epilogue."""
    M, K = x.shape
    I = out.shape[1]
    if w_gate_up.shape != (2 * I, K) or out.shape[0] != M or out.dtype != torch.bfloat16:
        raise KernelError("gemm_swiglu_sm100: shapes do not fit")
    status = _ptr(_gemm_status(w_gate_up.device))
    f = _fn("gemm_sm100", "ng_gemm_sm100", _GEMM_ARGS)
    _check(f(_ptr(x), _ptr(w_gate_up), None, _ptr(out), M, I, K, 2 * I, I, 2, 1, I, token_tile, status, _stream()),
           "gemm_swiglu_sm100")


# ----------------------------------------------------------------------------- matrix products
_SMS = {}


def sm_count(device) -> int:
    key = str(device)
    if key not in _SMS:
        _SMS[key] = torch.cuda.get_device_properties(device).multi_processor_count
    return _SMS[key]


MAX_RESIDUAL_SPLITS = 16


def linear_to_residual(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], ws, name: str,
                       residual: Optional[torch.Tensor] = None):
    """A product whose consumer can add partial sums (``add_rmsnorm``, ``residual_add``,
    ``shortconv``, ``rope_cache``).  Returns [M,N] in the activation dtype, or, for few rows on
    the tcgen05 path, a float32 stack [S,M,N] of split-K partial sums: with few rows the product
    is a stream of the weights, and splitting K puts every SM on it.

    ``residual`` (float32 [M,N]): the product is added straight into it when the kernel can
    do that, and None is returned: nothing is left for the caller to add."""
    M, K = x.shape
    N = weight.shape[0]
    if bias is None and M <= 64 and gemm_sm100_ok(x, weight):
        tiles = -(-N // 128)
        want = min(MAX_RESIDUAL_SPLITS, max(1, sm_count(weight.device) // tiles), max(1, -(-K // 64) // 4))
        s = gemm_splits(K, want)
        if FUSE_RED and residual is not None and M <= FUSE_MAX_ROWS:
            _f32(residual, "residual")
            f = _fn("gemm_sm100", "ng_gemm_sm100", _GEMM_ARGS)
            _check(f(_ptr(x), _ptr(weight), None, _ptr(residual), M, N, K, N, N, 3, s, 0, 0,
                     _ptr(_gemm_status(weight.device)), _stream()), "gemm_sm100 (residual add)")
            return None
        if s > 1:
            # partial sums exist for steps of at most 64 rows only
            buf = ws.flat(name + "_partials", s * M * N, torch.float32,
                          reserve=MAX_RESIDUAL_SPLITS * min(ws.max_rows, 64) * N)
            buf = buf[: s * M * N].view(s, M, N)
            gemm_sm100(x, weight, None, buf, splits=s)
            return buf
    out = ws.buf(name, M, N, x.dtype)
    linear(x, weight, bias, out)
    return out


def linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor) -> None:
    """out = x @ weight^T (+ bias).  float32: the FFMA kernel above.  bfloat16: the tcgen05
    kernel of this package, or the vendor library's product (``NEUROGRID_B200_GEMM=cublas``,
    and for operands the kernel does not take; the reference uses cuBLAS for every
    contraction, gpu/cuda/matmul.cu:316-355); float32 accumulation either way; ``out`` may be
    float32 (logits)."""
    if x.dtype == torch.float32:
        gemm_f32(x, weight, bias, out)
        return
    if not x.is_cuda:
        raise KernelError("linear: tensors must be on a CUDA device (there is no CPU path)")
    if gemm_sm100_ok(x, weight) and (bias is None or out.dtype == torch.bfloat16):
        gemm_sm100(x, weight, bias, out)
        return
    if out.dtype == torch.float32:
        torch.mm(x, weight.t(), out_dtype=torch.float32, out=out)
        if bias is not None:
            out += bias
    elif bias is not None:
        torch.addmm(bias, x, weight.t(), out=out)
    else:
        torch.mm(x, weight.t(), out=out)
