"""Recorder and launcher of operation chains for the persistent kernel of ``chain_sm100.cu``.

While a chain is open (``ops.chain_scope``), the launchers of ``ops`` that the kernel can run
(RMSNorm, the tensor-core products with their epilogues, the one-token short convolution)
append an operation here instead of launching; any other launch first flushes what was
recorded, as one kernel.  A chain is described to the kernel by an array of tensor maps and an
array of operation records on the device; both depend only on pointers and sizes, so they are
built once per distinct chain and kept (a CUDA graph that replays the launch keeps reading
them).
"""
from __future__ import annotations

import ctypes
import struct
from typing import Dict, List, Optional, Tuple

import torch

OP_GEMM, OP_NORM, OP_CONV = 0, 1, 2
EPI_BF16, EPI_F32, EPI_SWIGLU, EPI_RED = 0, 1, 2, 3
_OP_FORMAT = "<8Q18iqf3i"
assert struct.calcsize(_OP_FORMAT) == 160

_c_int, _c_void_p = ctypes.c_int, ctypes.c_void_p


class ChainError(RuntimeError):
    pass


def token_tile(rows: int) -> Optional[int]:
    """The kernel's token tile for a step of ``rows`` rows (None: the kernel does not take it)."""
    for tn in (16, 32, 64):
        if rows <= tn:
            return tn
    return None


class _Prepared:
    """Device copies of one chain's tensor maps and operation records, and its barrier words."""

    def __init__(self, maps: torch.Tensor, ops: torch.Tensor, n_ops: int):
        self.maps, self.ops, self.n_ops = maps, ops, n_ops


class Chain:
    def __init__(self, device, tn: int, lib):
        self.device, self.tn, self.lib = torch.device(device), tn, lib
        self.records: List[tuple] = []          # hashable description of each operation
        self.maps: List[Tuple[int, int, int, int]] = []   # (ptr, rows, cols, box_rows)
        self.keep: List[torch.Tensor] = []      # tensors whose pointers the records hold
        self.launching = False
        self.launches = 0
        self.max_ops = int(lib.ng_chain_max_ops()) - 4

    # ------------------------------------------------------------------ recording
    def _map(self, t: torch.Tensor, box_rows: int) -> int:
        key = (t.data_ptr(), t.shape[0], t.shape[1], box_rows)
        if key in self.maps:
            return self.maps.index(key)
        self.maps.append(key)
        return len(self.maps) - 1

    def _room(self):
        if len(self.records) >= self.max_ops:
            self.flush()

    def plan(self, M: int, N: int, K: int, epi: int, splits: int):
        out = [ctypes.c_int() for _ in range(5)]
        rc = self.lib.ng_chain_plan(M, N, K, epi, splits, *[ctypes.byref(o) for o in out])
        if rc != 0:
            raise ChainError(f"chain: a product of {M} x {N} x {K} cannot be planned")
        return tuple(o.value for o in out)      # rows, n_tiles, splits, kb_per_split, w_bytes

    def gemm(self, x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, epi: int, splits: int = 1,
             n_out: Optional[int] = None, up_row_offset: int = 0, ldc: Optional[int] = None) -> int:
        """Record out = x w^T; returns the K splits the kernel will use."""
        M, K = x.shape
        N = n_out if n_out is not None else w.shape[0]
        if M > self.tn:
            raise ChainError(f"chain: {M} rows exceed the token tile {self.tn}")
        self._room()
        rows, n_tiles, s_eff, per, w_bytes = self.plan(M, N, K, epi, splits)
        rec = (OP_GEMM, out.data_ptr(), M, N, K, rows, n_tiles, s_eff, per, epi, ldc if ldc is not None else N,
               up_row_offset, w_bytes, self._map(w, rows), self._map(x, self.tn))
        self.records.append(rec)
        self.keep += [x, w, out]
        return s_eff

    def norm(self, h: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, eps: float,
             rows: Optional[torch.Tensor] = None) -> None:
        self._room()
        self.records.append((OP_NORM, h.data_ptr(), weight.data_ptr(), out.data_ptr(),
                             rows.data_ptr() if rows is not None else 0, out.shape[0], out.shape[1], float(eps)))
        self.keep += [h, weight, out] + ([rows] if rows is not None else [])

    def conv(self, partials: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], state: torch.Tensor,
             out: torch.Tensor, cu_q: torch.Tensor, ctx_before: torch.Tensor, slots: torch.Tensor, n_entries: int) -> None:
        self._room()
        H, L = out.shape[1], weight.shape[1]
        if partials.dim() == 3:                 # float32 stack of K-split partial sums
            S, stride = partials.shape[0], partials.shape[1] * partials.shape[2]
        else:                                   # the product itself, bfloat16
            S, stride = 0, 0
        self.records.append((OP_CONV, partials.data_ptr(), weight.data_ptr(), bias.data_ptr() if bias is not None else 0,
                             state.data_ptr(), out.data_ptr(), cu_q.data_ptr(), ctx_before.data_ptr(), slots.data_ptr(),
                             n_entries, H, L, S, stride))
        self.keep += [partials, weight, state, out, cu_q, ctx_before, slots] + ([bias] if bias is not None else [])

    # ------------------------------------------------------------------ launching
    def _pack(self, rec: tuple) -> bytes:
        p = [0] * 8
        i = dict(type=rec[0], M=0, N=0, K=0, rows=0, n_tiles=0, splits=0, kb=0, epi=0, ldc=0, up=0, w_bytes=0,
                 w_map=0, x_map=0, H=0, L=0, n_part=0, flags=0)
        pstride, eps = 0, 0.0
        if rec[0] == OP_GEMM:
            (_, p[0], i["M"], i["N"], i["K"], i["rows"], i["n_tiles"], i["splits"], i["kb"], i["epi"], i["ldc"],
             i["up"], i["w_bytes"], i["w_map"], i["x_map"]) = rec
        elif rec[0] == OP_NORM:
            _, p[0], p[1], p[2], p[3], i["M"], i["H"], eps = rec
        else:
            _, p[0], p[1], p[2], p[3], p[4], p[5], p[6], p[7], i["M"], i["H"], i["L"], i["n_part"], pstride = rec
        return struct.pack(_OP_FORMAT, *p, *i.values(), pstride, eps, 0, 0, 0)

    def _prepare(self) -> _Prepared:
        n_maps = max(1, len(self.maps))
        host_maps = (ctypes.c_ubyte * (128 * n_maps))()
        for j, (ptr, rows, cols, box) in enumerate(self.maps):
            rc = self.lib.ng_chain_encode_map(ptr, rows, cols, box, ctypes.byref(host_maps, 128 * j))
            if rc != 0:
                raise ChainError(f"chain: no tensor map for a [{rows}, {cols}] operand (error {rc})")
        blob = b"".join(self._pack(r) for r in self.records)
        maps = torch.frombuffer(bytearray(host_maps), dtype=torch.uint8).to(self.device)
        ops = torch.frombuffer(bytearray(blob), dtype=torch.uint8).to(self.device)
        if maps.data_ptr() % 64 or ops.data_ptr() % 16:
            raise ChainError("chain: device buffers are not aligned")
        return _Prepared(maps, ops, len(self.records))

    def flush(self) -> None:
        """Launch what was recorded as one kernel (nothing if nothing was)."""
        if not self.records:
            return
        key = (self.tn, tuple(self.records), tuple(self.maps))
        cache = _prepared.setdefault(self.device, {})
        prep = cache.get(key)
        if prep is None:
            if torch.cuda.is_current_stream_capturing():
                raise ChainError("chain: a chain must run once outside a graph capture before it is captured")
            prep = cache[key] = self._prepare()
            prep.keep = list(self.keep)
        self.records, self.maps, self.keep = [], [], []
        self.launching = True
        try:
            rc = self.lib.ng_chain_launch(prep.maps.data_ptr(), prep.ops.data_ptr(), prep.n_ops, self.tn,
                                          counters(self.device).data_ptr(), status_word(self.device).data_ptr(),
                                          torch.cuda.current_stream().cuda_stream)
        finally:
            self.launching = False
        if rc != 0:
            raise ChainError(f"chain: the launch of {prep.n_ops} operations failed (error {rc})")
        self.launches += 1


_prepared: Dict[torch.device, Dict[tuple, _Prepared]] = {}
_counters: Dict[torch.device, torch.Tensor] = {}
_status: Dict[torch.device, torch.Tensor] = {}


def counters(device) -> torch.Tensor:
    """Two words per device: arrivals at the kernel's barriers and blocks that have left; the
    kernel leaves them zero."""
    device = torch.device(device)
    t = _counters.get(device)
    if t is None:
        t = _counters[device] = torch.zeros(2, dtype=torch.int32, device=device)
    return t


def status_word(device) -> torch.Tensor:
    device = torch.device(device)
    t = _status.get(device)
    if t is None:
        t = _status[device] = torch.zeros(1, dtype=torch.int32, device=device)
    return t


def read_status(device) -> int:
    """Error bits the chain kernel recorded on ``device`` (32 = a bounded wait ran out); clears
    them, and the barrier words with them (a kernel that gave up leaves them undefined)."""
    t = _status.get(torch.device(device))
    if t is None:
        return 0
    bits = int(t.item())
    if bits:
        t.zero_()
        counters(device).zero_()
    return bits


def load_library(build):
    import os
    trace = os.environ.get("NEUROGRID_B200_CHAIN_TRACE")          # a block index: build with its clock stamps
    lib = build.load("chain_sm100", {"CHAIN_TRACE": 1, "CHAIN_TRACE_CTA": int(trace)} if trace else None)
    lib.ng_chain_plan.argtypes = [_c_int] * 5 + [ctypes.POINTER(ctypes.c_int)] * 5
    lib.ng_chain_plan.restype = _c_int
    lib.ng_chain_encode_map.argtypes = [_c_void_p, _c_int, _c_int, _c_int, _c_void_p]
    lib.ng_chain_encode_map.restype = _c_int
    lib.ng_chain_launch.argtypes = [_c_void_p, _c_void_p, _c_int, _c_int, _c_void_p, _c_void_p, _c_void_p]
    lib.ng_chain_launch.restype = _c_int
    lib.ng_chain_max_ops.restype = _c_int
    lib.ng_chain_op_bytes.restype = _c_int
    if lib.ng_chain_op_bytes() != struct.calcsize(_OP_FORMAT):
        raise ChainError("chain: the operation record of the library and of the host differ in size")
    return lib


def _trace_main(argv=None) -> int:
    """``python -m neurogrid_b200.csrc.chain --block B``: run three layers' worth of
    [norm, out_proj (+= h), norm, gate/up + SwiGLU, down (+= h)] as one chain in a build that stamps
    block B's SM clock at the stations of every operation, and print the stamps in microseconds."""
    import argparse
    import os
    ap = argparse.ArgumentParser(description=_trace_main.__doc__)
    ap.add_argument("--block", type=int, default=0)
    ap.add_argument("--rows", type=int, default=8)
    ap.add_argument("--width", type=int, default=2048)
    ap.add_argument("--ffn", type=int, default=8192)
    ap.add_argument("--ghz", type=float, default=1.9, help="SM clock for the conversion to microseconds")
    a = ap.parse_args(argv)
    os.environ["NEUROGRID_B200_CHAIN_TRACE"] = str(a.block)
    from . import ops as o
    o.CHAIN = True
    dev, bf = "cuda", torch.bfloat16
    M, H, I = a.rows, a.width, a.ffn
    g = torch.Generator(device="cpu").manual_seed(0)
    rnd = lambda *s: torch.randn(*s, generator=g)
    h = rnd(M, H).to(dev)
    x = torch.zeros(M, H, dtype=bf, device=dev)
    nw = torch.ones(H, device=dev)
    act = torch.zeros(M, I, dtype=bf, device=dev)
    w_out = [(rnd(H, H) * 0.02).to(bf).to(dev) for _ in range(3)]
    w_gu = [(rnd(2 * I, H) * 0.02).to(bf).to(dev) for _ in range(3)]
    w_dn = [(rnd(H, I) * 0.02).to(bf).to(dev) for _ in range(3)]

    class _Ws:
        max_rows = 64

    def run():
        with o.chain_scope(dev, M):
            for i in range(3):
                o.add_rmsnorm(h, None, nw, x, 1e-5)
                o.linear_to_residual(x, w_out[i], None, _Ws, "a", residual=h)
                o.add_rmsnorm(h, None, nw, x, 1e-5)
                o.gemm_swiglu_sm100(x, w_gu[i], act)
                o.linear_to_residual(act, w_dn[i], None, _Ws, "d", residual=h)
    for _ in range(3):
        run()
    torch.cuda.synchronize()
    lib = o._chain_lib
    buf = (ctypes.c_longlong * (64 * 16))()
    lib.ng_chain_trace.argtypes = [_c_void_p, _c_int]
    lib.ng_chain_trace.restype = _c_int
    if lib.ng_chain_trace(buf, 64 * 16) != 0:
        raise ChainError("chain: the trace could not be read")
    names = ["norm", "out+=h", "norm", "gate/up", "down+=h"] * 3
    base = min(v for v in buf if v)
    print("us since the first stamp; stations: gate seen | X issued | first stage full | last MMA committed | "
          "epilogue sees it | stores issued | before fence | after fence | arrived | barrier passed")
    for op in range(15):
        row = [buf[op * 16 + k] for k in range(10)]
        print(f"op{op:2d} {names[op]:8s} " + " ".join(f"{(v - base) / (a.ghz * 1e3):8.2f}" if v else "       -" for v in row))
    return 0


if __name__ == "__main__":
    raise SystemExit(_trace_main())
