"""What the step function hands to every part, and the interfaces parts implement.

Shapes: N rows (tokens) in the step, R entries (requests) in the step, H model width.
Activations have the compute dtype (float32 or bfloat16); the residual stream, norm
weights, per-request states and logits are float32 in both.

Interfaces (duck-typed; a part is any class with these members):

* every part: ``tensors() -> {relative name: TensorDecl}``, ``bind({relative name: tensor})``.
* norm:      ``forward(h, delta, out, rows=None)``  h float32 [N,H] is updated to h + delta
             (delta may be None) and ``out`` receives the normed rows in the compute dtype.
* mixer:     ``cache_need() -> PagedNeed | SlotNeed | None`` and
             ``forward(x, ctx, cache) -> y`` with x, y [N,H]; ``cache`` is a
             :class:`PagedView`, a :class:`SlotView` or None, matching the declared need.
* ffn:       ``forward(x, ctx) -> y`` with x, y [N,H].
             A mixer or ffn may return, instead of y, a float32 stack [S,N,H] whose sum over S
             is y (split-K partial sums); the norm that follows adds it up.  When
             ``ctx.residual`` is set (steps of few rows) it may also add y into that float32
             stream itself and return None.
* position:  ``kernel_args() -> PositionArgs`` (or, for rotations only, the tuple
             ``(inv_freq float32[hd/2] | None, half_pairing, pos_scale)``): what the q/k kernel rotates by
             and what the attention kernels add to the scores.
* block:     ``forward(h, pending, ctx, cache) -> pending`` (see ``block.py``).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import torch


class Workspace:
    """Named scratch buffers, shared between layers by role name.

    ``buf(name, rows, cols, dtype)`` returns the first ``rows`` rows of a buffer that grows
    (to the next power of two of rows) when a step needs more; it keeps its address while it
    does not grow.  ``frozen`` forbids growth (set while CUDA graphs hold the addresses).
    """

    def __init__(self, max_rows: int, device, fixed: bool = False, row_caps: Optional[Dict[str, int]] = None):
        """``fixed``: every buffer is allocated for ``max_rows`` rows at once and never moves
        (what CUDA graphs need, which bake addresses in).  ``row_caps`` bounds named buffers
        below ``max_rows`` (the logits of a step whose wanted rows are few: a fixed workspace
        would otherwise hold ``max_rows`` rows of the vocabulary's width)."""
        self.max_rows = max_rows
        self.device = device
        self.frozen = False
        self.fixed = fixed
        self.row_caps = dict(row_caps or {})
        self._bufs: Dict[Tuple[str, int, torch.dtype], torch.Tensor] = {}

    def buf(self, name: str, rows: int, cols: int, dtype: torch.dtype) -> torch.Tensor:
        max_rows = min(self.max_rows, self.row_caps.get(name, self.max_rows))
        if rows > max_rows:
            raise ValueError(f"{rows} rows of {name!r} exceed the workspace ({max_rows} rows)")
        key = (name, cols, dtype)
        t = self._bufs.get(key)
        if t is None or t.shape[0] < rows:
            if self.frozen and t is not None:
                raise RuntimeError(f"workspace buffer {name!r} would have to grow while frozen")
            cap = max_rows if self.fixed else min(max_rows, max(16, 1 << (rows - 1).bit_length()))
            t = torch.zeros((cap, cols), dtype=dtype, device=self.device)
            self._bufs[key] = t
        return t[:rows]

    def flat(self, name: str, numel: int, dtype: torch.dtype, reserve: int = 0) -> torch.Tensor:
        """A 1-D scratch buffer of at least ``numel`` elements (grows by powers of two).  In a
        fixed workspace the first call allocates ``reserve`` elements, the caller's upper bound."""
        key = (name, -1, dtype)
        t = self._bufs.get(key)
        if t is None or t.numel() < numel:
            if (self.frozen or self.fixed) and t is not None:
                raise RuntimeError(f"workspace buffer {name!r} would have to grow while its address is fixed")
            numel = max(numel, reserve if self.fixed else 0)
            t = torch.zeros(max(1024, 1 << (max(numel, 1) - 1).bit_length()), dtype=dtype, device=self.device)
            self._bufs[key] = t
        return t

    def nbytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self._bufs.values())


@dataclass
class PositionArgs:
    """How positions enter an attention layer, as parameters of its kernels.

    Rotation of q and k (in the q/k kernel): ``inv_freq`` float32 [head_dim/2] gives the angle per
    pair and position (None: no rotation; a zero entry leaves its pair unrotated), ``half_pairing``
    pairs (i, i + head_dim/2) instead of (2i, 2i+1), ``pos_scale`` divides positions first.
    Score bias (in the attention kernels): ``score_slopes`` float32 [n_heads] subtracts
    ``slope[head] * (query position - key position)`` from every score before the softmax."""
    inv_freq: Optional[torch.Tensor] = None
    half_pairing: bool = False
    pos_scale: float = 1.0
    score_slopes: Optional[torch.Tensor] = None

    @classmethod
    def of(cls, args) -> "PositionArgs":
        return args if isinstance(args, cls) else cls(*args)


@dataclass
class PagedView:
    """One layer's keys and values, [pages, n_kv_heads, page_size, head_dim] each, and the
    step's block table [R, max_pages] (entry-indexed; -1 = no page)."""
    k_pages: torch.Tensor
    v_pages: torch.Tensor
    table: torch.Tensor
    writes: bool = True          # False: this run of the layer reads another layer's cache


@dataclass
class SlotView:
    """One layer's fixed-size state for every slot, [slots, *shape] in the dtype its need names."""
    state: torch.Tensor


@dataclass
class StepContext:
    """Device-side description of one step's ragged batch plus what the host knows of it."""
    n_rows: int
    n_entries: int
    max_q: int                      # longest portion in the step
    tokens: torch.Tensor            # int32 [N]
    positions: torch.Tensor         # int32 [N]  absolute position of each row in its request
    row_entry: torch.Tensor         # int32 [N]  entry of each row (-1 = padding row)
    cu_q: torch.Tensor              # int32 [R+1] first row of each entry
    ctx_before: torch.Tensor        # int32 [R]  tokens of the request already in the cache
    slots: torch.Tensor             # int32 [R]  state slot of each entry
    status: torch.Tensor            # int32 [1]  error bits set by kernels
    ws: Workspace
    dtype: torch.dtype              # compute dtype of activations
    q_lens: Sequence[int] = ()      # host copies, for dispatch decisions only
    ctx_lens: Sequence[int] = ()
    slot_ids: Sequence[int] = ()
    graph_safe: bool = False        # True while a CUDA graph is being captured
    fuse_residual: bool = False     # few rows: parts may add their outputs into the stream themselves
    residual: Optional[torch.Tensor] = None   # the float32 stream (set by the block when fuse_residual)
    decode_max_ctx: int = 0         # set (with decode_batch) when launch shapes must not follow the batch
    decode_batch: int = 0
    prefill_ctx: int = 0            # set when a graph serves a class of contexts: the context length its portion kernels plan for
    fixed_launches: bool = False    # a CUDA graph of a padded step that may hold portions and single tokens: parts launch
                                    # for both kinds whatever the host lists say (the kernels skip what is not there)
