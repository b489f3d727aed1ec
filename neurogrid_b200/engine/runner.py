"""The step function: one ragged batch in, logits at the wanted places out.

A step is a list of entries ``(request, its next tokens, wanted places)``: portions of
prompts beside single decode tokens, cut anywhere.  The runner takes pages for the new
tokens, packs the batch description into one host buffer, copies it to the device in one
transfer, runs only the rows it was given through the model (keys, values and states of
earlier steps come from the cache) and returns float32 logits for the wanted rows.

The reference has three separate entry points instead (whole-prompt prefill of one request,
one token of one request, one token of N requests looped inside:
gpu/engine/decode_all.cu:509-603,629-792,820-943) and cannot mix or cut them.
"""
from __future__ import annotations

import os

from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence

import numpy as np
import torch

from ..cache.manager import CacheManager
from ..cache.pages import OutOfPages
from ..cache.storage import CacheStorage
from ..parts.base import PagedView, SlotView, StepContext, Workspace


def _next_pow2(n: int) -> int:
    return 1 << max(0, int(n) - 1).bit_length()


class StepError(RuntimeError):
    """The step was refused before anything ran (bad token, no room, unknown request...)."""


@dataclass
class StepEntry:
    req_id: Hashable
    tokens: Sequence[int]
    want: Sequence[int] = ()        # indices into ``tokens`` whose logits are returned


class ModelRunner:
    MAX_PORTION_GRAPHS = 8
    MAX_MIXED_GRAPHS = 24
    MIXED_GRAPH_MAX_ROWS = 1024    # steps of portions beside single tokens up to this many rows replay graphs of padded
                                   # shapes (launching such a step kernel by kernel costs the host more than the device)
    PORTION_LONG_CTX = 8192        # portion graphs come in classes of context: below this many tokens, and by powers of two from it on
    MAX_PORTION_ROWS = 4096        # portion graphs use a workspace allocated whole for this many rows
    MAX_PORTION_LOGITS_BYTES = 64 << 20   # ... and for this much of logits (a portion that wants more rows runs eagerly)

    def __init__(self, model, *, num_pages, page_size: int = 16, max_requests: int = 8,
                 max_seq_len: Optional[int] = None, max_tokens_per_step: int = 2048, cuda_graphs: bool = True):
        self.model = model
        self.device, self.dtype = model.device, model.dtype
        spec = model.spec
        # a model that states no limit is bounded by the pool alone
        self.max_seq_len = int(max_seq_len or spec.max_positions or num_pages * page_size)
        self.max_tokens_per_step = int(max_tokens_per_step)
        self.max_requests = int(max_requests)
        self.storage = CacheStorage(model.cache_needs(), pages_per_group=num_pages, page_size=page_size,
                                    max_requests=max_requests, dtype=self.dtype, device=self.device)
        self.cache = CacheManager(self.storage.paged_needs, self.storage.pages_per_group, page_size,
                                  max_requests, self.max_seq_len)
        self.ws = Workspace(self.max_tokens_per_step, self.device)
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.stride = self.cache.max_pages_per_request
        n_groups = len(self.storage.paged_needs)
        # rows of a step, padded as the graphs of padded steps pad them
        rows_cap = max(_next_pow2(self.max_tokens_per_step), _next_pow2(max_requests), 16)
        cap = 4 * rows_cap + (4 + n_groups * self.stride) * _next_pow2(max_requests) + 1
        self._on_cuda = torch.device(self.device).type == "cuda"
        if self._on_cuda:
            # compile (side by side) what this model launches, rather than one library at a time
            # when the first step first meets each kernel
            from ..csrc import build, kernel_sets
            build.compile_many(kernel_sets.needed_by(model))
        # the batch description is staged in pinned host buffers used in turn; a buffer is
        # written again only after the copy that last read it has finished
        self._ring = [torch.zeros(cap, dtype=torch.int32, pin_memory=self._on_cuda) for _ in range(4)]
        self._ring_events = [torch.cuda.Event() if self._on_cuda else None for _ in self._ring]
        self._ring_used = [False] * len(self._ring)
        self._ring_next = 0
        self._dev = torch.zeros(cap, dtype=torch.int32, device=self.device)
        self._feed = None
        self._greedy_into = None
        self.sampled_in_graph = False
        self.fed_in_graph = False
        self.feed_source: Optional[torch.Tensor] = None    # the buffer a sampler leaves its tokens in (set by the engine)
        self._feed_idx = None
        self._feed_ring = [torch.zeros(rows_cap, dtype=torch.int32, pin_memory=self._on_cuda) for _ in range(4)]
        self._feed_events = [torch.cuda.Event() if self._on_cuda else None for _ in self._feed_ring]
        self._feed_used = [False] * len(self._feed_ring)
        self._feed_next = 0
        self._feed_dev = torch.zeros(rows_cap, dtype=torch.int32, device=self.device)
        self.steps_run = 0
        self.tokens_run = 0
        self.last_meta_words = 0
        # decode-only steps replay CUDA graphs per (padded batch, context bucket), captured the second
        # time a shape is met (the first time runs eagerly and warms up).  The schedule is cut into
        # pieces: stretches of layers whose parts are ``graph_safe`` are graphs, a layer with a part that
        # is not (one that decides launches from host data of the step) runs eagerly between them
        self._pieces = model.graph_pieces()
        self.cuda_graphs = bool(cuda_graphs) and self._on_cuda and any(safe and idx for safe, idx in self._pieces)
        self._graph_ws = Workspace(_next_pow2(max_requests), self.device, fixed=True) if self.cuda_graphs else None
        self.portion_graphs = os.environ.get("NEUROGRID_B200_PORTION_GRAPHS", "1") == "1"
        self._portion_ws = None
        self._mixed_ws = None
        self.mixed_graphs = os.environ.get("NEUROGRID_B200_MIXED_GRAPHS", "1") == "1"
        self._portion_wanted = max(16, min(self.MAX_PORTION_ROWS, self.MAX_PORTION_LOGITS_BYTES // (4 * spec.vocab_size)))
        self._graphs: Dict[tuple, object] = {}
        self.graph_replays = 0
        self.eager_steps = 0
        self.keep_graphs = False       # keep the captured graphs beside their executables (for `graph_kernel_nodes`)

    @staticmethod
    def bytes_per_page(model, page_size: int) -> int:
        """Device bytes one page id costs over all paged layers (keys and values)."""
        from ..cache.manager import PagedNeed
        esz = torch.empty((), dtype=model.dtype).element_size()
        return sum(2 * n.n_kv_heads * n.head_dim * page_size * esz
                   for n in model.cache_needs().values() if isinstance(n, PagedNeed))

    # ------------------------------------------------------------------ requests
    def admit(self, req_id: Hashable) -> int:
        slot = self.cache.admit(req_id)
        self.storage.reset_slot(slot)
        return slot

    def finish(self, req_id: Hashable) -> None:
        """Give back the request's pages and slot."""
        if self.cache.is_live(req_id):
            self.cache.release(req_id)

    # ------------------------------------------------------------------ the step
    def step(self, entries: Sequence[StepEntry], token_feed=None, greedy_into: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
        """Run one batch; returns float32 logits [wanted, vocab] in entry order then ``want``
        order (None if nothing is wanted).  Requests not yet live are admitted.  The tensor is
        workspace memory: it is overwritten by the next step.

        ``token_feed = (src, idx)``: ``src`` is an int32 device tensor (tokens a sampler left
        there) and ``idx`` gives, per row of the step, the element of ``src`` that is the row's
        token (-1: the token given in the entry).  The host then need not know those tokens
        when it launches the step.

        ``greedy_into``: an int32 device tensor; a decode-only step that runs as a CUDA graph
        also takes the argmax of every row's logits into it, inside the graph
        (``sampled_in_graph`` then says so, and the caller launches no sampling kernel)."""
        self._feed = token_feed
        self._greedy_into = greedy_into
        self.sampled_in_graph = False
        self.fed_in_graph = False
        if self.cuda_graphs and all(len(e.tokens) == 1 for e in entries) and entries:
            logits = self._step_graphed(entries)
        elif self.cuda_graphs and self.portion_graphs and len(entries) == 1 and token_feed is None \
                and len(entries[0].tokens) <= self.MAX_PORTION_ROWS and len(entries[0].want) <= self._portion_wanted:
            logits = self._portion_graphed(entries)
        elif self.cuda_graphs and self.mixed_graphs and token_feed is None and self._mixed_graph_takes(entries):
            logits = self._mixed_graphed(entries)
        else:
            ctx, want_rows, n_want = self._prepare(entries)
            self._apply_feed(ctx)
            ctx.fuse_residual = self._fuse_rows(ctx.n_rows)
            logits = self.model.forward(ctx, self._cache_views(ctx), want_rows, n_want)
            self.eager_steps += 1
        reqs = self.cache._req
        for e in entries:
            if len(e.tokens) == 1 and self.cache.slack(e.req_id) >= 1:
                reqs[e.req_id].length += 1
            else:
                self.cache.advance(e.req_id, len(e.tokens))
        self.steps_run += 1
        self.tokens_run += sum(len(e.tokens) for e in entries)
        return logits

    def _step_graphed(self, entries: Sequence[StepEntry]) -> Optional[torch.Tensor]:
        R = len(entries)
        bucket = _next_pow2(R)
        # tokens that are still on the device: when they lie in the buffer this runner was told of
        # (``feed_source``), the graph itself gathers them, from indices that travel with the
        # batch description; otherwise a kernel in front of the graph does
        feed_in_graph = self.feed_source is not None and (
            self._feed is None or self._feed[0].data_ptr() == self.feed_source.data_ptr())
        prepared = self._prepare_decode(entries, bucket, self._feed[1] if (feed_in_graph and self._feed is not None) else None)
        ctx, want_rows, n_want = prepared if prepared is not None else self._prepare(entries, pad_to=bucket)
        feed_in_graph = feed_in_graph and prepared is not None
        need = max(ctx.ctx_lens) + 1
        ctx_bucket = min(-(-need // 1024) * 1024, max(self.max_seq_len, need))
        if not feed_in_graph:
            self._apply_feed(ctx)
        self._feed = None
        ctx.ws, ctx.graph_safe = self._graph_ws, True
        ctx.fuse_residual = self._fuse_rows(ctx.n_rows)
        ctx.decode_max_ctx, ctx.decode_batch = ctx_bucket, bucket
        greedy = self._greedy_into if (self._greedy_into is not None and all(len(e.want) == 1 for e in entries)) else None
        key = (bucket, ctx_bucket, feed_in_graph, greedy.data_ptr() if greedy is not None else 0)

        from ..csrc import ops

        def pre():
            if feed_in_graph:
                ops.gather_tokens(ctx.tokens, self.feed_source, self._feed_idx)

        def post(out):
            if greedy is not None:
                ops.sample(out, None, None, None, greedy[:out.shape[0]], None)

        logits = self._graphed_forward(key, ctx, want_rows, n_want, pre, post)
        self.sampled_in_graph = greedy is not None
        self.fed_in_graph = feed_in_graph
        wanted = [i for i, e in enumerate(entries) if len(e.want)]
        if not wanted:
            return None
        if len(wanted) == R:
            return logits[:R]
        return logits[torch.tensor(wanted, device=self.device)]

    def _portion_graphed(self, entries: Sequence[StepEntry]) -> Optional[torch.Tensor]:
        """A step that is one request's prompt portion: a CUDA graph per (rows, wanted rows).  What
        the launches depend on besides those two (positions, the context so far, the block table,
        the state slot) is device data that the step's one copy brings, so one graph serves every
        portion of that size, at any context.  Prompts cut into portions of `chunk_size` meet the
        same size again and again; a step's hundred and more launches cost the host about 2 ms,
        which for small models is more than the device needs for them.  The first meeting of a
        size runs eagerly, the second captures; at most `MAX_PORTION_GRAPHS` sizes are kept."""
        ctx, want_rows, n_want = self._prepare(entries)
        # parts plan a portion's launches by the context too (a long one is cut into runs of keys): a graph per class
        seen = ctx.ctx_lens[0] + ctx.n_rows
        ctx.prefill_ctx = 1 << (seen.bit_length() - 1) if seen >= self.PORTION_LONG_CTX else 1
        key = ("portion", ctx.n_rows, n_want, ctx.prefill_ctx)
        state = self._graphs.get(key)
        if state is None and sum(1 for k in self._graphs if k[0] == "portion") >= self.MAX_PORTION_GRAPHS:
            ctx.fuse_residual = self._fuse_rows(ctx.n_rows)
            self.eager_steps += 1
            return self.model.forward(ctx, self._cache_views(ctx), want_rows, n_want)
        if self._portion_ws is None:
            caps = {"logits": self._portion_wanted, "head_in": self._portion_wanted}
            self._portion_ws = Workspace(min(self.max_tokens_per_step, self.MAX_PORTION_ROWS), self.device, fixed=True,
                                         row_caps=caps)
        ctx.ws, ctx.graph_safe = self._portion_ws, True
        ctx.fuse_residual = self._fuse_rows(ctx.n_rows)
        return self._graphed_forward(key, ctx, want_rows, n_want)

    def _mixed_graph_takes(self, entries: Sequence[StepEntry]) -> bool:
        rows = sum(len(e.tokens) for e in entries)
        return (1 < len(entries) and rows <= self.MIXED_GRAPH_MAX_ROWS and not self.cache.windowed
                and all(len(e.want) <= 1 for e in entries))

    def _mixed_graphed(self, entries: Sequence[StepEntry]) -> Optional[torch.Tensor]:
        """A step of several entries, portions beside single tokens: rows, entries and wanted rows are
        padded (to powers of two; rows above 256 to multiples of 128) and the step replays a graph per
        (rows, entries, context bucket).
        Padding rows belong to no entry, padding entries have no rows, padding wanted rows repeat row 0;
        every launch has the padded shape and the kernels skip what is not there."""
        n_real = sum(len(e.tokens) for e in entries)
        # rows: powers of two up to 256, multiples of 128 above (padding costs compute there)
        n_pad = max(16, _next_pow2(n_real)) if n_real <= 256 else -(-n_real // 128) * 128
        r_pad = _next_pow2(len(entries))
        ctx, want_rows, n_want = self._prepare(entries, pads=(n_pad, r_pad, r_pad))
        w_real = sum(len(e.want) for e in entries)
        need = max(c + q for c, q in zip(ctx.ctx_lens, ctx.q_lens))
        ctx_bucket = min(-(-need // 1024) * 1024, max(self.max_seq_len, need))
        key = ("mixed", n_pad, r_pad, ctx_bucket)
        if key not in self._graphs and sum(1 for k in self._graphs if k[0] == "mixed") >= self.MAX_MIXED_GRAPHS:
            key = None
        if self._mixed_ws is None:
            cap = _next_pow2(self.max_requests)
            self._mixed_ws = Workspace(self.MIXED_GRAPH_MAX_ROWS, self.device, fixed=True,
                                       row_caps={"logits": cap, "head_in": cap})
        ctx.ws, ctx.graph_safe, ctx.fixed_launches = self._mixed_ws, True, True
        ctx.fuse_residual = self._fuse_rows(ctx.n_rows)
        ctx.decode_max_ctx, ctx.decode_batch, ctx.prefill_ctx = ctx_bucket, r_pad, ctx_bucket
        if key is None:
            logits = self.model.forward(ctx, self._cache_views(ctx), want_rows, n_want)
            self.eager_steps += 1
        else:
            logits = self._graphed_forward(key, ctx, want_rows, n_want)
        return logits[:w_real] if w_real else None

    def _graphed_forward(self, key, ctx, want_rows, n_want, pre=None, post=None):
        """The model over ``ctx`` through the graphs kept under ``key``: the first meeting of a key
        runs eagerly, the second captures every graph-safe piece of the schedule (replaying each as
        soon as it is captured, since what follows needs its results), later ones replay.  Pieces
        that are not graph-safe run eagerly every time; what they hand to the next piece is copied
        to a buffer of fixed address.  ``pre()`` launches in front of the embedding, ``post(logits)``
        after the head, inside the first and the last piece."""
        pieces, model = self._pieces, self.model
        views = self._cache_views(ctx)
        last = len(pieces) - 1

        def body(k, h, pending):
            if k == 0:
                if pre is not None:
                    pre()
                h = model.begin(ctx)
            pending = model.run_entries(ctx, views, pieces[k][1], h, pending)
            logits = None
            if k == last:
                logits = model.finish(ctx, h, pending, want_rows, n_want)
                if post is not None and logits is not None:
                    post(logits)
            return h, pending, logits

        def handoff(pending, expect):
            """An eager piece's output at the address the next graph was captured with."""
            if (pending is None) != (expect is None):
                raise RuntimeError("a part that runs outside the CUDA graphs returned a tensor in one step and "
                                   "None in another; the graphs after it were captured for one of the two")
            if pending is None:
                return None
            if pending.dim() == 3:
                pending = pending.sum(0).to(self.dtype)
            buf = ctx.ws.buf("handoff", pending.shape[0], pending.shape[1], pending.dtype)
            if buf.data_ptr() != pending.data_ptr():
                buf.copy_(pending)
            return buf

        state = self._graphs.get(key)
        h = pending = logits = None
        if state is None:                                   # first meeting: this is the real step, run eagerly
            for k in range(len(pieces)):
                h, pending, logits = body(k, h, pending)
            self._graphs[key] = "warm"
            self.eager_steps += 1
            return logits
        if state == "warm":                                 # second meeting: capture piece by piece
            recs = []
            for k, (safe, _) in enumerate(pieces):
                if safe:
                    graph = torch.cuda.CUDAGraph(keep_graph=self.keep_graphs)
                    with torch.cuda.graph(graph):
                        h, pending, logits = body(k, h, pending)
                    if self.keep_graphs:
                        graph.instantiate()
                    graph.replay()
                    recs.append((graph, h, pending, logits))
                else:
                    h, pending, logits = body(k, h, pending)
                    pending = handoff(pending, pending)
                    recs.append(("eager", pending))
            self._graphs[key] = recs
            self.graph_replays += 1
            return logits
        for k, rec in enumerate(state):
            if rec[0] == "eager":
                h, pending, logits = body(k, h, pending)
                pending = handoff(pending, rec[1])
            else:
                rec[0].replay()
                _, h, pending, logits = rec
        self.graph_replays += 1
        return logits

    def _fuse_rows(self, n_rows: int) -> bool:
        from ..csrc import ops
        return (self._on_cuda and self.dtype == torch.bfloat16 and ops.GEMM_BACKEND == "sm100"
                and ops.FUSE_RED and n_rows <= ops.FUSE_MAX_ROWS)

    def _apply_feed(self, ctx) -> None:
        """Overwrite fed rows of the step's tokens with tokens that are still on the device."""
        if self._feed is None:
            return
        from ..csrc import ops
        src, idx = self._feed
        n = len(idx)
        feed_dev = self._feed_dev[:n]
        ri = self._feed_next
        self._feed_next = (ri + 1) % len(self._feed_ring)
        if self._feed_used[ri] and self._on_cuda:
            self._feed_events[ri].synchronize()
        host = self._feed_ring[ri]
        host[:n] = torch.as_tensor(idx, dtype=torch.int32)
        feed_dev.copy_(host[:n], non_blocking=True)
        if self._on_cuda:
            self._feed_events[ri].record()
            self._feed_used[ri] = True
        ops.gather_tokens(ctx.tokens[:n], src, feed_dev)
        self._feed = None

    def _prepare_decode(self, entries: Sequence[StepEntry], pad_to: int, feed_idx=None):
        """`_prepare` for the common decode-only step (every request live, one token each, no
        windowed group), with array operations instead of per-entry loops.  Returns None when
        the step is not of that kind."""
        cache = self.cache
        reqs = cache._req
        if cache.windowed:
            return None
        recs = []
        for e in entries:
            r = reqs.get(e.req_id)
            if r is None:
                return None
            recs.append(r)
        R = len(entries)
        if len({id(r) for r in recs}) != R:
            raise StepError("a request appears twice in one step")
        V = self.model.spec.vocab_size
        toks = np.fromiter((e.tokens[0] for e in entries), dtype=np.int64, count=R)
        if (toks < 0).any() or (toks >= V).any():
            raise StepError(f"a token is outside the vocabulary (0..{V - 1})")
        for e in entries:
            if len(e.want) and (len(e.want) != 1 or int(e.want[0]) != 0):
                raise StepError(f"request {e.req_id!r}: wanted place outside its one token")
        lens = np.fromiter((r.length for r in recs), dtype=np.int32, count=R)
        slots = np.fromiter((r.slot for r in recs), dtype=np.int32, count=R)
        if R > self.max_requests or int(lens.max()) + 1 > self.max_seq_len:
            raise StepError("step exceeds max_requests or a request would pass its capacity")
        grow = np.nonzero(lens % cache.page_size == 0)[0]
        if len(grow):
            for pool in cache.pools:
                if len(grow) > pool.free:
                    raise OutOfPages(f"step needs {len(grow)} more pages, {pool.free} free")
            for i in grow:
                cache.extend(entries[int(i)].req_id, 1)
        P = pad_to
        ri = self._ring_next
        self._ring_next = (ri + 1) % len(self._ring)
        if self._ring_used[ri] and self._on_cuda:
            self._ring_events[ri].synchronize()
        host = self._ring[ri]
        hp = host.numpy()
        n_groups = len(cache.pools)
        off = 0
        spans = []
        # the layout of `_prepare(pad_to=P)` (graphs captured from either are replayed for both),
        # then the indices of the token feed
        for n in (P, P, P, P + 1, P, P, P) + (P * self.stride,) * n_groups + (P,):
            spans.append((off, off + n))
            off += n
        s_tok, s_pos, s_re, s_cu, s_ctx, s_slot, s_want = spans[:7]
        s_tab, s_feed = spans[7:-1], spans[-1]
        hp[s_feed[0]:s_feed[1]] = -1                       # rows whose token a sampler left on the device
        if feed_idx is not None:
            hp[s_feed[0]:s_feed[0] + R] = np.asarray(feed_idx, dtype=np.int32)
        hp[s_tok[0]:s_tok[0] + R] = toks
        hp[s_tok[0] + R:s_tok[1]] = 0
        hp[s_pos[0]:s_pos[0] + R] = lens
        hp[s_pos[0] + R:s_pos[1]] = 0
        hp[s_re[0]:s_re[0] + R] = np.arange(R, dtype=np.int32)
        hp[s_re[0] + R:s_re[1]] = -1
        hp[s_cu[0]:s_cu[0] + R] = np.arange(R, dtype=np.int32)
        hp[s_cu[0] + R:s_cu[1]] = R
        hp[s_ctx[0]:s_ctx[0] + R] = lens
        hp[s_ctx[0] + R:s_ctx[1]] = 0
        hp[s_slot[0]:s_slot[0] + R] = slots
        hp[s_slot[0] + R:s_slot[1]] = 0
        hp[s_want[0]:s_want[1]] = np.arange(P, dtype=np.int32)
        for g, st in enumerate(s_tab):
            tab = hp[st[0]:st[1]].reshape(P, self.stride)
            tab[:R] = cache.table_rows[g][slots]
            tab[R:] = -1
        self._dev[:off].copy_(host[:off], non_blocking=True)
        self.last_meta_words = off
        if self._on_cuda:
            self._ring_events[ri].record()
            self._ring_used[ri] = True
        d = self._dev
        lens_l = lens.tolist()
        ctx = StepContext(
            n_rows=P, n_entries=P, max_q=1,
            tokens=d[s_tok[0]:s_tok[1]], positions=d[s_pos[0]:s_pos[1]], row_entry=d[s_re[0]:s_re[1]],
            cu_q=d[s_cu[0]:s_cu[1]], ctx_before=d[s_ctx[0]:s_ctx[1]], slots=d[s_slot[0]:s_slot[1]],
            status=self.status, ws=self.ws, dtype=self.dtype, q_lens=[1] * R, ctx_lens=lens_l,
            slot_ids=slots.tolist())
        self._tables = [d[st[0]:st[1]].view(P, self.stride) for st in s_tab]
        self._feed_idx = d[s_feed[0]:s_feed[1]]
        return ctx, d[s_want[0]:s_want[1]], P

    def _prepare(self, entries: Sequence[StepEntry], pad_to: int = 0, pads=None):
        """Validate, take pages, pack and upload the batch description.  ``pad_to`` (decode-only
        steps) pads rows and entries to a fixed count so that the layout does not depend on
        the batch: padding rows belong to no entry (row_entry -1), padding entries have no rows,
        and every row's logits are computed.  ``pads = (rows, entries, wanted rows)`` pads a step of
        any mix the same way; the wanted rows keep their places and the padding repeats row 0."""
        if not entries:
            raise StepError("a step needs at least one entry")
        V = self.model.spec.vocab_size
        seen = set()
        n_rows = 0
        for e in entries:
            if e.req_id in seen:
                raise StepError(f"request {e.req_id!r} appears twice in one step")
            seen.add(e.req_id)
            if len(e.tokens) == 0:
                raise StepError(f"request {e.req_id!r} brings no tokens")
            for t in e.tokens:
                if not (0 <= int(t) < V):
                    raise StepError(f"request {e.req_id!r}: token {t} is outside the vocabulary (0..{V - 1})")
            for w in e.want:
                if not (0 <= int(w) < len(e.tokens)):
                    raise StepError(f"request {e.req_id!r}: wanted place {w} is outside its {len(e.tokens)} tokens")
            if len(set(int(w) for w in e.want)) != len(e.want):
                raise StepError(f"request {e.req_id!r}: a wanted place is named twice")
            n_rows += len(e.tokens)
        if n_rows > self.max_tokens_per_step:
            raise StepError(f"step of {n_rows} tokens exceeds max_tokens_per_step = {self.max_tokens_per_step}")
        if len(entries) > self.max_requests:
            raise StepError(f"step of {len(entries)} requests exceeds max_requests = {self.max_requests}")
        new = [e.req_id for e in entries if not self.cache.is_live(e.req_id)]
        if len(new) > self.cache.slots_free():
            raise StepError(f"{len(new)} new requests but {self.cache.slots_free()} free slots")
        # room for every entry, or nothing is taken
        demand = [0] * len(self.cache.pools)
        for e in entries:
            n = len(e.tokens)
            if e.req_id in new:
                length, take, freed = 0, [-(-n // self.cache.page_size)] * len(demand), [0] * len(demand)
            else:
                length = self.cache.length(e.req_id)
                take, freed = self.cache.pages_to_take(e.req_id, n), self.cache.pages_freed_first(e.req_id)
            if length + n > self.max_seq_len:
                raise StepError(f"request {e.req_id!r} would reach {length + n} tokens; capacity {self.max_seq_len}")
            for g in range(len(demand)):
                demand[g] += take[g] - freed[g]
        for g, pool in enumerate(self.cache.pools):
            if demand[g] > pool.free:
                raise OutOfPages(f"step needs {demand[g]} more pages in group {g}, {pool.free} free")
        for r in new:
            self.admit(r)
        for e in entries:
            self.cache.extend(e.req_id, len(e.tokens))

        R, N = len(entries), n_rows
        W = sum(len(e.want) for e in entries)
        R_real, N_real, W_real = R, N, W
        if pad_to:
            R = N = W = pad_to
        elif pads:
            N, R, W = pads
            if N < N_real or R < R_real or W < W_real:
                raise StepError("the padded shape is smaller than the step")
        ri = self._ring_next
        self._ring_next = (ri + 1) % len(self._ring)
        if self._ring_used[ri] and self._on_cuda:
            self._ring_events[ri].synchronize()
        host = self._ring[ri]
        hp = host.numpy()
        off = 0

        def take_(n):
            nonlocal off
            v = (off, off + n)
            off += n
            return v

        s_tok, s_pos, s_re = take_(N), take_(N), take_(N)
        s_cu, s_ctx, s_slot, s_want = take_(R + 1), take_(R), take_(R), take_(W)
        s_tab = [take_(R * self.stride) for _ in self.cache.pools]
        row = 0
        wi = s_want[0]
        q_lens, ctx_lens, slot_ids = [], [], []
        for i, e in enumerate(entries):
            n = len(e.tokens)
            length = self.cache.length(e.req_id)
            hp[s_tok[0] + row: s_tok[0] + row + n] = np.asarray(e.tokens, dtype=np.int32)
            hp[s_pos[0] + row: s_pos[0] + row + n] = np.arange(length, length + n, dtype=np.int32)
            hp[s_re[0] + row: s_re[0] + row + n] = i
            hp[s_cu[0] + i] = row
            hp[s_ctx[0] + i] = length
            hp[s_slot[0] + i] = self.cache.slot(e.req_id)
            if not pad_to:
                for w in e.want:
                    hp[wi] = row + int(w)
                    wi += 1
            for g, s in enumerate(s_tab):
                t = self.cache.table(e.req_id, g)
                base = s[0] + i * self.stride
                hp[base: base + len(t)] = t
                hp[base + len(t): base + self.stride] = -1
            q_lens.append(n)
            ctx_lens.append(length)
            slot_ids.append(self.cache.slot(e.req_id))
            row += n
        hp[s_cu[0] + R_real: s_cu[0] + R + 1] = row
        if pad_to or pads:
            hp[s_tok[0] + N_real: s_tok[1]] = 0
            hp[s_pos[0] + N_real: s_pos[1]] = 0
            hp[s_re[0] + N_real: s_re[1]] = -1
            hp[s_ctx[0] + R_real: s_ctx[1]] = 0
            hp[s_slot[0] + R_real: s_slot[1]] = 0
            if pad_to:
                hp[s_want[0]: s_want[1]] = np.arange(W, dtype=np.int32)
            else:
                hp[s_want[0] + W_real: s_want[1]] = 0
            for st in s_tab:
                hp[st[0] + R_real * self.stride: st[1]] = -1
        self._dev[:off].copy_(host[:off], non_blocking=True)
        self.last_meta_words = off
        if self._on_cuda:
            self._ring_events[ri].record()
            self._ring_used[ri] = True
        d = self._dev
        ctx = StepContext(
            n_rows=N, n_entries=R, max_q=N if pads else max(q_lens),
            tokens=d[s_tok[0]:s_tok[1]], positions=d[s_pos[0]:s_pos[1]], row_entry=d[s_re[0]:s_re[1]],
            cu_q=d[s_cu[0]:s_cu[1]], ctx_before=d[s_ctx[0]:s_ctx[1]], slots=d[s_slot[0]:s_slot[1]],
            status=self.status, ws=self.ws, dtype=self.dtype, q_lens=q_lens, ctx_lens=ctx_lens, slot_ids=slot_ids)
        self._tables = [d[s[0]:s[1]].view(R, self.stride) for s in s_tab]
        return ctx, (d[s_want[0]:s_want[1]] if W else None), W

    def _cache_views(self, ctx: StepContext) -> List[object]:
        views = []
        st = self.storage
        for e in self.model.spec.schedule:
            lc = st.layers[e.cache]
            if lc.kind == "paged":
                views.append(PagedView(st.k[lc.group][lc.index], st.v[lc.group][lc.index],
                                       self._tables[lc.group], writes=e.writes))
            elif lc.kind == "slot":
                views.append(SlotView(st.state[lc.group][lc.index]))
            else:
                views.append(None)
        return views

    def check_status(self) -> None:
        """Raise if a kernel recorded an error bit (synchronises)."""
        from ..csrc import ops
        bits = int(self.status.item())
        if self._on_cuda:
            bits |= ops.gemm_status(self.device)
        if bits:
            self.status.zero_()
            raise StepError(f"a kernel reported status bits {bits:#x} (1 bad token, 2 bad page, 4 bad position, 8 a bounded wait of the tensor-core product ran out)")

    def graph_kernel_nodes(self) -> Dict[tuple, int]:
        """Kernel nodes of every captured graph, asked from the CUDA runtime (``keep_graphs`` must
        have been set before the captures): what one replay launches."""
        import ctypes
        rt = ctypes.CDLL("libcudart.so.12")
        out = {}
        for key, state in self._graphs.items():
            if state == "warm":
                continue
            kernels = 0
            for rec in state:
                if rec[0] == "eager":
                    continue
                g = ctypes.c_void_p(rec[0].raw_cuda_graph())
                n = ctypes.c_size_t(0)
                if rt.cudaGraphGetNodes(g, None, ctypes.byref(n)) != 0 or n.value == 0:
                    continue
                nodes = (ctypes.c_void_p * n.value)()
                rt.cudaGraphGetNodes(g, nodes, ctypes.byref(n))
                for node in nodes:
                    t = ctypes.c_int(-1)
                    rt.cudaGraphNodeGetType(ctypes.c_void_p(node), ctypes.byref(t))
                    kernels += t.value == 0                     # cudaGraphNodeTypeKernel
            out[key] = kernels
        return out

    def stats(self) -> Dict[str, object]:
        return {"steps": self.steps_run, "tokens": self.tokens_run, "eager_steps": self.eager_steps,
                "pages_free": self.cache.pages_free(),
                "slots_free": self.cache.slots_free(), "live_requests": len(self.cache.live_requests()),
                "cache_bytes": self.storage.nbytes(), "workspace_bytes": self.ws.nbytes(),
                "graphs": sum(1 for g in self._graphs.values() if g != "warm"), "graph_replays": self.graph_replays}
