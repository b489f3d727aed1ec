"""A decoder-only language model assembled from a :class:`ModelSpec`.

Nothing here names an architecture: the embedding, the blocks (built through the part
registries), the order in which they run (``spec.schedule``), the final norm and the output
head are all read from the spec.  The head shares the embedding's storage when the spec
ties them (the reference uploads the table twice, pkg/inference/engine_gpu.go:52-69).
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..config.specs import ModelSpec
from ..csrc import ops
from ..parts import registry
from ..parts.base import StepContext
from ..weights.decl import TensorDecl


class Decoder:
    def __init__(self, spec: ModelSpec, *, dtype: torch.dtype, device):
        if dtype not in (torch.float32, torch.bfloat16):
            raise ValueError(f"compute dtype must be float32 or bfloat16, got {dtype}")
        self.spec, self.dtype, self.device = spec, dtype, device
        writers = {e.layer for e in spec.schedule if e.writes}
        self.blocks = []
        for i, layer in enumerate(spec.layers):
            kw = dict(dtype=dtype, device=device)
            if i not in writers and any(e.layer == i for e in spec.schedule):
                kw["owns_cache"] = False        # only ever reads another entry's keys and values
            self.blocks.append(registry.build("block", _BlockSpec(layer), **kw))
        self.final_norm = registry.build("norm", spec.final_norm, dtype=dtype, device=device)
        self.embed_table: Optional[torch.Tensor] = None
        self.head_weight: Optional[torch.Tensor] = None
        self.position_table: Optional[torch.Tensor] = None

    # ------------------------------------------------------------------ weights
    def tensors(self) -> Dict[str, TensorDecl]:
        s = self.spec
        out = {s.embed_name: TensorDecl((s.vocab_size, s.hidden))}
        for layer, block in zip(s.layers, self.blocks):
            for name, decl in block.tensors().items():
                out[layer.prefix + name] = decl
        for name, decl in self.final_norm.tensors().items():
            out[_join(s.final_norm_name, name)] = decl
        if not s.tie_head:
            out[s.head_name] = TensorDecl((s.vocab_size, s.hidden))
        if s.position_table_name:
            out[s.position_table_name] = TensorDecl((s.max_positions, s.hidden))
        return out

    def bind(self, weights: Dict[str, torch.Tensor]) -> None:
        s = self.spec
        kw = dict(device=self.device, dtype=self.dtype)
        self.embed_table = weights[s.embed_name].to(**kw).contiguous()
        self.head_weight = self.embed_table if s.tie_head else weights[s.head_name].to(**kw).contiguous()
        self.position_table = weights[s.position_table_name].to(**kw).contiguous() if s.position_table_name else None
        for layer, block in zip(s.layers, self.blocks):
            pre = layer.prefix
            block.bind({k[len(pre):]: v for k, v in weights.items() if k.startswith(pre)})
        base = s.final_norm_name[: -len("weight")] if s.final_norm_name.endswith("weight") else s.final_norm_name + "."
        self.final_norm.bind({k[len(base):]: v for k, v in weights.items() if k.startswith(base)})

    def cache_needs(self) -> Dict[int, object]:
        """Cache id -> what the layers that use it need to keep between steps."""
        needs: Dict[int, object] = {}
        for e in self.spec.schedule:
            need = self.blocks[e.layer].cache_need()
            if e.cache in needs and needs[e.cache] != need:
                raise ValueError(f"schedule entry {e}: cache {e.cache} is shared by layers with different needs")
            if not e.writes and type(need).__name__ != "PagedNeed":
                raise ValueError(f"schedule entry {e}: only paged keys and values can be read by another layer")
            needs[e.cache] = need
        return needs

    def kernels(self):
        """Libraries of this package the model launches: the embedding's and the head's, and what
        every part declares (``kernels()``; a part that declares nothing launches nothing here)."""
        jobs = [("elementwise", None), ("gemm_sm100" if self.dtype == torch.bfloat16 else "gemm_f32", None)]
        for part in list(self.blocks) + [self.final_norm]:
            jobs += getattr(part, "kernels", list)()
        return jobs

    def activation_bytes_per_row(self) -> int:
        """An upper estimate of the workspace one row of a step takes: the float32 stream, the
        normed rows, and every matrix product's output of the widest block (doubled: a part also
        holds a few buffers of such widths that are no product's output).  Used to leave room for
        the workspaces when the page pool is sized from the free device memory."""
        e = torch.empty((), dtype=self.dtype).element_size()
        widest = max((sum(d.shape[0] for d in b.tensors().values() if len(d.shape) == 2) for b in self.blocks),
                     default=0)
        # scratch that a part keeps per row besides its products' outputs (a part says so with scratch_bytes_per_row())
        extra = max((getattr(part, "scratch_bytes_per_row", lambda: 0)() for b in self.blocks for part in (b.mixer, b.ffn)),
                    default=0)
        return 8 * self.spec.hidden + e * self.spec.hidden + 2 * e * widest + extra

    def weight_bytes(self) -> int:
        seen, total = set(), 0
        for t in self._all_tensors():
            if t.data_ptr() not in seen:
                seen.add(t.data_ptr())
                total += t.numel() * t.element_size()
        return total

    def _all_tensors(self):
        def walk(o, depth=0):
            if isinstance(o, torch.Tensor):
                yield o
            elif depth < 4 and hasattr(o, "__dict__"):
                for v in vars(o).values():
                    yield from walk(v, depth + 1)
            elif isinstance(o, (list, tuple)) and depth < 4:
                for v in o:
                    yield from walk(v, depth + 1)
        yield from walk(self.blocks)
        yield from walk(self.final_norm)
        yield self.embed_table
        if self.head_weight is not self.embed_table:
            yield self.head_weight

    # ------------------------------------------------------------------ forward
    def forward(self, ctx: StepContext, caches: List[object], want_rows: Optional[torch.Tensor],
                n_want: int) -> Optional[torch.Tensor]:
        """Run the step's rows through the scheduled layers; float32 logits [n_want, vocab]
        for the rows listed in ``want_rows`` (None when nothing is wanted)."""
        h = self.begin(ctx)
        pending = self.run_entries(ctx, caches, range(len(self.spec.schedule)), h, None)
        return self.finish(ctx, h, pending, want_rows, n_want)

    # The same in pieces, for a caller that runs some stretches of the schedule as CUDA graphs and
    # others (parts that are not ``graph_safe``) eagerly between them.
    def begin(self, ctx: StepContext) -> torch.Tensor:
        """The float32 residual stream [N, H] holding the embeddings of the step's tokens."""
        s = self.spec
        h = ctx.ws.buf("residual", ctx.n_rows, s.hidden, torch.float32)
        ops.embed(self.embed_table, ctx.tokens, h, ctx.status)
        if self.position_table is not None:                  # learned absolute positions: h += table[position]
            ops.embed(self.position_table, ctx.positions, h, ctx.status, accumulate=True)
        return h

    def run_entries(self, ctx: StepContext, caches: List[object], entries, h: torch.Tensor, pending):
        """Schedule entries ``entries`` (indices), in order; takes and returns the feed-forward
        output that is not yet added to the stream."""
        sched = self.spec.schedule
        for i in entries:
            pending = self.blocks[sched[i].layer].forward(h, pending, ctx, caches[i])
        return pending

    def finish(self, ctx: StepContext, h: torch.Tensor, pending, want_rows: Optional[torch.Tensor],
               n_want: int) -> Optional[torch.Tensor]:
        s = self.spec
        if n_want == 0:
            if pending is not None:
                ops.residual_add(h, pending)     # keeps the stream whole for callers that inspect it
            return None
        x = ctx.ws.buf("head_in", n_want, s.hidden, self.dtype)
        self.final_norm.forward(h, pending, x, rows=want_rows)
        logits = ctx.ws.buf("logits", n_want, s.vocab_size, torch.float32)
        ops.linear(x, self.head_weight, None, logits)
        return logits

    def graph_pieces(self):
        """The schedule cut into stretches that can be captured in a CUDA graph and stretches that
        cannot: [(safe, [schedule indices])].  The embedding belongs to the first piece and the
        final norm with the head to the last (a final norm that is not graph-safe gets an empty
        unsafe piece of its own at the end)."""
        pieces: List[list] = []
        for i, e in enumerate(self.spec.schedule):
            safe = bool(getattr(self.blocks[e.layer], "graph_safe", False))
            if pieces and pieces[-1][0] == safe:
                pieces[-1][1].append(i)
            else:
                pieces.append([safe, [i]])
        if not pieces or pieces[0][0] is False:
            pieces.insert(0, [True, []])                     # the embedding alone
        tail_safe = bool(getattr(self.final_norm, "graph_safe", False))
        if pieces[-1][0] != tail_safe:
            pieces.append([tail_safe, []])
        return [(s, idx) for s, idx in pieces]


class _BlockSpec:
    """Adapter: a LayerSpec seen as the spec of its block arrangement."""

    def __init__(self, layer):
        self.kind = layer.block
        self.mixer, self.ffn = layer.mixer, layer.ffn
        self.mixer_norm, self.ffn_norm = layer.mixer_norm, layer.ffn_norm
        self.names = layer.names


def _join(full_name: str, rel: str) -> str:
    # the final norm's file name is given whole ("model.embedding_norm.weight"): a norm's other tensors stand beside it
    if full_name.endswith("weight"):
        return full_name[: -len("weight")] + rel
    return f"{full_name}.{rel}"
