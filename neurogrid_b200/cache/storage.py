"""Device memory behind the cache manager's bookkeeping.

Layers with the same need share a group.  A paged group holds, for each of its layers,
keys and values as ``[pages, n_kv_heads, page_size, head_dim]`` in the compute dtype; one
page id is valid in every layer of its group.  A slot group holds ``[layers, slots, *shape]``
in the element type its need names, set to the need's initial value when a request starts.  The reference keeps one pool per attention layer in fp16
(gpu/cuda/paged_attention.cu:34-67) and conv states on the host between steps.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from .manager import PagedNeed, SlotNeed


_SLOT_DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16, "float16": torch.float16, "int32": torch.int32}


@dataclass
class LayerCache:
    kind: str                 # "paged" | "slot" | "none"
    group: int = -1           # index among groups of its kind
    index: int = -1           # layer's index inside the group


class CacheStorage:
    def __init__(self, needs: Sequence[object], *, pages_per_group, page_size: int, max_requests: int,
                 dtype: torch.dtype, device):
        """``needs`` maps a cache id to its PagedNeed / SlotNeed / None.  ``pages_per_group`` is
        an int (every paged group gets that many pages) or a callable ``need -> pages``."""
        self.page_size, self.dtype, self.device = page_size, dtype, device
        self.paged_needs: List[PagedNeed] = []
        self.slot_needs: List[SlotNeed] = []
        self.layers: Dict[int, LayerCache] = {}
        counts_p: List[int] = []
        counts_s: List[int] = []
        for cid in sorted(needs):
            need = needs[cid]
            if need is None:
                self.layers[cid] = LayerCache("none")
            elif isinstance(need, PagedNeed):
                if need not in self.paged_needs:
                    self.paged_needs.append(need)
                    counts_p.append(0)
                g = self.paged_needs.index(need)
                self.layers[cid] = LayerCache("paged", g, counts_p[g])
                counts_p[g] += 1
            elif isinstance(need, SlotNeed):
                if need not in self.slot_needs:
                    self.slot_needs.append(need)
                    counts_s.append(0)
                g = self.slot_needs.index(need)
                self.layers[cid] = LayerCache("slot", g, counts_s[g])
                counts_s[g] += 1
            else:
                raise TypeError(f"a layer declared an unknown cache need: {need!r}")
        self.pages_per_group = [pages_per_group(n) if callable(pages_per_group) else int(pages_per_group)
                                for n in self.paged_needs]
        self.k: List[torch.Tensor] = []
        self.v: List[torch.Tensor] = []
        for need, n_layers, pages in zip(self.paged_needs, counts_p, self.pages_per_group):
            shape = (n_layers, pages, need.n_kv_heads, page_size, need.head_dim)
            self.k.append(torch.zeros(shape, dtype=dtype, device=device))
            self.v.append(torch.zeros(shape, dtype=dtype, device=device))
        for need in self.slot_needs:
            if need.dtype not in _SLOT_DTYPES:
                raise TypeError(f"a layer asks for state of dtype {need.dtype!r}; one of {sorted(_SLOT_DTYPES)}")
        self.state: List[torch.Tensor] = [
            torch.full((n_layers, max_requests) + tuple(need.shape), need.init, dtype=_SLOT_DTYPES[need.dtype],
                       device=device)
            for need, n_layers in zip(self.slot_needs, counts_s)]

    def reset_slot(self, slot: int) -> None:
        """Every layer's state of the slot back to its need's initial value (a request starts)."""
        for s, need in zip(self.state, self.slot_needs):
            s[:, slot].fill_(need.init)

    def bytes_per_token(self) -> int:
        esz = torch.empty((), dtype=self.dtype).element_size()
        return sum(2 * k.shape[0] * n.n_kv_heads * n.head_dim * esz for k, n in zip(self.k, self.paged_needs))

    def nbytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self.k + self.v + self.state)
