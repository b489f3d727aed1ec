"""Which libraries a model needs, so that a first call compiles those (side by side) and no others."""
from __future__ import annotations

from typing import List, Mapping, Optional, Tuple

import torch

Job = Tuple[str, Optional[Mapping[str, object]]]


def flagship_specialisations() -> List[Job]:
    """The ``-D`` specialisations of the published LFM2 shapes (head_dim 64)."""
    return [("attention_bf16", {"NG_HEAD_DIM": 64}), ("shortconv", {"NG_CONV_L": 3}), ("rope_cache", {"NG_ROPE_PAIRS": 1})]


def needed_by(model) -> List[Job]:
    """Libraries the bound model can launch in its compute dtype (the sampler's included)."""
    jobs: List[Job] = [("elementwise", None), ("sampling", None)]
    bf16 = model.dtype == torch.bfloat16
    jobs.append(("gemm_sm100", None) if bf16 else ("gemm_f32", None))
    for block in model.blocks:
        mixer = getattr(block, "mixer", None)
        name = type(mixer).__name__
        if name == "ShortConv":
            jobs.append(("shortconv", {"NG_CONV_L": mixer.spec.width}))
        elif name == "Attention":
            s = mixer.spec
            jobs.append(("rope_cache", {"NG_ROPE_PAIRS": 1 if s.head_dim <= 64 else 2 if s.head_dim <= 128 else 4}))
            if bf16 and s.n_heads // s.n_kv_heads <= 16:
                jobs.append(("attention_bf16", {"NG_HEAD_DIM": s.head_dim}))
                if s.head_dim == 64:
                    jobs.append(("attention_sm100", None))
            else:
                jobs.append(("attention_generic", None))
    seen, out = set(), []
    for name, d in jobs:
        key = (name, tuple(sorted((d or {}).items())))
        if key not in seen:
            seen.add(key)
            out.append((name, d))
    return out
