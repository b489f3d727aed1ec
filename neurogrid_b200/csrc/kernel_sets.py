"""Which specialised libraries a model needs, so that a first call compiles those and no others."""
from __future__ import annotations

from typing import List, Mapping, Tuple


def flagship_specialisations() -> List[Tuple[str, Mapping[str, object]]]:
    """The ``-D`` specialisations of the published LFM2 shapes (head_dim 64)."""
    return [("attention_bf16", {"NG_HEAD_DIM": 64})]
