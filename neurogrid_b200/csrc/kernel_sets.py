"""Which libraries a model needs, so that a first call compiles those (side by side) and no others.

Nothing here names a part: every part declares the libraries it launches
(``kernels() -> [(library, defines or None), ...]``, for its compute dtype) and this module
collects what the parts of a model declare.  A part without ``kernels`` (one that launches
nothing of this package) adds nothing.
"""
from __future__ import annotations

from typing import Iterable, List, Mapping, Optional, Tuple

Job = Tuple[str, Optional[Mapping[str, object]]]


def unique(jobs: Iterable[Job]) -> List[Job]:
    seen, out = set(), []
    for name, d in jobs:
        key = (name, tuple(sorted((d or {}).items())))
        if key not in seen:
            seen.add(key)
            out.append((name, d))
    return out


def needed_by(model) -> List[Job]:
    """Libraries the model can launch in its compute dtype, and the sampler's."""
    return unique(list(model.kernels()) + [("sampling", None)])
