"""What a part asks of the weight files: a name, a shape, a class of dtype, a way to
draw it at random.  Parts produce these; the loader and the random-weights writer consume them."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Tuple


@dataclass(frozen=True)
class TensorDecl:
    shape: Tuple[int, ...]
    init: str = "matrix"       # matrix | conv | norm | bias  (how random weights are drawn)
    integer: bool = False      # an integer table (kept as int32) rather than a float tensor

    def __post_init__(self):
        if self.init not in ("matrix", "conv", "norm", "bias", "zeros"):
            raise ValueError(f"unknown init {self.init!r}")
