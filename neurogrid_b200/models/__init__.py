"""Model construction: spec -> declared tensors -> bound model."""
from __future__ import annotations

from typing import Dict

import torch

from .. import parts as _parts  # noqa: F401  (registers the built-in parts)
from ..config.specs import ModelSpec
from ..weights.decl import TensorDecl
from .decoder import Decoder


def declare_tensors(spec: ModelSpec) -> Dict[str, TensorDecl]:
    """Every tensor the model reads from its weight files, by full name."""
    return Decoder(spec, dtype=torch.float32, device="cpu").tensors()


def build_model(spec: ModelSpec, weights: Dict[str, torch.Tensor], *, dtype: torch.dtype, device) -> Decoder:
    m = Decoder(spec, dtype=dtype, device=device)
    m.bind(weights)
    return m
