"""Random-weights mode: draw every declared tensor from a seed, or write a whole model folder.

Distributions: matrices N(0, 0.02); short-conv kernels N(0, 0.2); norm weights 1 + N(0, 0.1);
biases N(0, 0.02).  Tensors are drawn in sorted-name order from one generator, so a
(configuration, seed) pair names one model.  The reference has random weights only for its
INT8 Llama layer (``gpu/engine/layer.cu:260-386``).
"""
from __future__ import annotations

import json
import os
from typing import Dict, Mapping

import torch

from .decl import TensorDecl
from .safetensors_io import write_file

_STD = {"matrix": 0.02, "conv": 0.2, "norm": 0.1, "bias": 0.02}


def draw(decls: Mapping[str, TensorDecl], seed: int, *, dtype=torch.bfloat16, device="cpu") -> Dict[str, torch.Tensor]:
    gen = torch.Generator(device=device)
    gen.manual_seed(int(seed))
    out: Dict[str, torch.Tensor] = {}
    for name in sorted(decls):
        d = decls[name]
        if d.integer:
            out[name] = torch.zeros(d.shape, dtype=torch.int32, device=device)
            continue
        if d.init == "zeros":
            out[name] = torch.zeros(d.shape, dtype=dtype, device=device)
            continue
        t = torch.empty(d.shape, dtype=torch.float32, device=device).normal_(0.0, _STD[d.init], generator=gen)
        if d.init == "norm":
            t += 1.0
        out[name] = t.to(dtype)
    return out


def write_random_model(config_dict: Mapping, seed: int, folder: str, *, dtype=torch.bfloat16) -> str:
    """Write ``config.json`` and ``model.safetensors`` for the configuration; returns ``folder``."""
    from ..config import config_from_dict
    from ..models import declare_tensors

    cfg = config_from_dict(config_dict)
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(dict(config_dict), f, indent=1)
    tensors = draw(declare_tensors(cfg.model_spec()), seed, dtype=dtype)
    write_file(os.path.join(folder, "model.safetensors"), tensors,
               metadata={"format": "pt", "seed": str(int(seed))})
    return folder
