"""Bind tensors of a model folder to the names a model declares.

Floating tensors keep the width they are stored with: BF16 stays bfloat16, F32 stays
float32 (F16 and F64 become float32: every F16 value is exact there); integer tables become
int32.  Parts cast what they need for their compute dtype when they bind.  Everything that
is wrong with a folder is reported in ONE error that lists missing tensors, unexpected
tensors, wrong shapes and wrong dtype classes.

The reference binds by exact name as well (``pkg/model/loader.go:406-458,530-600``) but
stops at the first missing tensor (``tensor not found``, ``loader.go:241``) and only warns
about shapes (``loader.go:673-789``).
"""
from __future__ import annotations

from typing import Dict, Mapping

import torch

from .decl import TensorDecl
from .safetensors_io import MappedFiles, index_model_dir


class WeightError(ValueError):
    """The model folder does not hold exactly the tensors the model declares."""

    def __init__(self, model_dir, missing, unexpected, wrong_shape, wrong_dtype):
        self.missing, self.unexpected = list(missing), list(unexpected)
        self.wrong_shape, self.wrong_dtype = list(wrong_shape), list(wrong_dtype)
        lines = [f"weights in {model_dir} do not match the model:"]
        if self.missing:
            lines.append(f"  missing ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        for name, want, got in self.wrong_shape:
            lines.append(f"  wrong shape: {name} expected {list(want)}, file has {list(got)}")
        for name, want, got in self.wrong_dtype:
            lines.append(f"  wrong dtype: {name} expected {want}, file has {got}")
        super().__init__("\n".join(lines))


def _kept_dtype(dt: torch.dtype) -> torch.dtype:
    if dt == torch.bfloat16:
        return torch.bfloat16
    if dt.is_floating_point:
        return torch.float32
    return torch.int32


def load_weights(model_dir: str, decls: Mapping[str, TensorDecl]) -> Dict[str, torch.Tensor]:
    """CPU tensors for every declared name, or one :class:`WeightError`."""
    entries = index_model_dir(model_dir)
    missing = sorted(n for n in decls if n not in entries)
    unexpected = sorted(n for n in entries if n not in decls)
    wrong_shape, wrong_dtype = [], []
    for name, d in decls.items():
        e = entries.get(name)
        if e is None:
            continue
        if tuple(e.shape) != tuple(d.shape):
            wrong_shape.append((name, d.shape, e.shape))
        is_int = not e.dtype.is_floating_point
        if is_int != d.integer:
            wrong_dtype.append((name, "an integer type" if d.integer else "a floating type", str(e.dtype)))
    if missing or unexpected or wrong_shape or wrong_dtype:
        raise WeightError(model_dir, missing, unexpected, wrong_shape, wrong_dtype)
    files = MappedFiles()
    out: Dict[str, torch.Tensor] = {}
    try:
        for name in decls:
            t = files.read(entries[name])
            out[name] = t.to(_kept_dtype(t.dtype))
    finally:
        files.close()
    return out
