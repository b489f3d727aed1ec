"""RMSNorm with the residual sum fused in front of it."""
from __future__ import annotations

import torch

from ..csrc import ops
from ..weights.decl import TensorDecl
from .registry import register


@register("norm", "rmsnorm")
class RMSNorm:
    """y = x * rsqrt(mean(x^2) + eps) * w, everything float32 until the one rounding of y.

    Reference: gpu/cuda/bf16_utils.cu:57-93 (norm), gpu/cuda/kernels.cu:196-262 (fused add).
    """

    graph_safe = True      # launches depend on device data and on launch-time constants only

    def __init__(self, spec, *, dtype, device):
        self.spec, self.dtype, self.device = spec, dtype, device
        self.weight = None

    def tensors(self):
        return {"weight": TensorDecl((self.spec.size,), "norm")}

    def bind(self, t):
        self.weight = t["weight"].to(device=self.device, dtype=torch.float32).contiguous()

    def kernels(self):
        return [("elementwise", None)]

    def forward(self, h, delta, out, rows=None):
        ops.add_rmsnorm(h, delta, self.weight, out, self.spec.eps, rows)
        return out
