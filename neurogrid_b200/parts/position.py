"""Position encodings, as parameters of the q/k kernel."""
from __future__ import annotations

import torch

from .base import PositionArgs
from .registry import register


@register("position", "rope")
class Rope:
    """angle(pos, i) = (pos / scale) * theta^(-2i/head_dim); pairs (2i, 2i+1) or (i, i+hd/2).

    Reference: gpu/cuda/bf16_utils.cu:330-378.  The frequencies are formed in float64 on the
    host and rounded once; the angle and its sine and cosine are float32 on the device.
    """

    def __init__(self, spec, *, device):
        self.spec = spec
        i = torch.arange(spec.head_dim // 2, dtype=torch.float64)
        self.inv_freq = (float(spec.theta) ** (-2.0 * i / spec.head_dim)).to(torch.float32).to(device)

    def kernel_args(self):
        return PositionArgs(self.inv_freq, self.spec.pairing == "half", float(self.spec.scale))


@register("position", "none")
class NoPosition:
    def __init__(self, spec, *, device):
        self.spec = spec

    def kernel_args(self):
        return PositionArgs()
