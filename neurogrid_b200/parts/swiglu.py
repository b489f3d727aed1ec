"""SwiGLU feed-forward: down( silu(gate x) * up x )."""
from __future__ import annotations

import torch

from ..csrc import ops
from ..weights.decl import TensorDecl
from .registry import register


@register("ffn", "swiglu")
class SwiGLU:
    """Reference: gpu/engine/conv_layer.cu:334-338, gpu/engine/layer.cu:1751-1761 (two GEMMs,
    SiLU, multiply, GEMM).  Gate and up weights are stacked at bind time so that one product
    feeds the gate kernel."""

    graph_safe = True      # launches depend on device data and on launch-time constants only

    def __init__(self, spec, *, dtype, device):
        self.spec, self.dtype, self.device = spec, dtype, device
        self.w_gate_up = self.w_down = None

    def tensors(self):
        s, n = self.spec, self.spec.names
        return {f"{n['gate']}.weight": TensorDecl((s.intermediate, s.hidden)),
                f"{n['up']}.weight": TensorDecl((s.intermediate, s.hidden)),
                f"{n['down']}.weight": TensorDecl((s.hidden, s.intermediate))}

    def bind(self, t):
        n = self.spec.names
        kw = dict(device=self.device, dtype=self.dtype)
        self.w_gate_up = torch.cat([t[f"{n['gate']}.weight"].to(**kw), t[f"{n['up']}.weight"].to(**kw)]).contiguous()
        self.w_down = t[f"{n['down']}.weight"].to(**kw).contiguous()

    def kernels(self):
        return [("gemm_sm100" if self.dtype == torch.bfloat16 else "gemm_f32", None), ("elementwise", None)]

    def forward(self, x, ctx):
        s = self.spec
        n = x.shape[0]
        act = ctx.ws.buf("ffn_act", n, s.intermediate, self.dtype)
        if ops.gemm_sm100_ok(x, self.w_gate_up):
            ops.gemm_swiglu_sm100(x, self.w_gate_up, act)          # the gate rides in the epilogue
        else:
            gu = ctx.ws.buf("ffn_gate_up", n, 2 * s.intermediate, self.dtype)
            ops.linear(x, self.w_gate_up, None, gu)
            ops.swiglu(gu, act)
        return ops.linear_to_residual(act, self.w_down, None, ctx.ws, "ffn_out", residual=ctx.residual)
