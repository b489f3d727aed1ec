"""The gated short-convolution mixer."""
from __future__ import annotations

import torch

from ..cache.manager import SlotNeed
from ..csrc import ops
from ..weights.decl import TensorDecl
from .registry import register


@register("mixer", "short_conv")
class ShortConv:
    """in_proj -> [B | C | x];  u = B*x;  c = causal depthwise conv of width L over u;
    y = out_proj(C * c).  State per request: the last L-1 values of u (float32).

    Reference: gpu/engine/conv_layer.cu:222-250,325 (order of the B, C, x split and the two
    gates), gpu/cuda/conv.cu:52-66 (taps: tap L-1 multiplies the current token).  The
    reference ignores ``conv_bias``; here all three parametrised parts carry a bias when it
    is set, the conv's added before the C gate.
    """

    graph_safe = True      # launches depend on device data and on launch-time constants only

    def __init__(self, spec, *, dtype, device):
        self.spec, self.dtype, self.device = spec, dtype, device
        self.w_in = self.b_in = self.w_conv = self.b_conv = self.w_out = self.b_out = None

    def tensors(self):
        s, n = self.spec, self.spec.names
        d = {f"{n['in_proj']}.weight": TensorDecl((3 * s.hidden, s.hidden)),
             f"{n['conv']}.weight": TensorDecl((s.hidden, 1, s.width), "conv"),
             f"{n['out_proj']}.weight": TensorDecl((s.hidden, s.hidden))}
        if s.bias:
            d[f"{n['in_proj']}.bias"] = TensorDecl((3 * s.hidden,), "bias")
            d[f"{n['conv']}.bias"] = TensorDecl((s.hidden,), "bias")
            d[f"{n['out_proj']}.bias"] = TensorDecl((s.hidden,), "bias")
        return d

    def bind(self, t):
        s, n = self.spec, self.spec.names
        kw = dict(device=self.device, dtype=self.dtype)
        f32 = dict(device=self.device, dtype=torch.float32)
        self.w_in = t[f"{n['in_proj']}.weight"].to(**kw).contiguous()
        self.w_out = t[f"{n['out_proj']}.weight"].to(**kw).contiguous()
        self.w_conv = t[f"{n['conv']}.weight"].to(**f32).reshape(s.hidden, s.width).contiguous()
        if s.bias:
            self.b_in = t[f"{n['in_proj']}.bias"].to(**kw).contiguous()
            self.b_out = t[f"{n['out_proj']}.bias"].to(**kw).contiguous()
            self.b_conv = t[f"{n['conv']}.bias"].to(**f32).contiguous()

    def cache_need(self):
        return SlotNeed((self.spec.width - 1, self.spec.hidden))

    def kernels(self):
        return [("gemm_sm100" if self.dtype == torch.bfloat16 else "gemm_f32", None),
                ("shortconv", {"NG_CONV_L": self.spec.width})]

    def forward(self, x, ctx, cache):
        s = self.spec
        n = x.shape[0]
        p = ops.linear_to_residual(x, self.w_in, self.b_in, ctx.ws, "conv_in")
        g = ctx.ws.buf("conv_gated", n, s.hidden, self.dtype)
        ops.shortconv(p, self.w_conv, self.b_conv, cache.state, g, ctx.cu_q, ctx.ctx_before, ctx.slots,
                      ctx.n_entries, ctx.max_q)
        return ops.linear_to_residual(g, self.w_out, self.b_out, ctx.ws, "mixer_out", residual=ctx.residual)
