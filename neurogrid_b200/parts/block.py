"""Block arrangements: how norms, mixer and feed-forward sit around the residual stream."""
from __future__ import annotations

from . import registry
from .registry import register


@register("block", "prenorm")
class PreNormBlock:
    """r = x + mixer(norm1(x));  y = r + ffn(norm2(r)).

    The residual stream ``h`` is float32.  A block receives the previous block's
    feed-forward output as ``pending`` (not yet added) so that each residual sum rides in the
    norm kernel that follows it; it returns its own feed-forward output the same way.
    Reference: gpu/engine/conv_layer.cu:220,328-341 and gpu/engine/layer.cu:1662-1765.
    """

    def __init__(self, spec, *, dtype, device, owns_cache=True):
        self.spec, self.dtype = spec, dtype
        kw = dict(dtype=dtype, device=device)
        mixer_kw = dict(kw)
        if not owns_cache:
            mixer_kw["owns_cache"] = False
        self.mixer = registry.build("mixer", spec.mixer, **mixer_kw)
        self.ffn = registry.build("ffn", spec.ffn, **kw)
        self.mixer_norm = registry.build("norm", spec.mixer_norm, **kw)
        self.ffn_norm = registry.build("norm", spec.ffn_norm, **kw)

    def parts(self):
        n = self.spec.names
        return {n["mixer"]: self.mixer, n["ffn"]: self.ffn, n["mixer_norm"]: self.mixer_norm,
                n["ffn_norm"]: self.ffn_norm}

    def tensors(self):
        out = {}
        for sub, part in self.parts().items():
            for name, decl in part.tensors().items():
                out[f"{sub}.{name}"] = decl
        return out

    def bind(self, t):
        for sub, part in self.parts().items():
            pre = sub + "."
            part.bind({k[len(pre):]: v for k, v in t.items() if k.startswith(pre)})

    def cache_need(self):
        return self.mixer.cache_need()

    def kernels(self):
        return [job for p in self.parts().values() for job in getattr(p, "kernels", list)()]

    @property
    def graph_safe(self):
        return all(getattr(p, "graph_safe", False) for p in self.parts().values())

    def forward(self, h, pending, ctx, cache):
        n, H = h.shape
        buf = ctx.ws.buf("normed", n, H, self.dtype)
        ctx.residual = h if ctx.fuse_residual else None      # parts may add their output into it and return None
        x = self.mixer_norm.forward(h, pending, buf)
        m = self.mixer.forward(x, ctx, cache)
        x = self.ffn_norm.forward(h, m, buf)
        return self.ffn.forward(x, ctx)
