"""neurogrid_b200: a small, whole inference engine for one B200, built from parts.

One architecture is registered (``Lfm2ForCausalLM``: gated short-convolution layers
interleaved with grouped-query attention).  The public entry points are
:class:`neurogrid_b200.Engine` (generate), ``bin/neurogrid`` (command line) and
``bin/trace_run`` (token-by-token replay that writes logits).
"""
__version__ = "0.1.0"


def __getattr__(name):
    if name in ("Engine", "SamplingParams"):
        from .engine import api
        return getattr(api, name)
    raise AttributeError(name)
