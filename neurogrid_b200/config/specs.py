"""Architecture-neutral descriptions of a decoder, produced by a typed model configuration.

A model configuration (one class per architecture, e.g. ``Lfm2Config``) turns the keys of
its ``config.json`` into a :class:`ModelSpec`: a tuple of :class:`LayerSpec` (one per
distinct layer, each naming its mixer, feed-forward, norms and block arrangement by
*spec objects*) and a ``schedule`` that says in which order layers run and whose cache
each run uses.  Parts are built from specs alone; no part sees the model configuration.

Every spec carries ``kind``: the key under which the part class is registered
(:mod:`neurogrid_b200.parts.registry`).  A new part brings its own frozen dataclass with a
``kind`` field; nothing here needs to change for it.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Mapping, Optional, Tuple


def _names(**kw) -> Mapping[str, str]:
    return dict(kw)


@dataclass(frozen=True)
class RMSNormSpec:
    """y = x * rsqrt(mean(x^2) + eps) * w  (weight multiplies directly, no 1+w)."""
    size: int
    eps: float
    kind: str = "rmsnorm"


@dataclass(frozen=True)
class RopeSpec:
    """Rotary position encoding over the whole head.

    ``pairing`` "adjacent" rotates (2i, 2i+1); "half" rotates (i, i+head_dim/2).
    ``scale`` divides positions before the angle is formed (linear position scaling).
    """
    head_dim: int
    theta: float
    pairing: str = "half"
    scale: float = 1.0
    kind: str = "rope"

    def __post_init__(self):
        if self.pairing not in ("adjacent", "half"):
            raise ValueError(f"rope pairing must be 'adjacent' or 'half', got {self.pairing!r}")
        if self.head_dim % 2:
            raise ValueError("rope needs an even head_dim")


@dataclass(frozen=True)
class NoPositionSpec:
    """No position encoding (queries and keys pass unchanged)."""
    kind: str = "none"


@dataclass(frozen=True)
class AttentionSpec:
    """Grouped-query attention over a paged key/value cache.

    ``window`` None = every earlier key is visible; W = only the last W keys (the query's own
    position included).  ``qk_norm`` applies an RMSNorm over head_dim to q and k (weights
    shared by all heads) before the position encoding.
    """
    hidden: int
    n_heads: int
    n_kv_heads: int
    head_dim: int
    position: object
    qk_norm: bool = False
    qk_norm_eps: float = 1e-6
    window: Optional[int] = None
    softmax_scale: Optional[float] = None      # None -> 1/sqrt(head_dim)
    bias: bool = False
    names: Mapping[str, str] = field(default_factory=lambda: _names(
        q="q_proj", k="k_proj", v="v_proj", o="o_proj", q_norm="q_norm", k_norm="k_norm"))
    kind: str = "attention"

    def __post_init__(self):
        if self.n_heads % self.n_kv_heads:
            raise ValueError(f"n_heads {self.n_heads} is not a multiple of n_kv_heads {self.n_kv_heads}")
        if self.head_dim % 16 or not (16 <= self.head_dim <= 256):
            raise ValueError(f"head_dim must be a multiple of 16 in [16, 256], got {self.head_dim}")
        if self.window is not None and self.window < 1:
            raise ValueError("attention window must be >= 1")


@dataclass(frozen=True)
class ShortConvSpec:
    """Gated causal depthwise convolution of width ``width`` (state: last width-1 inputs)."""
    hidden: int
    width: int
    bias: bool = False
    names: Mapping[str, str] = field(default_factory=lambda: _names(
        in_proj="in_proj", conv="conv", out_proj="out_proj"))
    kind: str = "short_conv"

    def __post_init__(self):
        if not (2 <= self.width <= 8):
            raise ValueError(f"short-conv width must be in [2, 8], got {self.width}")


@dataclass(frozen=True)
class SwiGLUSpec:
    """down( silu(gate(x)) * up(x) ), no biases."""
    hidden: int
    intermediate: int
    names: Mapping[str, str] = field(default_factory=lambda: _names(
        gate="gate_proj", up="up_proj", down="down_proj"))
    kind: str = "swiglu"


@dataclass(frozen=True)
class LayerSpec:
    """One decoder layer: a block arrangement around a mixer and a feed-forward.

    ``prefix`` is the tensor-name prefix of the layer; ``names`` maps the four roles
    (mixer, ffn, mixer_norm, ffn_norm) to the sub-prefix used in the weight files.
    """
    mixer: object
    ffn: object
    mixer_norm: object
    ffn_norm: object
    prefix: str
    names: Mapping[str, str]
    block: str = "prenorm"


@dataclass(frozen=True)
class ScheduleEntry:
    """Run ``layer`` (index into ModelSpec.layers) with cache ``cache``.

    Cache ids form a namespace of their own; ``cache == layer`` with ``writes`` is the ordinary
    case.  The same ``layer`` may appear twice (shared weights), each time with a cache id of
    its own.  ``writes=False`` lets a layer read the keys and values that another entry wrote
    under that cache id, without adding its own; such a layer needs no k/v weights.
    """
    layer: int
    cache: int
    writes: bool = True


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    vocab_size: int
    hidden: int
    layers: Tuple[LayerSpec, ...]
    schedule: Tuple[ScheduleEntry, ...]
    final_norm: object
    tie_head: bool
    max_positions: int
    embed_name: str = "model.embed_tokens.weight"
    final_norm_name: str = "model.norm.weight"
    head_name: str = "lm_head.weight"
    eos_token_ids: Tuple[int, ...] = ()
    position_table_name: Optional[str] = None    # a table [max_positions, hidden] of learned positions, added to the
                                                 # token embeddings (no LFM2 configuration has one)

    def __post_init__(self):
        n = len(self.layers)
        if self.position_table_name and self.max_positions <= 0:
            raise ValueError("a table of learned positions needs max_positions")
        writers = set()
        for e in self.schedule:
            if not (0 <= e.layer < n) or e.cache < 0:
                raise ValueError(f"schedule entry {e} names a layer outside 0..{n - 1} or a negative cache id")
            if e.writes:
                if e.cache in writers:
                    raise ValueError(f"schedule entry {e}: cache {e.cache} already has a writer")
                writers.add(e.cache)
            elif e.cache not in writers:
                raise ValueError(f"schedule entry {e} reads cache {e.cache} before any entry writes it")
