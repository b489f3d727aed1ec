"""Typed configuration of the LFM2 hybrid decoder, read from its own ``config.json`` keys.

LFM2 interleaves gated short-convolution layers with grouped-query attention layers; every
layer ends in a SwiGLU feed-forward (pre-norm, two residuals).  The reference reads the same
keys in ``pkg/model/model_config.go:19-49`` and derives the feed-forward width in
``cmd/neurogrid/main.go:831-841``; head_dim, eps fallbacks and tying are at
``cmd/neurogrid/main.go:813-823,857``.

Rotary pairing.  A published LFM2 ``config.json`` has no key for it.  The reference's engine
rotates adjacent pairs (2i, 2i+1) for this family (``pkg/model/model_config.go:93-99``,
``gpu/bindings/gpu.go:1077``), while the model its golden data is generated from
(``scripts/generate_golden_lfm2.py:37-93``) is the checkpoint format's own, which rotates
(i, i + head_dim/2).  Weights are trained for one pairing only, so the default here is the
checkpoint format's ("half"); ``"rope_pairing": "adjacent"`` in config.json selects the
reference engine's.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

from .specs import (AttentionSpec, LayerSpec, ModelSpec, RMSNormSpec, RopeSpec, ScheduleEntry,
                    ShortConvSpec, SwiGLUSpec)


class ConfigError(ValueError):
    """A config.json key is missing, has the wrong type, or contradicts another key."""


def _get(d: Mapping[str, Any], key: str, typ, *, alt: Optional[str] = None, default=None, required=True):
    for k in (key, alt):
        if k is not None and k in d and d[k] is not None:
            v = d[k]
            if typ is float and isinstance(v, int) and not isinstance(v, bool):
                v = float(v)
            if typ is int and isinstance(v, bool):
                raise ConfigError(f"config key {k!r} must be {typ.__name__}, got {v!r}")
            if not isinstance(v, typ):
                raise ConfigError(f"config key {k!r} must be {typ.__name__}, got {v!r}")
            return v
    if required and default is None:
        names = key if alt is None else f"{key!r} (or {alt!r})"
        raise ConfigError(f"config.json lacks required key {names}")
    return default


LAYER_KINDS = ("conv", "full_attention")


@dataclass(frozen=True)
class Lfm2Config:
    vocab_size: int
    hidden_size: int
    num_hidden_layers: int
    layer_types: Tuple[str, ...]
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    intermediate_size: int          # SwiGLU width after any adjustment
    block_ff_dim: int
    block_auto_adjust_ff_dim: bool
    block_multiple_of: int
    block_ffn_dim_multiplier: float
    conv_L_cache: int
    conv_bias: bool
    tie_embedding: bool
    rope_theta: float
    rope_pairing: str
    norm_eps: float
    max_position_embeddings: int    # 0: config.json gives none, the cache alone bounds a request
    eos_token_ids: Tuple[int, ...]
    bos_token_id: Optional[int]
    stored_dtype: Optional[str]

    architecture = "Lfm2ForCausalLM"

    @staticmethod
    def ffn_width(block_ff_dim: int, auto_adjust: bool, multiple_of: int, multiplier: float) -> int:
        """SwiGLU width: with auto-adjust, 2/3 of block_ff_dim, scaled, rounded up to multiple_of."""
        if not auto_adjust:
            return block_ff_dim
        d = int(2 * block_ff_dim / 3)
        d = int(multiplier * d)
        return multiple_of * ((d + multiple_of - 1) // multiple_of)

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "Lfm2Config":
        hidden = _get(d, "hidden_size", int)
        n_layers = _get(d, "num_hidden_layers", int)
        lt = d.get("layer_types")
        if not isinstance(lt, (list, tuple)) or not lt:
            raise ConfigError("config.json lacks required key 'layer_types' (a list of 'conv' / 'full_attention')")
        for i, t in enumerate(lt):
            if t not in LAYER_KINDS:
                raise ConfigError(f"layer_types[{i}] = {t!r}; allowed: {', '.join(LAYER_KINDS)}")
        if len(lt) != n_layers:
            raise ConfigError(f"num_hidden_layers = {n_layers} but layer_types has {len(lt)} entries")
        n_heads = _get(d, "num_attention_heads", int)
        n_kv = _get(d, "num_key_value_heads", int)
        if n_heads <= 0 or n_kv <= 0 or n_heads % n_kv:
            raise ConfigError(f"num_attention_heads = {n_heads} must be a positive multiple of "
                              f"num_key_value_heads = {n_kv}")
        head_dim = _get(d, "head_dim", int, required=False)
        if head_dim is None:
            if hidden % n_heads:
                raise ConfigError(f"hidden_size {hidden} is not divisible by num_attention_heads {n_heads} "
                                  "and no 'head_dim' is given")
            head_dim = hidden // n_heads
        ff = _get(d, "block_ff_dim", int, alt="intermediate_size")
        auto = _get(d, "block_auto_adjust_ff_dim", bool, default=False, required=False)
        mult_of = _get(d, "block_multiple_of", int, required=bool(auto), default=None if auto else 1)
        ffn_mult = _get(d, "block_ffn_dim_multiplier", float, default=1.0, required=False)
        if mult_of <= 0:
            raise ConfigError(f"block_multiple_of must be positive, got {mult_of}")
        inter = cls.ffn_width(ff, bool(auto), mult_of, ffn_mult)
        lc = _get(d, "conv_L_cache", int)
        if lc < 2:
            raise ConfigError(f"conv_L_cache must be >= 2, got {lc}")
        conv_dim = _get(d, "conv_dim", int, required=False)
        if conv_dim is not None and conv_dim != hidden:
            raise ConfigError(f"conv_dim {conv_dim} must equal hidden_size {hidden}")
        tie = bool(d.get("tie_embedding", False)) or bool(d.get("tie_word_embeddings", False))
        eos = d.get("eos_token_id")
        if eos is None:
            eos_ids: Tuple[int, ...] = ()
        elif isinstance(eos, int):
            eos_ids = (eos,)
        elif isinstance(eos, (list, tuple)) and all(isinstance(e, int) for e in eos):
            eos_ids = tuple(eos)
        else:
            raise ConfigError(f"eos_token_id must be an int or a list of ints, got {eos!r}")
        pairing = d.get("rope_pairing", "half")
        if pairing not in ("adjacent", "half"):
            raise ConfigError(f"rope_pairing must be 'adjacent' or 'half', got {pairing!r}")
        # newer exports nest the base under "rope_parameters"; the flat key wins where both stand
        nested = d.get("rope_parameters")
        rope_src = d if d.get("rope_theta") is not None or not isinstance(nested, Mapping) else nested
        cfg = cls(
            vocab_size=_get(d, "vocab_size", int),
            hidden_size=hidden,
            num_hidden_layers=n_layers,
            layer_types=tuple(lt),
            num_attention_heads=n_heads,
            num_key_value_heads=n_kv,
            head_dim=head_dim,
            intermediate_size=inter,
            block_ff_dim=ff,
            block_auto_adjust_ff_dim=bool(auto),
            block_multiple_of=mult_of,
            block_ffn_dim_multiplier=ffn_mult,
            conv_L_cache=lc,
            conv_bias=_get(d, "conv_bias", bool, default=False, required=False),
            tie_embedding=tie,
            rope_theta=_get(rope_src, "rope_theta", float),
            rope_pairing=pairing,
            norm_eps=_get(d, "norm_eps", float, alt="rms_norm_eps"),
            max_position_embeddings=_get(d, "max_position_embeddings", int, default=0, required=False),
            eos_token_ids=eos_ids,
            bos_token_id=_get(d, "bos_token_id", int, required=False),
            stored_dtype=d.get("dtype") or d.get("torch_dtype"),
        )
        if cfg.vocab_size <= 0 or cfg.hidden_size <= 0 or cfg.intermediate_size <= 0:
            raise ConfigError("vocab_size, hidden_size and the feed-forward width must be positive")
        if cfg.max_position_embeddings < 0:
            raise ConfigError("max_position_embeddings must be positive")
        if not (cfg.rope_theta > 0 and cfg.norm_eps > 0 and math.isfinite(cfg.rope_theta)):
            raise ConfigError("rope_theta and norm_eps must be positive")
        return cfg

    def to_dict(self) -> dict:
        """The config.json content that round-trips through :meth:`from_dict`."""
        d = {
            "architectures": [self.architecture],
            "model_type": "lfm2",
            "vocab_size": self.vocab_size,
            "hidden_size": self.hidden_size,
            "num_hidden_layers": self.num_hidden_layers,
            "layer_types": list(self.layer_types),
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "block_ff_dim": self.block_ff_dim,
            "block_auto_adjust_ff_dim": self.block_auto_adjust_ff_dim,
            "block_multiple_of": self.block_multiple_of,
            "block_ffn_dim_multiplier": self.block_ffn_dim_multiplier,
            "conv_L_cache": self.conv_L_cache,
            "conv_bias": self.conv_bias,
            "tie_embedding": self.tie_embedding,
            "rope_theta": self.rope_theta,
            "rope_pairing": self.rope_pairing,
            "norm_eps": self.norm_eps,
        }
        if self.max_position_embeddings:
            d["max_position_embeddings"] = self.max_position_embeddings
        if self.stored_dtype:
            d["dtype"] = self.stored_dtype
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids) if len(self.eos_token_ids) > 1 else self.eos_token_ids[0]
        if self.bos_token_id is not None:
            d["bos_token_id"] = self.bos_token_id
        return d

    # ------------------------------------------------------------------ the model, as data
    def model_spec(self) -> ModelSpec:
        H = self.hidden_size
        norm = RMSNormSpec(H, self.norm_eps)
        ffn = SwiGLUSpec(H, self.intermediate_size, names=dict(gate="w1", up="w3", down="w2"))
        attn = AttentionSpec(
            hidden=H, n_heads=self.num_attention_heads, n_kv_heads=self.num_key_value_heads,
            head_dim=self.head_dim,
            position=RopeSpec(self.head_dim, self.rope_theta, self.rope_pairing),
            qk_norm=True, qk_norm_eps=self.norm_eps,
            names=dict(q="q_proj", k="k_proj", v="v_proj", o="out_proj",
                       q_norm="q_layernorm", k_norm="k_layernorm"))
        conv = ShortConvSpec(H, self.conv_L_cache, self.conv_bias,
                             names=dict(in_proj="in_proj", conv="conv", out_proj="out_proj"))
        layers = []
        for i, t in enumerate(self.layer_types):
            is_attn = t == "full_attention"
            layers.append(LayerSpec(
                mixer=attn if is_attn else conv, ffn=ffn, mixer_norm=norm, ffn_norm=norm,
                prefix=f"model.layers.{i}.",
                names=dict(mixer="self_attn" if is_attn else "conv", ffn="feed_forward",
                           mixer_norm="operator_norm", ffn_norm="ffn_norm")))
        return ModelSpec(
            architecture=self.architecture, vocab_size=self.vocab_size, hidden=H,
            layers=tuple(layers),
            schedule=tuple(ScheduleEntry(i, i) for i in range(len(layers))),
            final_norm=norm, tie_head=self.tie_embedding,
            max_positions=self.max_position_embeddings,
            embed_name="model.embed_tokens.weight",
            final_norm_name="model.embedding_norm.weight",
            head_name="lm_head.weight",
            eos_token_ids=self.eos_token_ids)
