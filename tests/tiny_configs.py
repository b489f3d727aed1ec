"""Tiny LFM2 configurations for the tests: A and B differ in every size and option."""

TINY_A = dict(
    architectures=["Lfm2ForCausalLM"], model_type="lfm2",
    vocab_size=256, hidden_size=64, num_hidden_layers=4,
    layer_types=["conv", "conv", "full_attention", "conv"],
    num_attention_heads=4, num_key_value_heads=2,          # head_dim = 64/4 = 16 (computed)
    block_ff_dim=288, block_auto_adjust_ff_dim=True, block_multiple_of=64, block_ffn_dim_multiplier=1.0,
    conv_L_cache=3, conv_bias=False, tie_embedding=True, rope_theta=1000000.0, norm_eps=1e-5,
    rope_pairing="adjacent",                               # the reference engine's pairing stays under test
    max_position_embeddings=256,
)

TINY_B = dict(
    architectures=["Lfm2ForCausalLM"], model_type="lfm2",
    vocab_size=512, hidden_size=96, num_hidden_layers=6,
    layer_types=["full_attention", "conv", "conv", "full_attention", "conv", "full_attention"],
    num_attention_heads=3, num_key_value_heads=1, head_dim=32,
    block_ff_dim=256, block_auto_adjust_ff_dim=False,
    conv_L_cache=4, conv_bias=True, tie_embedding=False, rope_theta=10000.0, norm_eps=1e-6,
    rope_pairing="half",                                   # the checkpoint format's pairing (the default)
    max_position_embeddings=512,
)

# A third shape for generality: vocabulary and widths that are no power of two, head_dim 48
# with the width not equal to heads * head_dim, "half" rotary pairing, conv width 2.
TINY_C = dict(
    architectures=["Lfm2ForCausalLM"], model_type="lfm2",
    vocab_size=301, hidden_size=80, num_hidden_layers=3,
    layer_types=["conv", "full_attention", "full_attention"],
    num_attention_heads=6, num_key_value_heads=3, head_dim=48,
    block_ff_dim=200, block_auto_adjust_ff_dim=True, block_multiple_of=24, block_ffn_dim_multiplier=1.3,
    conv_L_cache=2, conv_bias=True, tie_embedding=True, rope_theta=50000.0, norm_eps=3e-6,
    rope_pairing="half", max_position_embeddings=384,
)

# The published head size (64) with 4 query heads per KV head, page size 16 and conv width 3:
# the shapes of the tcgen05 attention kernel, the split decode kernel and the one-pair-per-lane
# rotary path, inside a model small enough for the plain implementation.  No rope_pairing key:
# the default is under test here.
TINY_D = dict(
    architectures=["Lfm2ForCausalLM"], model_type="lfm2",
    vocab_size=384, hidden_size=128, num_hidden_layers=5,
    layer_types=["conv", "full_attention", "conv", "full_attention", "full_attention"],
    num_attention_heads=8, num_key_value_heads=2, head_dim=64,
    block_ff_dim=384, block_auto_adjust_ff_dim=True, block_multiple_of=32, block_ffn_dim_multiplier=1.0,
    conv_L_cache=3, conv_bias=False, tie_embedding=True, rope_theta=1000000.0, norm_eps=1e-5,
    max_position_embeddings=1024,
)

TINY = {"A": (TINY_A, 0), "B": (TINY_B, 1), "C": (TINY_C, 2), "D": (TINY_D, 3)}
PAGE_SIZE = {"A": 16, "B": 8, "C": 32, "D": 16}
