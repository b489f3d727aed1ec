"""The plain implementation against the reference's OWN engine.

``tests/golden/reference_tiny_a.npz`` holds logits that Leeaandrob/neurogrid's unmodified CUDA
library (``libgpu_engine.so``, driven through its stock entry points by
``tests/golden/make_reference_golden.py`` on a B200) returned for the Tiny A model with the
weights ``write_random_model(TINY_A, 0)`` draws: after a 41-token prompt (cuda_prefill_batch) and
after each of 30 fed tokens (cuda_decode_step_gpu).  The plain implementation must give those
logits.  The reference computes in bfloat16 with float16 hops and rounds its residual stream, so
the agreement is to a few thousandths of the largest logit; that it means something is shown by
the controls: every wrong reading of the reference's formulas (the other rotary pairing, another
order of the B, C, x split, reversed conv taps, per-head norm weights ignored) misses the
golden numbers several times further.
"""
import os

import numpy as np
import pytest
import torch

import plain_lfm2
from tiny_configs import TINY_A

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_tiny_a.npz")


@pytest.fixture(scope="module")
def golden(model_dirs):
    g = np.load(GOLDEN)
    cfg, w = plain_lfm2.load_plain(model_dirs["A"])
    drawn = float(sum(v.abs().sum() for v in w.values()))
    if abs(drawn - float(g["weights_abs_sum"])) > 1e-6 * drawn:
        pytest.skip("this torch draws other random weights than the one the golden file was made with")
    return cfg, w, g["tokens"].tolist(), int(g["prompt_len"]), torch.from_numpy(g["logits"]).double()


def _miss(cfg, w, tokens, prompt_len, ref, rb=True):
    lg = plain_lfm2.forward(cfg, w, tokens, round_bf16=rb)[prompt_len - 1:]
    assert lg.shape == ref.shape
    return float((lg - ref).abs().max() / ref.abs().max())


def test_plain_gives_the_reference_engines_logits(golden):
    cfg, w, tokens, P, ref = golden
    assert cfg["rope_pairing"] == "adjacent" == TINY_A["rope_pairing"]      # the reference engine's pairing
    assert _miss(cfg, w, tokens, P, ref) < 6e-3
    assert _miss(cfg, w, tokens, P, ref, rb=False) < 6e-3


def test_wrong_readings_miss_the_reference(golden):
    cfg, w, tokens, P, ref = golden
    right = _miss(cfg, w, tokens, P, ref)
    H = cfg["hidden_size"]

    def with_in_proj_blocks(order):
        w2 = dict(w)
        for k, v in w.items():
            if k.endswith("conv.in_proj.weight"):
                w2[k] = torch.cat([v[i * H:(i + 1) * H] for i in order])
        return w2

    wrong = {
        "rotary pairing (i, i + hd/2)": _miss(dict(cfg, rope_pairing="half"), w, tokens, P, ref),
        "split read as C|B|x": _miss(cfg, with_in_proj_blocks([1, 0, 2]), tokens, P, ref),
        "split read as B|x|C": _miss(cfg, with_in_proj_blocks([0, 2, 1]), tokens, P, ref),
        "conv taps reversed": _miss(cfg, {k: (v.flip(-1) if k.endswith("conv.conv.weight") else v)
                                          for k, v in w.items()}, tokens, P, ref),
        "per-head norm weights ignored": _miss(cfg, {k: (torch.ones_like(v) if "layernorm" in k else v)
                                                     for k, v in w.items()}, tokens, P, ref),
    }
    for what, miss in wrong.items():
        assert miss > 3 * right, (what, miss, right)
    assert wrong["rotary pairing (i, i + hd/2)"] > 20 * right
    # B and x enter only as their product: reading the split as x|C|B is the same model
    assert abs(_miss(cfg, with_in_proj_blocks([2, 1, 0]), tokens, P, ref) - right) < 1e-9
