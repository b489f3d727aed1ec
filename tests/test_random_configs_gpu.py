"""Configurations drawn at random (head sizes 16..256, any number of heads and groups, widths
and vocabularies that are no power of two, every conv width, every page size), each replayed in
portions and in mixed batches with reused pages, against the plain implementation."""
import random

import pytest
import torch

import plain_lfm2
import scenarios
from helpers import make_runner, rel_err
from neurogrid_b200.engine import StepEntry
from neurogrid_b200.weights import write_random_model

pytestmark = pytest.mark.gpu
TOL = {torch.float32: 1e-4, torch.bfloat16: 2e-2}


def draw_config(rng: random.Random) -> dict:
    n_kv = rng.choice([1, 2, 3, 4])
    n_layers = rng.randint(2, 5)
    kinds = [rng.choice(["conv", "full_attention"]) for _ in range(n_layers)]
    if "full_attention" not in kinds:
        kinds[rng.randrange(n_layers)] = "full_attention"
    d = dict(architectures=["Lfm2ForCausalLM"], model_type="lfm2", vocab_size=rng.randint(90, 1100),
             hidden_size=rng.choice([40, 64, 72, 88, 100, 104, 136, 200, 264]), num_hidden_layers=n_layers,
             layer_types=kinds, num_attention_heads=n_kv * rng.choice([1, 2, 3, 4, 5]), num_key_value_heads=n_kv,
             head_dim=16 * rng.randint(1, 16), block_ff_dim=rng.choice([96, 200, 264, 328, 500]),
             block_auto_adjust_ff_dim=rng.random() < 0.5, block_multiple_of=rng.choice([8, 24, 32, 64]),
             block_ffn_dim_multiplier=rng.choice([1.0, 1.3, 0.8]), conv_L_cache=rng.choice([2, 3, 4, 5]),
             conv_bias=rng.random() < 0.5, tie_embedding=rng.random() < 0.5,
             rope_theta=rng.choice([1e4, 5e4, 1e6]), norm_eps=rng.choice([1e-5, 1e-6, 3e-6]))
    d["rope_pairing"] = "half" if rng.random() < 0.5 else "adjacent"
    return d


def _replay(runner, steps):
    got = []
    for s in steps:
        got.append(runner.step([StepEntry(e["id"], e["tokens"], e["want"]) for e in s["entries"]]).clone())
        for r in s["end"]:
            runner.finish(r)
    runner.check_status()
    runner.cache.check()
    return scenarios.collect(steps, lambda i: got[i])


@pytest.mark.parametrize("seed", [3, 11, 42, 205, 1009])
def test_random_configuration(tmp_path, seed):
    rng = random.Random(seed)
    cfg = draw_config(rng)
    ps = rng.choice([8, 16, 32, 64])
    lens = [rng.randint(1, 200) for _ in range(rng.randint(3, 5))] + [rng.choice([64, 65, 128, 129, 257])]
    write_random_model(cfg, seed, str(tmp_path))
    pc, w = plain_lfm2.load_plain(str(tmp_path))
    reqs = scenarios.make_requests(lens, pc["vocab_size"], seed=seed)
    cap = max(256, 2 * 64 * -(-max(lens) // 64))
    for dtype in (torch.float32, torch.bfloat16):
        want = {r: plain_lfm2.forward(pc, w, t, round_bf16=(dtype == torch.bfloat16)) for r, t in reqs.items()}
        for steps in (scenarios.portions(reqs, seed), scenarios.mixed(reqs, cap, round_to=ps, seed=seed)):
            runner = make_runner(str(tmp_path), dtype=dtype, device="cuda", page_size=ps, num_pages=cap // ps,
                                 max_requests=4, max_seq_len=cap, max_tokens_per_step=cap)
            got = _replay(runner, steps)
            for r in reqs:
                assert rel_err(got[r], want[r]) < TOL[dtype], (cfg, ps, lens, r)
            assert runner.cache.pages_free() == [cap // ps]
