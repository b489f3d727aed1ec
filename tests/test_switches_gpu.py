"""The switches of the bfloat16 path (library products, the own product at every size, no
residual-add epilogue, the mma.sync attention for portions): each must give the model's logits."""
import pytest
import torch

import plain_lfm2
import scenarios
from helpers import make_runner, rel_err
from neurogrid_b200.engine import StepEntry
from tiny_configs import PAGE_SIZE

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("switch", ["library_products", "own_product_at_every_size", "no_residual_add_epilogue",
                                    "mma_sync_portion_attention"])
@pytest.mark.parametrize("name", ["B", "C", "D"])
def test_switch_keeps_the_logits(model_dirs, monkeypatch, switch, name):
    from neurogrid_b200.csrc import ops
    if switch == "library_products":
        monkeypatch.setattr(ops, "GEMM_BACKEND", "cublas")
    elif switch == "own_product_at_every_size":
        monkeypatch.setattr(ops, "SM100_MAX_ROWS", 1 << 20)
    elif switch == "no_residual_add_epilogue":
        monkeypatch.setattr(ops, "FUSE_RED", False)
    else:
        monkeypatch.setattr(ops, "ATTN_BACKEND", "mma")
    cfg, w = plain_lfm2.load_plain(model_dirs[name])
    reqs = scenarios.make_requests([5, 90, 33, 130], cfg["vocab_size"], seed=21)
    want = {r: plain_lfm2.forward(cfg, w, t, round_bf16=True) for r, t in reqs.items()}
    ps = PAGE_SIZE[name]
    runner = make_runner(model_dirs[name], dtype=torch.bfloat16, device="cuda", page_size=ps, num_pages=256 // ps,
                         max_requests=4, max_seq_len=256)
    steps = scenarios.mixed(reqs, 256, round_to=ps, seed=3)
    got = []
    for s in steps:
        got.append(runner.step([StepEntry(e["id"], e["tokens"], e["want"]) for e in s["entries"]]).clone())
        for r in s["end"]:
            runner.finish(r)
    runner.check_status()
    out = scenarios.collect(steps, lambda i: got[i])
    for r in reqs:
        assert rel_err(out[r], want[r]) < 2e-2, (switch, r, rel_err(out[r], want[r]))
