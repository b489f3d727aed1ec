"""The bfloat16 fast path at the published layer sizes (width 2048, 32/8 heads of 64, SwiGLU
8192, vocabulary 65536; 3 of the 16 layers to stay small) against the engine's own float32
path, under different cuts and batch sizes.  Tiny configurations cannot reach the code that
only real sizes use: K-split products with many splits, 64-token MMA tiles, context splits of
the decode attention, graphs of padded batches."""
import pytest
import torch

from helpers import rel_err
from neurogrid_b200.engine import ModelRunner, StepEntry
from neurogrid_b200.engine.loading import model_from_seed

pytestmark = pytest.mark.gpu

CFG = dict(
    architectures=["Lfm2ForCausalLM"], model_type="lfm2", vocab_size=65536, hidden_size=2048, num_hidden_layers=3,
    layer_types=["conv", "full_attention", "conv"], num_attention_heads=32, num_key_value_heads=8,
    block_ff_dim=12288, block_auto_adjust_ff_dim=True, block_multiple_of=256, block_ffn_dim_multiplier=1.0,
    conv_L_cache=3, conv_bias=False, tie_embedding=True, rope_theta=1000000.0, norm_eps=1e-5,
    max_position_embeddings=4096,
)


@pytest.fixture(scope="module")
def runners():
    out = {}
    for dtype in (torch.float32, torch.bfloat16):
        _, model = model_from_seed(CFG, 0, dtype=dtype, device="cuda")
        out[dtype] = ModelRunner(model, num_pages=40 * 1024 // 16, page_size=16, max_requests=40, max_seq_len=1024,
                                 max_tokens_per_step=1024)
    return out


def _tokens(n, seed):
    return torch.randint(0, 65536, (n,), generator=torch.Generator().manual_seed(seed)).tolist()


def _run(runner, reqs, cuts_of, decode_tail):
    """Prefill each request in the portions ``cuts_of(len)``, then decode the last
    ``decode_tail`` tokens of all requests together, one batched step per token."""
    rows = {r: [] for r in reqs}
    for r, toks in reqs.items():
        head = len(toks) - decode_tail
        at = 0
        for n in cuts_of(head):
            lg = runner.step([StepEntry(r, toks[at:at + n], [n - 1])]).clone()
            at += n
        rows[r].append(lg)                                   # the last prompt position only: cuts differ before it
    for i in range(decode_tail):
        lg = runner.step([StepEntry(r, [t[len(t) - decode_tail + i]], [0]) for r, t in reqs.items()]).clone()
        for j, r in enumerate(reqs):
            rows[r].append(lg[j:j + 1])
    for r in reqs:
        runner.finish(r)
    runner.check_status()
    return {r: torch.cat(v) for r, v in rows.items()}


@pytest.mark.parametrize("n_req", [1, 8, 33])
def test_bf16_follows_float32_at_real_sizes(runners, n_req):
    reqs = {f"r{i}": _tokens(300 + 37 * (i % 5), 10 + i) for i in range(n_req)}
    whole = lambda n: [n]
    cut = lambda n: [100, 3, n - 103]
    want = _run(runners[torch.float32], reqs, whole, 12)
    for cuts in (whole, cut):
        got = _run(runners[torch.bfloat16], reqs, cuts, 12)
        for r in reqs:
            assert got[r].shape == want[r].shape
            assert torch.isfinite(got[r]).all()
            assert rel_err(got[r], want[r]) < 3e-2, (r, rel_err(got[r], want[r]))
            # the token bfloat16 ranks first is one that float32 ranks (almost) first: its float32
            # logit lies within the rounding of the float32 maximum.  (With random weights the two
            # best logits often lie closer than that, so the winner itself may differ.)
            chosen = want[r].gather(1, torch.argmax(got[r], -1, keepdim=True)).squeeze(1)
            gap = want[r].max(-1).values - chosen
            assert float(gap.max()) <= 2 * 3e-2 * float(want[r].abs().max())
    assert runners[torch.bfloat16].stats()["graph_replays"] > 0
    assert runners[torch.bfloat16].cache.pages_free() == [40 * 1024 // 16]


def test_float32_cuts_agree_at_real_sizes(runners):
    reqs = {"a": _tokens(260, 1), "b": _tokens(130, 2)}
    a = _run(runners[torch.float32], reqs, lambda n: [n], 4)
    b = _run(runners[torch.float32], reqs, lambda n: [64, 1, 2, n - 67], 4)
    for r in reqs:
        assert rel_err(a[r], b[r]) < 5e-6
