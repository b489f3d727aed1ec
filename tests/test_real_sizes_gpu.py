"""Both paths at the published layer sizes (width 2048, 32/8 heads of 64, SwiGLU 8192,
vocabulary 65536; 3 of the 16 layers to stay small).  Tiny configurations cannot reach the code
that only real sizes use: K-split products with many splits, 64-token MMA tiles, context splits
of the decode attention, graphs of padded batches, the library products of long portions.
The float32 path is compared with the plain implementation (float64 on the CPU); the bfloat16
path with the plain implementation rounding at the same places, and with the float32 path under
more cuts and batch sizes than the CPU could follow."""
import pytest
import torch

import plain_lfm2
from helpers import rel_err
from neurogrid_b200.config import config_from_dict
from neurogrid_b200.engine import ModelRunner, StepEntry
from neurogrid_b200.models import build_model, declare_tensors
from neurogrid_b200.weights import draw

pytestmark = pytest.mark.gpu

CFG = dict(
    architectures=["Lfm2ForCausalLM"], model_type="lfm2", vocab_size=65536, hidden_size=2048, num_hidden_layers=3,
    layer_types=["conv", "full_attention", "conv"], num_attention_heads=32, num_key_value_heads=8,
    block_ff_dim=12288, block_auto_adjust_ff_dim=True, block_multiple_of=256, block_ffn_dim_multiplier=1.0,
    conv_L_cache=3, conv_bias=False, tie_embedding=True, rope_theta=1000000.0, norm_eps=1e-5,
    max_position_embeddings=4096,
)


@pytest.fixture(scope="module")
def weights():
    spec = config_from_dict(CFG).model_spec()
    return spec, draw(declare_tensors(spec), 0, dtype=torch.bfloat16, device="cuda")


@pytest.fixture(scope="module")
def runners(weights):
    spec, w = weights
    out = {}
    for dtype in (torch.float32, torch.bfloat16):
        model = build_model(spec, w, dtype=dtype, device="cuda")
        out[dtype] = ModelRunner(model, num_pages=40 * 1024 // 16, page_size=16, max_requests=40, max_seq_len=1024,
                                 max_tokens_per_step=1024)
    return out


@pytest.fixture(scope="module")
def plain_weights(weights):
    return {k: v.cpu().to(torch.float64) for k, v in weights[1].items()}


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


def _mixed_steps(reqs, long_id, portions):
    """The short requests whole (one step each, nothing wanted but the last place), then steps
    that hold a portion of ``long_id`` beside one decode token of every short request."""
    steps, fed = [], {}
    for r, t in reqs.items():
        if r != long_id:
            fed[r] = len(t) - len(portions)
            steps.append([(r, t[:fed[r]], [fed[r] - 1])])
    at = 0
    for n in portions:
        step = [(long_id, reqs[long_id][at:at + n], [0, n - 1])]
        at += n
        for r, t in reqs.items():
            if r != long_id:
                step.append((r, t[fed[r]:fed[r] + 1], [0]))
                fed[r] += 1
        steps.append(step)
    assert at == len(reqs[long_id])
    return steps


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_mixed_steps_at_real_sizes_against_plain(runners, plain_weights, dtype):
    """Steps that hold a prompt portion beside decode tokens, at head size 64 and real widths,
    against the plain implementation: a 100-token portion beside 8 decode tokens (more than 64
    rows: the library's products, the standalone gate kernel, both attention kernels in one step)
    and a 20-token portion beside them (at most 64 rows: the tensor-core products of this package
    on a ragged step, the portion attention skipping the single tokens), then short portions."""
    runner = runners[dtype]
    reqs = {f"d{i}": _tokens(70 + 23 * i, 40 + i) for i in range(8)}
    reqs["long"] = _tokens(100 + 20 + 3 + 41 + 2, 77)
    steps = _mixed_steps(reqs, "long", [100, 20, 3, 41, 2])
    got = {r: [] for r in reqs}
    places = {r: [] for r in reqs}
    seen = {r: 0 for r in reqs}
    for step in steps:
        lg = runner.step([StepEntry(r, toks, want) for r, toks, want in step]).clone()
        o = 0
        for r, toks, want in step:
            got[r].append(lg[o:o + len(want)])
            places[r] += [seen[r] + w for w in want]
            seen[r] += len(toks)
            o += len(want)
    for r in reqs:
        runner.finish(r)
    runner.check_status()
    rb = dtype == torch.bfloat16
    tol = 2e-2 if rb else 1e-4
    for r, t in reqs.items():
        want = plain_lfm2.forward(CFG, plain_weights, t, round_bf16=rb, rows=places[r])
        assert rel_err(torch.cat(got[r]), want) < tol, (r, rel_err(torch.cat(got[r]), want))
    assert runner.cache.pages_free() == [40 * 1024 // 16]


def test_float32_follows_plain_at_real_sizes(runners, plain_weights):
    """The float32 path against the float64 plain implementation at the published widths: one
    request whole, then its last tokens one by one."""
    toks = _tokens(290, 5)
    got = _run(runners[torch.float32], {"a": toks}, lambda n: [n], 6)["a"]
    want = plain_lfm2.forward(CFG, plain_weights, toks, rows=list(range(290 - 7, 290)))
    assert rel_err(got, want) < 1e-4, rel_err(got, want)
