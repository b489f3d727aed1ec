"""The engine on the GPU against the plain implementation, in float32 and in bfloat16, under
every way of cutting the work: whole, prefill + 32 decoded tokens, portions of changing size,
and mixed batches with so few pages that they are used again."""
import pytest
import torch

import plain_lfm2
import scenarios
from helpers import make_runner, rel_err
from neurogrid_b200.engine import StepEntry
from tiny_configs import PAGE_SIZE

pytestmark = pytest.mark.gpu

# error relative to the largest logit.  float32: accumulation order only.  bfloat16: compared
# with the plain implementation rounding at the same places; what is left is the order of the
# float32 sums and roundings that flip by one unit (2^-8 relative) and spread through the layers.
TOL = {torch.float32: 1e-4, torch.bfloat16: 2e-2}
LENS = {"A": [1, 7, 33, 100, 60, 45], "B": [5, 19, 64, 130, 40, 23, 77], "C": [3, 50, 97, 64, 31],
        "D": [2, 130, 65, 200, 47, 16]}


def _replay(runner, steps):
    got = []
    for s in steps:
        lg = runner.step([StepEntry(e["id"], e["tokens"], e["want"]) for e in s["entries"]])
        got.append(lg.clone())
        for r in s["end"]:
            runner.finish(r)
    runner.check_status()
    runner.cache.check()
    return scenarios.collect(steps, lambda i: got[i])


@pytest.fixture(scope="module")
def plain(model_dirs):
    out = {}
    for name in LENS:
        cfg, w = plain_lfm2.load_plain(model_dirs[name])
        reqs = scenarios.make_requests(LENS[name], cfg["vocab_size"], seed=7)
        out[name] = (reqs, {rb: {r: plain_lfm2.forward(cfg, w, t, round_bf16=rb) for r, t in reqs.items()}
                            for rb in (False, True)})
    return out


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
@pytest.mark.parametrize("cut", ["whole", "tail_decode", "portions", "mixed"])
def test_cuts_against_plain(model_dirs, plain, name, dtype, cut):
    reqs, want = plain[name]
    ps = PAGE_SIZE[name]
    cap = 256 if cut == "mixed" else 512                     # tokens; mixed: pages must be reused
    runner = make_runner(model_dirs[name], dtype=dtype, device="cuda", page_size=ps, num_pages=cap // ps,
                         max_requests=4, max_seq_len=cap)
    steps = {"whole": scenarios.whole, "tail_decode": scenarios.tail_decode, "portions": scenarios.portions,
             "mixed": lambda r: scenarios.mixed(r, cap, round_to=ps)}[cut](reqs)
    got = _replay(runner, steps)
    ref = want[dtype == torch.bfloat16]
    for r in reqs:
        assert got[r].shape == ref[r].shape
        assert rel_err(got[r], ref[r]) < TOL[dtype], (r, rel_err(got[r], ref[r]))
        if dtype == torch.bfloat16:                          # and not far from the exact model either
            assert rel_err(got[r], want[False][r]) < 2 * TOL[dtype]
    assert runner.cache.pages_free() == [cap // ps]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_first_tokens_and_long_decode(model_dirs, dtype):
    """The first tokens of a sequence one by one (empty cache, conv state before position 0),
    then decoding across many page edges."""
    name = "B"
    cfg, w = plain_lfm2.load_plain(model_dirs[name])
    toks = scenarios.make_requests([200], cfg["vocab_size"], seed=11)["r0"]
    want = plain_lfm2.forward(cfg, w, toks, round_bf16=(dtype == torch.bfloat16))
    runner = make_runner(model_dirs[name], dtype=dtype, device="cuda", page_size=8, num_pages=32, max_seq_len=256)
    got = torch.cat([runner.step([StepEntry("x", [t], [0])]).clone() for t in toks])
    assert rel_err(got[:6], want[:6]) < TOL[dtype]
    assert rel_err(got, want) < TOL[dtype]


def test_float32_cuts_agree_closely(model_dirs):
    """In float32 a token's arithmetic does not depend on the cut: different cuts agree far
    more closely than either agrees with the float64 plain implementation."""
    cfg, _ = plain_lfm2.load_plain(model_dirs["A"])
    reqs = scenarios.make_requests([90], cfg["vocab_size"], seed=3)
    runner = make_runner(model_dirs["A"], dtype=torch.float32, device="cuda", num_pages=32)
    a = _replay(runner, scenarios.whole(reqs))["r0"]
    b = _replay(runner, scenarios.portions(reqs))["r0"]
    c = _replay(runner, scenarios.tail_decode(reqs))["r0"]
    assert rel_err(a, b) < 2e-6 and rel_err(a, c) < 2e-6


def test_refusals_leave_the_cache_whole(model_dirs):
    from neurogrid_b200.cache import OutOfPages
    from neurogrid_b200.engine import StepError
    runner = make_runner(model_dirs["A"], dtype=torch.float32, device="cuda", num_pages=4, page_size=16,
                         max_requests=2, max_seq_len=64)
    runner.step([StepEntry("a", list(range(40)), [39])])
    with pytest.raises(OutOfPages):
        runner.step([StepEntry("b", list(range(30)), [])])          # 3 + 2 pages > 4
    with pytest.raises(StepError):
        runner.step([StepEntry("a", [999], [0])])                    # outside the vocabulary
    with pytest.raises(StepError):
        runner.step([StepEntry("a", [1], [3])])                      # wanted place outside the portion
    runner.cache.check()
    assert runner.cache.length("a") == 40 and not runner.cache.is_live("b")
    runner.finish("a")
    assert runner.cache.pages_free() == [4]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_equal_portions_replay_one_graph(model_dirs, dtype):
    """A prompt cut into portions of one size: the first runs eagerly, the second is captured, the
    rest replay that graph at growing contexts; the logits are the plain implementation's."""
    name = "C"
    cfg, w = plain_lfm2.load_plain(model_dirs[name])
    toks = scenarios.make_requests([240], cfg["vocab_size"], seed=13)["r0"]
    want = plain_lfm2.forward(cfg, w, toks, round_bf16=(dtype == torch.bfloat16))
    runner = make_runner(model_dirs[name], dtype=dtype, device="cuda", page_size=PAGE_SIZE[name], num_pages=16, max_seq_len=512)
    got = [runner.step([StepEntry("x", toks[at:at + 40], list(range(40)))]).clone() for at in range(0, 240, 40)]
    runner.check_status()
    assert runner.stats()["graph_replays"] >= 4
    assert rel_err(torch.cat(got), want) < TOL[dtype]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("name", ["B", "D"])
def test_mixed_steps_replay_graphs_of_padded_shapes(model_dirs, name, dtype):
    """Steps that hold a portion beside single tokens replay a CUDA graph per padded shape (rows,
    entries, context bucket): the same shape met again and again, the real counts changing under it
    (portions of 20 and 17 rows both pad to 32; 3 and then 2 entries pad to 4 and 2); the logits
    are the plain implementation's at every wanted place."""
    cfg, w = plain_lfm2.load_plain(model_dirs[name])
    reqs = scenarios.make_requests([150, 40, 33], cfg["vocab_size"], seed=17)
    want = {r: plain_lfm2.forward(cfg, w, t, round_bf16=(dtype == torch.bfloat16)) for r, t in reqs.items()}
    ps = PAGE_SIZE[name]
    runner = make_runner(model_dirs[name], dtype=dtype, device="cuda", page_size=ps, num_pages=512 // ps, max_requests=4,
                         max_seq_len=256)
    fed = {"r0": 0, "r1": 30, "r2": 25}
    runner.step([StepEntry("r1", reqs["r1"][:30], [])])
    runner.step([StepEntry("r2", reqs["r2"][:25], [])])
    got = {r: {} for r in reqs}
    replays0 = runner.stats()["graph_replays"]
    for i, portion in enumerate([20, 17, 20, 20, 19, 20, 18, 16]):
        entries = [StepEntry("r0", reqs["r0"][fed["r0"]:fed["r0"] + portion], [portion - 1])]
        for r in ("r1", "r2"):
            if fed[r] < len(reqs[r]):
                entries.append(StepEntry(r, reqs[r][fed[r]:fed[r] + 1], [0]))
        lg = runner.step(entries).clone()
        assert lg.shape[0] == len(entries)
        for j, e in enumerate(entries):
            fed[e.req_id] += len(e.tokens)
            got[e.req_id][fed[e.req_id] - 1] = lg[j]
    runner.check_status()
    runner.cache.check()
    assert runner.stats()["graph_replays"] - replays0 >= 5          # the first meeting of a shape runs eagerly
    for r in reqs:
        places = sorted(got[r])
        assert rel_err(torch.stack([got[r][p] for p in places]), want[r][places]) < TOL[dtype], r


def test_long_portions_cut_the_keys_into_runs(model_dirs, monkeypatch):
    """A long prompt in portions, with the threshold from which the portion kernel cuts every
    block's keys into runs lowered so that a tiny model meets it: the later portions take that
    path (eagerly, captured and replayed: a graph per class of context), and the logits at the
    places asked for are the plain implementation's."""
    from neurogrid_b200.csrc import ops
    from neurogrid_b200.parts import attention
    name = "D"
    cfg, w = plain_lfm2.load_plain(model_dirs[name])
    T, portion = 3600, 600
    toks = scenarios.make_requests([T], cfg["vocab_size"], seed=23)["r0"]
    places = list(range(portion - 8, portion))
    want = plain_lfm2.forward(cfg, w, toks, round_bf16=True)
    monkeypatch.setattr(attention, "PREFILL_SPLIT_MIN_CTX", 2048)
    seen = []
    real = ops.attn_prefill_sm100
    monkeypatch.setattr(ops, "attn_prefill_sm100", lambda *a, **k: (seen.append(a[-1] if len(a) > 15 else k.get("n_splits", 1)), real(*a, **k))[1])
    ps = PAGE_SIZE[name]
    runner = make_runner(model_dirs[name], dtype=torch.bfloat16, device="cuda", page_size=ps, num_pages=4096 // ps,
                         max_tokens_per_step=1024, max_seq_len=4096)
    runner.PORTION_LONG_CTX = 2048
    got = [runner.step([StepEntry("x", toks[at:at + portion], places)]).clone() for at in range(0, T, portion)]
    runner.check_status()
    assert max(seen) > 1 and min(seen) == 1, seen                 # short contexts are not cut, long ones are
    assert runner.stats()["graph_replays"] >= 1
    rows = [at + p for at in range(0, T, portion) for p in places]
    assert rel_err(torch.cat(got), want[rows]) < TOL[torch.bfloat16]


@pytest.mark.parametrize("name", ["B", "C", "D"])
def test_decoding_under_graphs_crosses_every_tile_of_the_context(model_dirs, name):
    """Three requests of different lengths decode together, step after step, as replayed CUDA
    graphs, from a context shorter than one key tile of the decode attention to one of several
    (the kernel asks for the tiles of older positions before it waits for the kernel in front of
    it, and for the tile with the step's own key after: at every context length the split
    between the two moves).  Every step's logits are the plain implementation's."""
    cfg, w = plain_lfm2.load_plain(model_dirs[name])
    lens = [330, 290, 205]
    reqs = scenarios.make_requests(lens, cfg["vocab_size"], seed=29)
    want = {r: plain_lfm2.forward(cfg, w, t, round_bf16=True) for r, t in reqs.items()}
    ps = PAGE_SIZE[name]
    runner = make_runner(model_dirs[name], dtype=torch.bfloat16, device="cuda", page_size=ps, num_pages=1024 // ps,
                         max_requests=4, max_seq_len=512)
    start = {"r0": 40, "r1": 100, "r2": 3}
    for r, t in reqs.items():
        runner.step([StepEntry(r, t[:start[r]], [])])
    at = dict(start)
    got = {r: [] for r in reqs}
    while any(at[r] < len(reqs[r]) for r in reqs):
        live = [r for r in reqs if at[r] < len(reqs[r])]
        lg = runner.step([StepEntry(r, reqs[r][at[r]:at[r] + 1], [0]) for r in live]).clone()
        for j, r in enumerate(live):
            got[r].append(lg[j])
            at[r] += 1
    runner.check_status()
    assert runner.stats()["graph_replays"] > 250
    for r in reqs:
        err = [rel_err(g[None], want[r][start[r] + i][None]) for i, g in enumerate(got[r])]
        worst = max(range(len(err)), key=err.__getitem__)
        assert err[worst] < TOL[torch.bfloat16], (r, "position", start[r] + worst, err[worst])


@pytest.mark.parametrize("kinds", [["conv"] * 3, ["full_attention"] * 2, ["conv"]])
def test_models_of_one_layer_kind(tmp_path, kinds):
    """A configuration without attention layers has no pages to manage, one without convolution
    layers no state slots: both load, step (portions, then decoding as replayed graphs) and
    generate, and give the plain implementation's logits."""
    from tiny_configs import TINY_D
    from neurogrid_b200 import Engine
    from neurogrid_b200.weights import write_random_model
    cfg = dict(TINY_D, num_hidden_layers=len(kinds), layer_types=kinds)
    folder = write_random_model(cfg, 3, str(tmp_path / "m"))
    pc, w = plain_lfm2.load_plain(folder)
    reqs = scenarios.make_requests([90, 30], pc["vocab_size"], seed=7)
    for dtype in (torch.float32, torch.bfloat16):
        want = {r: plain_lfm2.forward(pc, w, t, round_bf16=(dtype == torch.bfloat16)) for r, t in reqs.items()}
        runner = make_runner(folder, dtype=dtype, device="cuda", page_size=16, num_pages=16, max_requests=4, max_seq_len=128)
        at = {"r0": 60, "r1": 7}
        got = {r: [runner.step([StepEntry(r, reqs[r][:at[r]], list(range(at[r])))]).clone()] for r in reqs}
        while any(at[r] < len(reqs[r]) for r in reqs):
            live = [r for r in reqs if at[r] < len(reqs[r])]
            lg = runner.step([StepEntry(r, reqs[r][at[r]:at[r] + 1], [0]) for r in live]).clone()
            for j, r in enumerate(live):
                got[r].append(lg[j:j + 1])
                at[r] += 1
        runner.check_status()
        runner.cache.check()
        for r in reqs:
            assert rel_err(torch.cat(got[r]), want[r]) < TOL[dtype], (kinds, dtype, r)
            runner.finish(r)
        assert runner.cache.pages_free() == ([16] if "full_attention" in kinds else [])
    out = Engine(folder, dtype="bfloat16", max_seq_len=128).generate([reqs["r1"][:5]], max_new_tokens=4, temperature=0.0)
    assert len(out) == 1 and len(out[0]) == 4
