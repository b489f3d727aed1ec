"""Host side of the step function on the CPU, with the kernels replaced by their plain
statements (tests/kernel_refs.py): packing of ragged batches, the cache and page reuse."""
import random

import pytest
import torch

import kernel_refs
import plain_lfm2
from helpers import make_runner, rel_err, run_cuts
from neurogrid_b200.engine import StepEntry
from tiny_configs import PAGE_SIZE, TINY


@pytest.fixture(autouse=True)
def _plain_kernels(monkeypatch):
    kernel_refs.install(monkeypatch)


def _tokens(n, vocab, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_whole_prompt_matches_plain(model_dirs, name):
    cfg, w = plain_lfm2.load_plain(model_dirs[name])
    runner = make_runner(model_dirs[name], page_size=PAGE_SIZE[name])
    for T in (1, 7, 33):
        toks = _tokens(T, cfg["vocab_size"], T)
        got = run_cuts(runner, "r", toks, [T])
        assert rel_err(got, plain_lfm2.forward(cfg, w, toks)) < 2e-5
    runner.cache.check()


@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_cuts_match_whole(model_dirs, name):
    cfg, w = plain_lfm2.load_plain(model_dirs[name])
    runner = make_runner(model_dirs[name], page_size=PAGE_SIZE[name])
    toks = _tokens(70, cfg["vocab_size"], 5)
    want = plain_lfm2.forward(cfg, w, toks)
    for cuts in ([38] + [1] * 32, [2, 3, 17, 1, 1, 30, 2, 14], [1] * 70):
        assert rel_err(run_cuts(runner, "r", toks, cuts), want) < 2e-5


@pytest.mark.parametrize("name", ["A", "B"])
def test_mixed_batches_with_page_reuse(model_dirs, name):
    cfg, w = plain_lfm2.load_plain(model_dirs[name])
    ps = PAGE_SIZE[name]
    lens = [5, 19, 64, 130, 40, 23]
    # room for about 256 tokens: later requests get pages that earlier ones gave back
    runner = make_runner(model_dirs[name], page_size=ps, num_pages=256 // ps, max_requests=4)
    rng = random.Random(0)
    reqs = {i: _tokens(n, cfg["vocab_size"], 100 + i) for i, n in enumerate(lens)}
    want = {i: plain_lfm2.forward(cfg, w, t) for i, t in reqs.items()}
    got = {i: [] for i in reqs}
    fed = {i: 0 for i in reqs}
    waiting, live = list(reqs), []
    while waiting or live:
        while waiting and len(live) < 4:
            nxt = waiting[0]
            held = sum(-(-max(fed[r], 1) // ps) * ps for r in live)
            if held + -(-len(reqs[nxt]) // ps) * ps + 64 > 256 and live:
                break
            live.append(waiting.pop(0))
        entries, done = [], []
        for r in live:
            left = len(reqs[r]) - fed[r]
            n = min(left, rng.choice([1, 1, 2, 3, 16]))
            part = reqs[r][fed[r]:fed[r] + n]
            entries.append(StepEntry(r, part, list(range(n))))
        try:
            logits = runner.step(entries)
        except Exception:
            runner.cache.check()
            raise
        o = 0
        for e in entries:
            n = len(e.tokens)
            got[e.req_id].append(logits[o:o + n].clone())
            o += n
            fed[e.req_id] += n
            if fed[e.req_id] == len(reqs[e.req_id]):
                done.append(e.req_id)
        for r in done:
            runner.finish(r)
            live.remove(r)
        runner.cache.check()
    for i in reqs:
        assert rel_err(torch.cat(got[i]), want[i]) < 2e-5, i
    assert runner.cache.pages_free() == [256 // ps]


@pytest.mark.parametrize("name", ["A", "C"])
def test_scenarios_replay_on_cpu(model_dirs, name):
    """The trace scenarios the GPU tests use, replayed here with the plain kernels."""
    import scenarios
    cfg, w = plain_lfm2.load_plain(model_dirs[name])
    ps = PAGE_SIZE[name]
    reqs = scenarios.make_requests([1, 7, 33, 100, 60, 45], cfg["vocab_size"], seed=7)
    want = {r: plain_lfm2.forward(cfg, w, t) for r, t in reqs.items()}
    for steps in (scenarios.tail_decode(reqs), scenarios.portions(reqs), scenarios.mixed(reqs, 256, round_to=ps)):
        runner = make_runner(model_dirs[name], page_size=ps, num_pages=256 // ps, max_seq_len=256)
        got = []
        for s in steps:
            got.append(runner.step([StepEntry(e["id"], e["tokens"], e["want"]) for e in s["entries"]]).clone())
            for r in s["end"]:
                runner.finish(r)
            runner.cache.check()
        res = scenarios.collect(steps, lambda i: got[i])
        for r in reqs:
            assert rel_err(res[r], want[r]) < 2e-5
        assert runner.cache.pages_free() == [256 // ps]


def test_model_without_a_position_limit(tmp_path):
    """config.json may give no max_position_embeddings: then the pool alone bounds a request."""
    from neurogrid_b200.weights import write_random_model
    from tiny_configs import TINY_B
    d = {k: v for k, v in TINY_B.items() if k != "max_position_embeddings"}
    write_random_model(d, 4, str(tmp_path))
    cfg, w = plain_lfm2.load_plain(str(tmp_path))
    runner = make_runner(str(tmp_path), page_size=8, num_pages=12)
    assert runner.max_seq_len == 96
    toks = _tokens(50, cfg["vocab_size"], 9)
    assert rel_err(run_cuts(runner, "r", toks, [20, 30]), plain_lfm2.forward(cfg, w, toks)) < 2e-5
