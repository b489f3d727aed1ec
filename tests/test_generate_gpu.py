"""Generation through the Python entry point: greedy tokens equal the plain implementation's,
sampled tokens equal a host mirror of the sampler and do not depend on the batch, a pool that
forces preemption does not change the output; the command line runs."""
import json
import os
import subprocess
import sys

import pytest
import torch

import plain_lfm2
from neurogrid_b200.sampling import SamplingParams, uniform_for
from tiny_configs import PAGE_SIZE

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _prompts(lens, vocab, seed):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, vocab, (n,), generator=g).tolist() for n in lens]


def _engine(model_dir, name, **kw):
    from neurogrid_b200 import Engine
    kw.setdefault("page_size", PAGE_SIZE[name])
    kw.setdefault("max_seq_len", 256)
    return Engine(model_dir, **kw)


def _check_greedy(cfg, w, prompt, out, rb, gap_tol):
    """Teacher-forced: wherever the engine's token is not the plain argmax, the plain logits
    of the two must be within ``gap_tol`` of the largest logit (a near tie), never more."""
    lg = plain_lfm2.forward(cfg, w, prompt + out, round_bf16=rb)
    flips = 0
    for i, tok in enumerate(out):
        row = lg[len(prompt) - 1 + i]
        best = int(torch.argmax(row))
        if tok != best:
            flips += 1
            assert float(row[best] - row[tok]) <= gap_tol * float(row.abs().max()), (i, tok, best)
    return flips


@pytest.mark.parametrize("dtype,gap", [("float32", 1e-4), ("bfloat16", 2e-2)])
def test_greedy_generation_equals_plain(model_dirs, dtype, gap):
    cfg, w = plain_lfm2.load_plain(model_dirs["A"])
    prompts = _prompts([1, 7, 33], cfg["vocab_size"], 0)
    eng = _engine(model_dirs["A"], "A", dtype=dtype)
    outs = eng.generate(prompts, max_new_tokens=16, temperature=0.0)
    assert [len(o) for o in outs] == [16, 16, 16] and eng.last_finish_reasons == ["length"] * 3
    flips = sum(_check_greedy(cfg, w, p, o, dtype == "bfloat16", gap) for p, o in zip(prompts, outs))
    if dtype == "float32":
        assert flips == 0
        assert outs == [plain_lfm2.generate_greedy(cfg, w, p, 16) for p in prompts]
    assert eng.stats()["pages_free"] == [eng.runner.cache.pools[0].num_pages]


def test_sampling_matches_host_mirror_and_ignores_the_batch(model_dirs):
    cfg, w = plain_lfm2.load_plain(model_dirs["B"])
    prompts = _prompts([5, 19, 64, 130], cfg["vocab_size"], 1)
    kw = dict(dtype="float32", max_tokens_per_step=48, chunk_size=16, max_requests=4)
    together = _engine(model_dirs["B"], "B", **kw).generate(prompts, max_new_tokens=12, temperature=0.8,
                                                          top_p=0.9, seed=7)
    for i, (p, out) in enumerate(zip(prompts, together)):
        lg = plain_lfm2.forward(cfg, w, p + out)
        for j, tok in enumerate(out):
            probs = plain_lfm2.sample_probs(lg[len(p) - 1 + j], 0.8, 0.9)
            u = uniform_for(7, i, j)
            want = plain_lfm2.sample_from(probs, u)
            if tok != want:                                  # only where u sits on a boundary of the CDF
                c = torch.cumsum(probs, 0)
                edge = min(abs(float(c[tok]) - u), abs(float(c[tok - 1]) - u) if tok else 1.0)
                assert edge < 1e-4, (i, j, tok, want, edge)
    # each request alone, with its own stream number: the same tokens
    eng = _engine(model_dirs["B"], "B", **kw)
    for i, p in enumerate(prompts):
        rid = eng.add_request(p, SamplingParams(temperature=0.8, top_p=0.9, max_new_tokens=12, seed=7), rng_key=i)
        eng.run()
        assert eng._requests[rid].output == together[i]


@pytest.mark.parametrize("name", ["B", "D"])
def test_bfloat16_sampling_matches_host_mirror_on_the_engine_logits(model_dirs, name):
    """Temperature and top-p sampling through the engine in bfloat16.  The draw is checked
    against the host mirror applied to the engine's own bfloat16 logits (the same sequence fed
    again through the step function, every row wanted): a token may differ from the mirror's
    only where the uniform number sits on a boundary of the distribution.  The logits themselves
    are compared with the plain implementation elsewhere."""
    from neurogrid_b200.engine import StepEntry
    cfg, w = plain_lfm2.load_plain(model_dirs[name])
    prompts = _prompts([5, 19, 64, 130], cfg["vocab_size"], 3)
    kw = dict(dtype="bfloat16", max_tokens_per_step=48, chunk_size=16, max_requests=4)
    eng = _engine(model_dirs[name], name, **kw)
    outs = eng.generate(prompts, max_new_tokens=12, temperature=0.7, top_p=0.95, seed=11)
    assert [len(o) for o in outs] == [12] * 4
    off_mirror = 0
    for i, (p, out) in enumerate(zip(prompts, outs)):
        seq = p + out
        lg = torch.cat([eng.runner.step([StepEntry(("again", i), seq[at:at + 40], list(range(len(seq[at:at + 40]))))])
                        .double().cpu() for at in range(0, len(seq), 40)])
        eng.runner.finish(("again", i))
        ref = plain_lfm2.forward(cfg, w, seq, round_bf16=True)
        assert float((lg - ref).abs().max() / ref.abs().max()) < 2e-2
        for j, tok in enumerate(out):
            probs = plain_lfm2.sample_probs(lg[len(p) - 1 + j], 0.7, 0.95)
            u = uniform_for(11, i, j)
            want = plain_lfm2.sample_from(probs, u)
            if tok != want:
                # the sampled step saw the same position in another batch: its logits may differ
                # from this replay's in the last bits of bfloat16 roundings, which moves the CDF a little
                off_mirror += 1
                c = torch.cumsum(probs, 0)
                edge = min(abs(float(c[tok]) - u), abs(float(c[tok - 1]) - u) if tok else 1.0)
                assert edge < 5e-3, (i, j, tok, want, edge)
    assert off_mirror <= 4                                  # of 48 draws: boundaries are rare


def test_small_pool_preempts_and_output_is_unchanged(model_dirs):
    cfg, _ = plain_lfm2.load_plain(model_dirs["B"])
    prompts = _prompts([30, 17, 44, 9, 25, 38], cfg["vocab_size"], 2)
    big = _engine(model_dirs["B"], "B", dtype="float32", max_requests=4)
    small = _engine(model_dirs["B"], "B", dtype="float32", max_requests=4, num_pages=10,     # 80 tokens
                    max_tokens_per_step=40, chunk_size=16)
    a = big.generate(prompts, max_new_tokens=20)
    b = small.generate(prompts, max_new_tokens=20)
    assert a == b
    assert small.stats()["preemptions"] > 0 and big.stats()["preemptions"] == 0
    assert small.stats()["pages_free"] == [10]


def test_command_line(model_dirs, tmp_path):
    cmd = [sys.executable, os.path.join(ROOT, "bin", "neurogrid"), "-model", model_dirs["A"], "-gpu", "0",
           "-max-seq-len", "128", "-dtype", "fp32", "-prompt-tokens", "5,17,3", "-prompt-len", "9",
           "-max-new-tokens", "6", "-log-level", "error"]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [json.loads(l) for l in r.stdout.strip().splitlines()]
    assert len(lines) == 2 and all(len(l["tokens"]) == 6 and l["finish_reason"] == "length" for l in lines)
    cfg, w = plain_lfm2.load_plain(model_dirs["A"])
    assert lines[0]["tokens"] == plain_lfm2.generate_greedy(cfg, w, [5, 17, 3], 6)
    # random-weights mode writes a model folder that loads
    cfgp = tmp_path / "c.json"
    cfgp.write_text(json.dumps(cfg))
    out = tmp_path / "model"
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "neurogrid"), "-config", str(cfgp),
                        "-random-weights", "3", "-write-model", str(out)], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and sorted(os.listdir(out)) == ["config.json", "model.safetensors"]


def test_running_a_step_ahead_changes_nothing(model_dirs):
    """The engine launches the next decode step before it has read the tokens of the one in
    flight.  Outputs equal those of an engine that waits for every token, also when requests
    stop on a token that is found one step late, finish at different lengths and leave the
    others to go on."""
    cfg, _ = plain_lfm2.load_plain(model_dirs["B"])
    prompts = _prompts([5, 19, 33, 8], cfg["vocab_size"], 3)
    kw = dict(dtype="float32", max_requests=4)
    base = _engine(model_dirs["B"], "B", pipeline=False, **kw).generate(prompts, max_new_tokens=24, temperature=0.9, seed=5)
    # stop tokens taken from the middle of two of the outputs: those requests end early
    stops = (base[0][7], base[2][15])
    for pipeline in (False, True):
        eng = _engine(model_dirs["B"], "B", pipeline=pipeline, **kw)
        outs = eng.generate(prompts, max_new_tokens=24, temperature=0.9, seed=5, stop_token_ids=stops)
        for o, b in zip(outs, base):
            cut = next((i for i, t in enumerate(b) if t in stops), len(b) - 1)
            assert o == b[:cut + 1]
        assert eng.last_finish_reasons[0] == "stop" and eng.last_finish_reasons[2] == "stop"
        assert eng.stats()["pages_free"] == [eng.runner.cache.pools[0].num_pages] and eng.stats()["slots_free"] == 4
    # uneven lengths: each request stops at its own limit while the others run on
    eng = _engine(model_dirs["B"], "B", **kw)
    from neurogrid_b200.sampling import SamplingParams
    ids = [eng.add_request(p, SamplingParams(temperature=0.9, seed=5, max_new_tokens=n), rng_key=i)
           for i, (p, n) in enumerate(zip(prompts, (3, 24, 1, 10)))]
    eng.run()
    for i, n in zip(ids, (3, 24, 1, 10)):
        assert eng._requests[i].output == base[i][:n] and eng._requests[i].finish_reason == "length"


def test_greedy_decode_feeds_and_samples_inside_the_graph(model_dirs):
    """While requests only decode greedily, the step's graph takes the fed tokens from the
    sampler's buffer and leaves its argmax there: nothing but the graph and two copies per step."""
    eng = _engine(model_dirs["B"], "B", dtype="bfloat16", max_requests=4)
    cfg, w = plain_lfm2.load_plain(model_dirs["B"])
    prompts = _prompts([9, 30, 4], cfg["vocab_size"], 5)
    for p in prompts:
        eng.add_request(p, SamplingParams(temperature=0.0, max_new_tokens=24))
    seen = []
    while eng.scheduler.has_work() or eng._inflight is not None:
        eng.step()
        seen.append((eng.runner.fed_in_graph, eng.runner.sampled_in_graph))
    assert (True, True) in seen
    assert eng.stats()["graph_replays"] > 10
    eng.runner.check_status()
