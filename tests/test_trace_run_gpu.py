"""bin/trace_run as a user runs it: a subprocess fed JSON lines, writing <step>.f32 files.
One trace per configuration and dtype holds all four ways of cutting the requests."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_lfm2
import scenarios
from helpers import rel_err
from tiny_configs import PAGE_SIZE

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TOL = {"float32": 1e-4, "bfloat16": 2e-2}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,lens", [("A", [1, 7, 33, 100, 60, 45]), ("B", [5, 19, 64, 130, 40, 23, 77]),
                                       ("D", [2, 130, 65, 200, 47, 16])])
def test_replay(model_dirs, tmp_path, name, lens, dtype):
    cfg, w = plain_lfm2.load_plain(model_dirs[name])
    V = cfg["vocab_size"]
    reqs = scenarios.make_requests(lens, V, seed=5)
    cap = 256
    families = {"whole": scenarios.whole(reqs), "tail": scenarios.tail_decode(reqs),
                "portions": scenarios.portions(reqs), "mixed": scenarios.mixed(reqs, cap, round_to=64)}
    steps, spans = [], {}
    for fam, st in families.items():
        # request ids are reused by the next family after their "end": pages and slots come back
        spans[fam] = (len(steps), len(steps) + len(st))
        steps += st
    steps = scenarios.number(steps)
    out = tmp_path / "out"
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", model_dirs[name],
                           "--dtype", dtype, "--out", str(out), "--max-tokens", str(cap),
                           "--page-size", str(PAGE_SIZE[name])],
                          input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True,
                          timeout=900)
    assert proc.returncode == 0, proc.stderr[-3000:]
    assert proc.stdout.split() == [x for s in steps for x in ("done", str(s["step"]))]

    def logits_of(i):
        a = np.fromfile(out / f"{i}.f32", dtype="<f4")
        return torch.from_numpy(a.reshape(-1, V))

    rb = dtype == "bfloat16"
    want = {r: plain_lfm2.forward(cfg, w, t, round_bf16=rb) for r, t in reqs.items()}
    for fam, (lo, hi) in spans.items():
        got = scenarios.collect(steps[lo:hi], lambda i: logits_of(lo + i))
        for r in reqs:
            assert got[r].shape == want[r].shape, (fam, r)
            assert rel_err(got[r], want[r]) < TOL[dtype], (fam, r, rel_err(got[r], want[r]))


def test_nothing_wanted_and_skipped_requests(model_dirs, tmp_path):
    """A step may want nothing (no file is written) and a request may sit out steps."""
    steps = [
        {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": []}], "end": []},
        {"step": 1, "entries": [{"id": "b", "tokens": [9, 9], "want": [1]}], "end": []},
        {"step": 2, "entries": [{"id": "a", "tokens": [4, 8], "want": [1]}, {"id": "b", "tokens": [2], "want": [0]}],
         "end": ["a", "b"]},
    ]
    out = tmp_path / "o"
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", model_dirs["A"],
                           "--dtype", "float32", "--out", str(out), "--max-tokens", "128"],
                          input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True,
                          timeout=900)
    assert proc.returncode == 0, proc.stderr[-3000:]
    assert sorted(os.listdir(out)) == ["1.f32", "2.f32"]
    cfg, w = plain_lfm2.load_plain(model_dirs["A"])
    got = torch.from_numpy(np.fromfile(out / "2.f32", dtype="<f4").reshape(2, -1))
    assert rel_err(got[0], plain_lfm2.forward(cfg, w, [5, 17, 3, 4, 8])[-1]) < 1e-4
    assert rel_err(got[1], plain_lfm2.forward(cfg, w, [9, 9, 2])[-1]) < 1e-4
