"""Shared helpers of the tests: build a runner, replay cuts, compare logits."""
from __future__ import annotations

import torch

from neurogrid_b200.config import load_config
from neurogrid_b200.engine import ModelRunner, StepEntry
from neurogrid_b200.models import build_model, declare_tensors
from neurogrid_b200.weights import load_weights


def make_runner(model_dir, *, dtype=torch.float32, device="cpu", num_pages=64, page_size=16, max_requests=4,
                max_tokens_per_step=512, max_seq_len=None):
    cfg = load_config(model_dir)
    spec = cfg.model_spec()
    weights = load_weights(model_dir, declare_tensors(spec))
    model = build_model(spec, weights, dtype=dtype, device=device)
    return ModelRunner(model, num_pages=num_pages, page_size=page_size, max_requests=max_requests,
                       max_tokens_per_step=max_tokens_per_step, max_seq_len=max_seq_len)


def rel_err(a: torch.Tensor, b: torch.Tensor) -> float:
    """max |a-b| over max |b|: error relative to the scale of the logits."""
    a, b = a.double().cpu(), b.double().cpu()
    return float((a - b).abs().max() / b.abs().max().clamp_min(1e-30))


def run_cuts(runner, req_id, tokens, cuts):
    """Feed ``tokens`` in portions of the sizes in ``cuts`` (all logits wanted); returns [T, V]."""
    out, i = [], 0
    for n in cuts:
        part = tokens[i:i + n]
        out.append(runner.step([StepEntry(req_id, part, list(range(len(part))))]).clone())
        i += n
    assert i == len(tokens)
    runner.finish(req_id)
    return torch.cat(out)
