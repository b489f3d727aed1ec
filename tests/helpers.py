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


def make_ctx(q_lens, ctx_lens, slots, *, dtype, device="cuda", max_rows=4096):
    """A StepContext for parts tested alone: entry e brings q_lens[e] rows after ctx_lens[e]."""
    from neurogrid_b200.parts import StepContext, Workspace
    pos, re, cu = [], [], [0]
    for e, (q, c) in enumerate(zip(q_lens, ctx_lens)):
        pos += list(range(c, c + q))
        re += [e] * q
        cu.append(cu[-1] + q)
    t = lambda x: torch.tensor(x, dtype=torch.int32, device=device)
    return StepContext(n_rows=cu[-1], n_entries=len(q_lens), max_q=max(q_lens), tokens=t([0] * cu[-1]),
                       positions=t(pos), row_entry=t(re), cu_q=t(cu), ctx_before=t(ctx_lens), slots=t(slots),
                       status=torch.zeros(1, dtype=torch.int32, device=device), ws=Workspace(max_rows, device),
                       dtype=dtype, q_lens=list(q_lens), ctx_lens=list(ctx_lens), slot_ids=list(slots))
