"""The Python entry point: ``Engine(...).generate(token lists) -> token lists``.

An ``Engine`` owns one model on one GPU, its cache, the step function, the scheduler and the
sampler.  ``generate`` is the blocking call; ``add_request`` / ``step`` / ``run`` expose the
loop.  Option names follow the reference's command line where it has them (``-model``,
``-gpu``, ``-max-seq-len``: cmd/neurogrid/main.go:884-898); the reference has no Python API
(its generation driver is pkg/inference/engine.go:387 behind an HTTP server).
"""
from __future__ import annotations

import time
from typing import Dict, Hashable, List, Mapping, Optional, Sequence

import torch

from ..sampling import DEFAULT_SEED, Sampler, SamplingParams, uniform_for
from .loading import model_from_dir, model_from_seed, parse_dtype, require_cuda
from .runner import ModelRunner, StepEntry
from .scheduler import FINISHED, Request, Scheduler, StepPlan


class Engine:
    def __init__(self, model: Optional[str] = None, *, config: Optional[Mapping] = None,
                 random_weights: Optional[int] = None, dtype="bfloat16", gpu: int = 0,
                 max_seq_len: int = 4096, page_size: int = 16, num_pages: Optional[int] = None,
                 max_requests: int = 8, max_tokens_per_step: int = 2048, chunk_size: Optional[int] = None,
                 cache_memory_fraction: float = 0.25, pipeline: bool = True):
        """``model``: folder with config.json and safetensors.  Without it, ``config`` (the
        config.json mapping) and ``random_weights`` (a seed) build a model with random weights
        on the device.  ``max_seq_len`` caps the model's max_position_embeddings (as the
        reference's flag does).  ``num_pages`` defaults to room for ``max_requests`` full
        contexts, limited to ``cache_memory_fraction`` of the free device memory (the reference
        sizes its pool to 25% of free VRAM, pkg/inference/engine_gpu.go:224-243)."""
        self.device = require_cuda(f"cuda:{gpu}")
        self.dtype = parse_dtype(dtype)
        if model is not None:
            self.config, self.model = model_from_dir(model, dtype=self.dtype, device=self.device)
        elif config is not None and random_weights is not None:
            self.config, self.model = model_from_seed(config, random_weights, dtype=self.dtype, device=self.device)
        else:
            raise ValueError("give a model folder, or a config and a random_weights seed")
        spec = self.model.spec
        self.max_seq_len = min(int(max_seq_len), spec.max_positions) if spec.max_positions else int(max_seq_len)
        if num_pages is None:
            num_pages = max_requests * -(-self.max_seq_len // page_size)
            probe = ModelRunner.bytes_per_page(self.model, page_size)
            if probe:
                # the eager workspace and the one the portion graphs keep are allocated at the first
                # steps, after the pool: leave them their room
                rows = max_tokens_per_step + min(max_tokens_per_step, ModelRunner.MAX_PORTION_ROWS)
                reserve = rows * self.model.activation_bytes_per_row() + 2 * ModelRunner.MAX_PORTION_LOGITS_BYTES
                free, _ = torch.cuda.mem_get_info(self.device)
                num_pages = max(1, min(num_pages, int(max(0, free - reserve) * cache_memory_fraction) // probe))
        self.runner = ModelRunner(self.model, num_pages=num_pages, page_size=page_size,
                                  max_requests=max_requests, max_seq_len=self.max_seq_len,
                                  max_tokens_per_step=max_tokens_per_step)
        self.scheduler = Scheduler(self.runner.cache, max_tokens_per_step=max_tokens_per_step,
                                   max_requests=max_requests, chunk_size=chunk_size,
                                   eos_token_ids=spec.eos_token_ids)
        self.sampler = Sampler(spec.vocab_size, max_requests, self.device)
        self.runner.feed_source = self.sampler.out       # decode graphs gather fed tokens from it themselves
        self._requests: Dict[Hashable, Request] = {}
        self._next_id = 0
        self._inflight = None          # (plan, pending tokens, row of each request, device tokens) of a launched step
        self.pipeline = bool(pipeline)  # decode one step ahead of the device
        self.h2d_bytes = 0
        self.d2h_bytes = 0

    # ------------------------------------------------------------------ the loop
    def add_request(self, prompt: Sequence[int], params: Optional[SamplingParams] = None,
                    request_id: Optional[Hashable] = None, rng_key: Optional[int] = None) -> Hashable:
        """Queue a request.  ``rng_key`` numbers its random stream (default: arrival order); with
        the same seed and key a request draws the same tokens whatever runs beside it."""
        if request_id is None:
            request_id = self._next_id
            self._next_id += 1
        if request_id in self._requests:
            raise KeyError(f"request id {request_id!r} is in use")
        V = self.model.spec.vocab_size
        prompt = [int(t) for t in prompt]
        for t in prompt:
            if not (0 <= t < V):
                raise ValueError(f"prompt token {t} is outside the vocabulary (0..{V - 1})")
        if len(prompt) >= self.max_seq_len:
            raise ValueError(f"prompt of {len(prompt)} tokens leaves no room in a context of {self.max_seq_len}")
        req = Request(request_id, prompt, params or SamplingParams(), key=rng_key)
        self._requests[request_id] = req
        self.scheduler.add(req)
        return request_id

    def step(self) -> List[Request]:
        """One turn of the loop; returns the requests that finished in it.

        While requests only decode, the host runs one step ahead of the device: the next step
        is launched with its tokens taken on the device from the sampler's output, and only
        then are the tokens of the step before read and checked for stop conditions.  A request
        that stops is found one step late; the token computed for it meanwhile is dropped."""
        done: List[Request] = []
        if self._inflight is None:
            plan = self.scheduler.plan()
            done += plan.failed
            if not plan.entries:
                return done
            rec = self._launch(plan, None)
            if rec is None:                                   # nothing sampled: nothing to wait for
                done += self.scheduler.commit(plan, [])
                return done
            self.scheduler.commit_ahead(plan)
            self._inflight = rec
        ahead = self.scheduler.decode_ahead_plan() if self.pipeline else None
        nxt = None
        if ahead is not None:
            nxt = self._launch(ahead, self._inflight)
            self.scheduler.commit_ahead(ahead)
        plan, pending = self._inflight[0], self._inflight[1]
        tokens = pending.tokens()                             # device -> host: the step's result
        self.d2h_bytes += 4 * len(tokens)
        done += self.scheduler.finalize(plan, tokens)
        self._inflight = nxt
        return done

    def _launch(self, plan: StepPlan, prev):
        """Launch the model and the sampler for ``plan``.  Returns (plan, pending tokens, row of
        each sampled request) or None if the plan samples nothing.  ``prev``: the record of the
        step in flight, whose sampled tokens are this step's inputs where the host has only a
        placeholder."""
        entries, feed, any_feed = [], [], False
        for e in plan.entries:
            toks = e.request.tokens[e.start:e.start + e.count]
            for j, t in enumerate(toks):
                if t < 0:                                     # a placeholder: the token is still on the device
                    toks[j] = 0
                    feed.append(prev[2][e.request.id])
                    any_feed = True
                else:
                    feed.append(-1)
            entries.append(StepEntry(e.request.id, toks, [e.count - 1] if e.sample else []))
        rows = [e.request for e in plan.entries if e.sample]
        # an all-greedy decode step takes its argmax inside the step's CUDA graph
        greedy = len(rows) == len(plan.entries) and all(not r.params.temperature > 0 for r in rows)
        logits = self.runner.step(entries, token_feed=(prev[3], feed) if any_feed else None,
                                  greedy_into=self.sampler.out if greedy else None)
        fed_apart = any_feed and not self.runner.fed_in_graph
        self.h2d_bytes += 4 * (self.runner.last_meta_words + (len(feed) if fed_apart else 0))
        if not rows:
            return None
        if self.runner.sampled_in_graph:
            tok = self.sampler.out[:len(rows)]
        else:
            tok = self.sampler.sample(
                logits, [r.params.temperature for r in rows], [r.params.top_p for r in rows],
                [uniform_for(r.params.seed, r.key, len(r.output)) for r in rows])
        return plan, self.sampler.fetch(tok), {r.id: i for i, r in enumerate(rows)}, tok

    def run(self) -> List[Request]:
        finished: List[Request] = []
        while self.scheduler.has_work() or self._inflight is not None:
            finished += self.step()
        return finished

    def generate(self, prompts: Sequence[Sequence[int]], *, max_new_tokens: int = 16, temperature: float = 0.0,
                 top_p: float = 1.0, seed: int = DEFAULT_SEED, stop_token_ids: Sequence[int] = (),
                 ignore_eos: bool = False) -> List[List[int]]:
        """Generated token ids for each prompt (prompt not included), in the order given."""
        params = SamplingParams(temperature=temperature, top_p=top_p, max_new_tokens=max_new_tokens, seed=seed,
                                stop_token_ids=tuple(stop_token_ids), ignore_eos=ignore_eos)
        ids = [self.add_request(p, params, rng_key=i) for i, p in enumerate(prompts)]
        self.run()
        self.runner.check_status()
        out = [self._requests[i].output for i in ids]
        self.last_finish_reasons = [self._requests[i].finish_reason for i in ids]
        for i in ids:
            del self._requests[i]
        return out

    def stats(self) -> Dict[str, object]:
        s = self.runner.stats()
        s.update(waiting=len(self.scheduler.waiting), running=len(self.scheduler.running),
                 h2d_bytes=self.h2d_bytes, d2h_bytes=self.d2h_bytes, preemptions=self.scheduler.preemptions)
        return s
