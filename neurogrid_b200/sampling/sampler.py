"""Sampling parameters, the per-request random stream and the device sampler.

The reference samples on the host with one engine-wide ``math/rand`` stream seeded 42
(pkg/inference/sampler.go:25-51, pkg/inference/engine.go:158): greedy when temperature <= 0,
else temperature softmax, optional top-p, inverse-CDF draw.  Here the draw runs on the
device over float32 logits, and the uniform number of a draw is a counter-based hash of
(seed, request key, index of the generated token), so a request's tokens do not depend on
what else was in its batches.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Sequence, Tuple

import torch

from ..csrc import ops

DEFAULT_SEED = 42          # the reference's engine-wide sampler seed (pkg/inference/engine.go:158)
_M64 = (1 << 64) - 1


@dataclass(frozen=True)
class SamplingParams:
    """temperature <= 0 is greedy.  Defaults follow the reference's API
    (api/types.go:31-41: temperature 0.7, top_p 1.0, max_tokens 2048)."""
    temperature: float = 0.7
    top_p: float = 1.0
    max_new_tokens: int = 2048
    seed: int = DEFAULT_SEED
    stop_token_ids: Tuple[int, ...] = ()
    ignore_eos: bool = False


def _splitmix64(x: int) -> int:
    x = (x + 0x9E3779B97F4A7C15) & _M64
    z = x
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _M64
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _M64
    return z ^ (z >> 31)


def uniform_for(seed: int, request_key: int, index: int) -> float:
    """A number in [0, 1) with 24 random bits, a pure function of its three arguments."""
    h = _splitmix64(_splitmix64(_splitmix64(seed & _M64) ^ (request_key & _M64)) ^ (index & _M64))
    return (h >> 40) / float(1 << 24)


class Sampler:
    """Device sampler: one launch for a batch of rows with per-row temperature and top-p.

    ``sample`` leaves the tokens on the device; ``fetch`` starts their copy to pinned host
    memory and returns a handle whose ``tokens()`` waits for it, so that the caller may launch
    more work before it reads them."""

    RING = 4

    def __init__(self, vocab_size: int, max_rows: int, device):
        self.vocab_size, self.max_rows, self.device = vocab_size, max_rows, device
        self._scratch: Optional[torch.Tensor] = None
        self._cuda = torch.device(device).type == "cuda"
        self._params = [torch.zeros((3, max_rows), dtype=torch.float32, pin_memory=self._cuda) for _ in range(self.RING)]
        self._param_events = [torch.cuda.Event() if self._cuda else None for _ in range(self.RING)]
        self._param_used = [False] * self.RING
        self._tokens = [torch.zeros(max_rows, dtype=torch.int32, pin_memory=self._cuda) for _ in range(self.RING)]
        self._next = 0
        self._dev = torch.zeros((3, max_rows), dtype=torch.float32, device=device)
        # One buffer for the sampled tokens: what reads it (the copy to the host, the next step's
        # token feed) is queued on the stream before the next sampling writes it.  Sized for a
        # batch padded to a power of two.
        self.out = torch.zeros(1 << max(0, (max_rows - 1).bit_length()), dtype=torch.int32, device=device)

    def sample(self, logits: torch.Tensor, temperature: Sequence[float], top_p: Sequence[float],
               uniform: Sequence[float]) -> torch.Tensor:
        """int32 [W] on the device, a view of ``self.out`` (valid until the next sampling).
        All-greedy batches take the argmax-only path (no scratch)."""
        W = logits.shape[0]
        if W > self.max_rows:
            raise ValueError(f"{W} rows to sample, sampler sized for {self.max_rows}")
        out = self.out[:W]
        if all(not t > 0 for t in temperature):
            ops.sample(logits, None, None, None, out, None)
            return out
        if self._scratch is None or self._scratch.shape[0] < W:
            self._scratch = torch.empty((max(W, min(self.max_rows, 8)), self.vocab_size), dtype=torch.float32,
                                        device=self.device)
        i = self._next
        self._next = (i + 1) % self.RING
        if self._param_used[i] and self._cuda:
            self._param_events[i].synchronize()
        h = self._params[i]
        h[:, :W] = torch.tensor([list(temperature), list(top_p), list(uniform)], dtype=torch.float32)
        self._dev.copy_(h, non_blocking=True)
        if self._cuda:
            self._param_events[i].record()
            self._param_used[i] = True
        ops.sample(logits, self._dev[0, :W], self._dev[1, :W], self._dev[2, :W], out, self._scratch)
        return out

    def fetch(self, tokens: torch.Tensor) -> "PendingTokens":
        """Start copying sampled tokens to the host."""
        i = self._next
        self._next = (i + 1) % self.RING
        host = self._tokens[i][: tokens.shape[0]]
        host.copy_(tokens, non_blocking=True)
        ev = None
        if self._cuda:
            ev = torch.cuda.Event()
            ev.record()
        return PendingTokens(host, ev)


class PendingTokens:
    def __init__(self, host: torch.Tensor, event):
        self._host, self._event = host, event

    def tokens(self) -> List[int]:
        if self._event is not None:
            self._event.synchronize()
        return self._host.tolist()
