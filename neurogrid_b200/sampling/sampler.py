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
    """Device sampler: one launch for a batch of rows with per-row temperature and top-p."""

    def __init__(self, vocab_size: int, max_rows: int, device):
        self.vocab_size, self.max_rows, self.device = vocab_size, max_rows, device
        self._scratch: Optional[torch.Tensor] = None
        pin = torch.device(device).type == "cuda"
        self._host = torch.zeros((3, max_rows), dtype=torch.float32, pin_memory=pin)
        self._dev = torch.zeros((3, max_rows), dtype=torch.float32, device=device)
        self._out = torch.zeros(max_rows, dtype=torch.int32, device=device)

    def sample(self, logits: torch.Tensor, temperature: Sequence[float], top_p: Sequence[float],
               uniform: Sequence[float]) -> torch.Tensor:
        """int32 [W] on the device.  All-greedy batches take the argmax-only path (no scratch)."""
        W = logits.shape[0]
        if W > self.max_rows:
            raise ValueError(f"{W} rows to sample, sampler sized for {self.max_rows}")
        out = self._out[:W]
        if all(not t > 0 for t in temperature):
            ops.sample(logits, None, None, None, out, None)
            return out
        if self._scratch is None or self._scratch.shape[0] < W:
            self._scratch = torch.empty((max(W, min(self.max_rows, 8)), self.vocab_size), dtype=torch.float32,
                                        device=self.device)
        h = self._host
        h[0, :W] = torch.tensor(list(temperature), dtype=torch.float32)
        h[1, :W] = torch.tensor(list(top_p), dtype=torch.float32)
        h[2, :W] = torch.tensor(list(uniform), dtype=torch.float32)
        self._dev.copy_(h, non_blocking=False)
        ops.sample(logits, self._dev[0, :W], self._dev[1, :W], self._dev[2, :W], out, self._scratch)
        return out
