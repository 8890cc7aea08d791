"""Token choice: greedy, and temperature sampling with a reproducible draw per (seed, request, step).

The reference chooses ``argmax`` and reads it back with one host sync per step
(ampere_kv/runner.py:346, ampere_kv/scheduler.py:142, :189).  Temperature sampling is added
here: ``p = softmax(logits / T)`` in float32 on the device, inverted at a uniform number that
depends only on the sampling seed, the request's stream number and the index of the token
within the request, never on what else is in the batch.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from ..kernels import ops

_MASK = (1 << 64) - 1


def _mix64(x: int) -> int:
    x = (x + 0x9E3779B97F4A7C15) & _MASK
    x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
    x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & _MASK
    return x ^ (x >> 31)


def uniform_for(seed: int, stream: int, step: int) -> float:
    """Uniform in [0, 1) with 24 random bits, a pure function of its three keys."""
    x = _mix64(seed & _MASK)
    x = _mix64(x ^ (stream & _MASK))
    x = _mix64(x ^ (step & _MASK))
    return (x >> 40) / float(1 << 24)


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.0   # 0 = greedy
    seed: int = 0
    stream: int = 0            # distinguishes requests that share a seed

    def __post_init__(self):
        if self.temperature < 0:
            raise ValueError("temperature must not be negative")


class Sampler:
    #: pinned staging buffers in turn: a copy may still be under way when the next step is prepared
    RING = 4

    def __init__(self, device):
        self.device = torch.device(device)
        self._staging: list[torch.Tensor] = []
        self._turn = 0

    def _stage(self, rows: int) -> torch.Tensor:
        """A pinned [2, rows] float32 buffer (temperatures, uniforms) that no copy of the last RING - 1 steps reads."""
        if not self._staging or self._staging[0].shape[1] < rows:
            size = max(64, 2 * rows)
            self._staging = [torch.empty((2, size), dtype=torch.float32).pin_memory() for _ in range(self.RING)]
        self._turn = (self._turn + 1) % self.RING
        return self._staging[self._turn][:, :rows]

    def sample(self, logits: torch.Tensor, params: list[SamplingParams], steps: list[int],
               out: torch.Tensor | None = None) -> torch.Tensor:
        """int32 token per row of ``logits`` (on the device; no sync), written into ``out`` when that is given."""
        if logits.shape[0] != len(params):
            raise ValueError("one SamplingParams per logits row")
        values = torch.tensor([[p.temperature for p in params],
                               [uniform_for(p.seed, p.stream, s) if p.temperature > 0 else 0.0
                                for p, s in zip(params, steps)]], dtype=torch.float32)
        if self.device.type == "cuda":
            host = self._stage(len(params))
            host.copy_(values)
            dev = torch.empty((2, len(params)), dtype=torch.float32, device=self.device)
            dev.copy_(host, non_blocking=True)
        else:
            dev = values
        return ops.sample(logits.contiguous(), dev[0], dev[1], out=out)
