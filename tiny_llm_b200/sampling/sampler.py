"""Chooses next tokens on the device from the step's 32-bit logits.  The reference copies the
logits to the host and runs its processor chain there (tiny_llm/pipeline/pipeline.cpp:193-207)."""
from __future__ import annotations

from typing import List, Sequence

import numpy as np
import torch

from .. import ops
from .params import SamplingParams


def uniform_from(seed: int, counter: int) -> float:
    """The uniform number in [0, 1) the sampling kernel draws for (seed, counter): splitmix64 of
    seed + (counter + 1) * golden ratio, top 24 bits."""
    mask = (1 << 64) - 1
    z = (seed + (counter + 1) * 0x9E3779B97F4A7C15) & mask
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & mask
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & mask
    z = z ^ (z >> 31)
    return (z >> 40) / 16777216.0


class SampleTicket:
    """A launched sampling call: the chosen ids are in `device_out` (stream-ordered) and on their
    way to a pinned host buffer; `Sampler.collect` waits for them."""

    def __init__(self, n: int, slot: int, event, device_out: torch.Tensor):
        self.n, self.slot, self.event, self.device_out = n, slot, event, device_out


class Sampler:
    RING = 3   # host buffers in flight: a caller may launch the next step before it collects this one

    def __init__(self, device, vocab_size: int, max_rows: int = 256):
        self.device = torch.device(device)
        self.vocab_size = vocab_size
        self.max_rows = max_rows + max_rows % 2   # the 64-bit regions of the block start at even words
        pin = self.device.type == "cuda"
        # one host block: temperature f32 | top_p f32 | top_k i32 | seeds i64 | counters i64, as int32 words
        self._words = self.max_rows * 7
        self._host = [torch.zeros(self._words, dtype=torch.int32, pin_memory=pin) for _ in range(self.RING)]
        self._host_free = [None] * self.RING      # event: the copy that last read this block has run
        self._dev = torch.zeros(self._words, dtype=torch.int32, device=self.device)
        # the chosen ids, and behind them the status word of the step's kernels (see collect)
        self._out = torch.zeros(self.max_rows + 1, dtype=torch.int32, device=self.device)
        self._out_host = [torch.zeros(self.max_rows + 1, dtype=torch.int32, pin_memory=pin) for _ in range(self.RING)]
        self._status = ops.status_word(self.device) if pin else None
        self._next = 0
        self._work = None

    def _views(self, buf, n):
        m = self.max_rows
        return (buf[0:n].view(torch.float32), buf[m:m + n].view(torch.float32), buf[2 * m:2 * m + n],
                buf[3 * m:3 * m + 2 * n].view(torch.int64), buf[5 * m:5 * m + 2 * n].view(torch.int64))

    def launch(self, logits: torch.Tensor, params: Sequence[SamplingParams], counters: Sequence[int]) -> SampleTicket:
        """Enqueues the choice of one token per row of `logits` and its copy to the host;
        `counters[i]` is how many tokens row i's request has drawn."""
        n = logits.shape[0]
        if n > self.max_rows:
            raise ValueError(f"{n} rows exceed the sampler's {self.max_rows}")
        slot = self._next
        self._next = (slot + 1) % self.RING
        out = self._out[:n + 1]
        if all(not p.do_sample for p in params):
            ops.argmax(logits, out, self._status)
        else:
            if self._host_free[slot] is not None:
                self._host_free[slot].synchronize()
            host = self._host[slot]
            t, pp, k, s, c = self._views(host, n)
            t.numpy()[:] = [p.temperature if p.do_sample else 0.0 for p in params]
            pp.numpy()[:] = [p.top_p for p in params]
            k.numpy()[:] = [p.top_k for p in params]
            s.numpy()[:] = np.array([p.seed & 0x7FFFFFFFFFFFFFFF for p in params], dtype=np.int64)
            c.numpy()[:] = np.array(list(counters), dtype=np.int64)
            self._dev.copy_(host, non_blocking=True)
            if self.device.type == "cuda":
                if self._host_free[slot] is None:
                    self._host_free[slot] = torch.cuda.Event()
                self._host_free[slot].record()
            if self._work is None or self._work.numel() < n * self.vocab_size:
                self._work = torch.empty(max(n, 8) * self.vocab_size, dtype=torch.float32, device=self.device)
            dt, dpp, dk, ds, dc = self._views(self._dev, n)
            ops.sample(logits, self._work, dt, dk, dpp, ds, dc, out, self._status)
        self._out_host[slot][:n + 1].copy_(out, non_blocking=True)
        event = None
        if self.device.type == "cuda":
            event = torch.cuda.Event()
            event.record()
        return SampleTicket(n, slot, event, out[:n])

    def collect(self, ticket: SampleTicket) -> List[int]:
        """Waits for a launched call's ids and returns them.  The status word of the step's kernels
        came with them in the same copy: if a kernel gave up one of its bounded waits, the ids were
        drawn from logits that are not valid, and this raises instead of returning them (the
        reference throws on every failed CUDA call, tiny_llm/common/cuda_checks.hpp:8-20)."""
        if ticket.event is not None:
            ticket.event.synchronize()
        row = self._out_host[ticket.slot][:ticket.n + 1].tolist()
        if row[ticket.n]:
            ops.raise_status(self.device, row[ticket.n])
        return row[:ticket.n]

    def sample(self, logits: torch.Tensor, params: Sequence[SamplingParams], counters: Sequence[int]) -> List[int]:
        """launch + collect."""
        return self.collect(self.launch(logits, params, counters))
