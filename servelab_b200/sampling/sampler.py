"""Device sampler: one kernel launch per step for all rows.

Semantics of greedy / temperature / top-k / top-p follow the reference's
``Sampler`` (servelab/engine/sampler.py:15-45).  Randomness differs on purpose:
the reference consumes one host generator in batch order and re-seeds a
per-request generator for every token (sampler.py:26-28); here each draw is a
counter-based random number keyed by (seed, request stream, output position), so
a request's tokens do not depend on what else is in the batch.  A request with
``seed >= 0`` uses that seed with stream 0; others use the engine's seed and
their own stream number.
"""

from __future__ import annotations

import struct
from typing import List, Sequence

import torch

from ..ops import kernels as K


def _f2i(x: float) -> int:
    return struct.unpack("<i", struct.pack("<f", x))[0]


class PendingTokens:
    """Tokens that have been sampled on the device and are on their way to the host:
    ``device`` holds them (int32 [R]) for kernels launched after the sampler; ``wait()``
    blocks until THEIR copy has arrived, not until the stream is idle, so work queued
    after the sampler keeps running."""

    def __init__(self, device_ids: torch.Tensor, host_ids: torch.Tensor, event):
        self.device, self._host, self._event = device_ids, host_ids, event

    def wait(self) -> List[int]:
        if self._event is not None:
            self._event.synchronize()
        return self._host.tolist()


class Sampler:
    def __init__(self, seed: int = 0, device: str = "cuda:0"):
        self.seed = int(seed) & ((1 << 63) - 1)
        self.device = device
        self._pinned = {}          # rows -> two pinned host buffers used in turn
        self._flip = 0

    def sample(self, logits: torch.Tensor, seqs: Sequence) -> List[int]:
        """One token per row of ``logits`` [R, V]; ``seqs[r]`` supplies
        ``sampling_params``, ``stream_id`` and ``num_output_tokens``."""
        return self.sample_async(logits, seqs).wait()

    def _pinned_words(self, n: int) -> torch.Tensor:
        """One of four pinned buffers of ``n`` ints, used in turn (a buffer is written
        again only after three later steps' parameters have been queued)."""
        ring = self._pinned.get(("words", n))
        if ring is None:
            ring = self._pinned[("words", n)] = [[torch.empty(n, dtype=torch.int32, pin_memory=True)
                                                  for _ in range(4)], 0]
        ring[1] = (ring[1] + 1) % 4
        return ring[0][ring[1]]

    def _to_host(self, out: torch.Tensor) -> PendingTokens:
        R = out.shape[0]
        pair = self._pinned.get(R)
        if pair is None:
            pair = self._pinned[R] = [torch.empty(R, dtype=torch.int32, pin_memory=True)
                                      for _ in range(2)]
        self._flip ^= 1
        host = pair[self._flip]
        host.copy_(out, non_blocking=True)
        event = torch.cuda.Event()
        event.record()
        return PendingTokens(out, host, event)

    def sample_async(self, logits: torch.Tensor, seqs: Sequence, ahead: int = 0) -> PendingTokens:
        """Launches the sampler and the copy of its result to the host; returns at once.
        ``ahead``: output tokens each request will have got between now and this draw
        (a step launched before the previous step's tokens were read back)."""
        R = logits.shape[0]
        if R == 0:
            return PendingTokens(torch.empty(0, dtype=torch.int32, device=self.device),
                                 torch.empty(0, dtype=torch.int32), None)
        out = torch.empty(R, dtype=torch.int32, device=self.device)
        if all(s.sampling_params.temperature == 0.0 for s in seqs):
            K.sample_rows(logits, out)
            return self._to_host(out)
        # [temperature | top_k | top_p | position | seed (2 words) | stream (2 words)]
        words: List[int] = []
        words += [_f2i(float(s.sampling_params.temperature)) for s in seqs]
        words += [int(s.sampling_params.top_k) for s in seqs]
        words += [_f2i(float(s.sampling_params.top_p)) for s in seqs]
        words += [int(s.num_output_tokens) + ahead for s in seqs]
        for s in seqs:
            sd = s.sampling_params.seed if s.sampling_params.seed >= 0 else self.seed
            words += [sd & 0xFFFFFFFF, (sd >> 32) & 0xFFFFFFFF]
        for s in seqs:
            st = 0 if s.sampling_params.seed >= 0 else int(s.stream_id)
            words += [st & 0xFFFFFFFF, (st >> 32) & 0xFFFFFFFF]
        # pinned and asynchronous: a pageable copy would make the host wait for the stream
        host = self._pinned_words(len(words))
        host.numpy()[:] = [w - (1 << 32) if w >= (1 << 31) else w for w in words]
        dev = host.to(self.device, non_blocking=True)
        temp = dev[0:R].view(torch.float32)
        top_k = dev[R:2 * R]
        top_p = dev[2 * R:3 * R].view(torch.float32)
        pos = dev[3 * R:4 * R]
        seed = dev[4 * R:6 * R]
        stream = dev[6 * R:8 * R]
        K.sample_rows(logits, out, temp, top_k, top_p, seed, stream, pos)
        return self._to_host(out)
