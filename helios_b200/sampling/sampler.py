"""Chooses the next token of every request that reached the end of its tokens in
a step (python/helios/exec/sampler.py:20-91).  One kernel launch per step samples
all rows on the device; one copy brings the token ids back."""
from __future__ import annotations

from typing import List, Sequence

import numpy as np
import torch

from ..csrc import ops


class _Staging:
    def __init__(self, words: int) -> None:
        self.host = torch.empty(words, dtype=torch.int32, pin_memory=True)
        self.event = torch.cuda.Event()


class Sampler:
    """The per-row options travel in one copy from pinned memory, so that sampling never
    makes the host wait for the device (a copy from pageable memory may)."""

    RING = 4

    def __init__(self) -> None:
        self._ring: List[_Staging] = []
        self._next = 0

    def _staging(self, words: int) -> _Staging:
        if len(self._ring) < self.RING:
            self._ring.append(_Staging(max(words, 7 * 64)))
            return self._ring[-1]
        st = self._ring[self._next]
        self._next = (self._next + 1) % self.RING
        st.event.synchronize()                 # its last copy has left the host
        if st.host.numel() < words:
            st.host = torch.empty(words, dtype=torch.int32, pin_memory=True)
        return st

    def sample(self, logits: torch.Tensor, params: Sequence, seeds: Sequence[int],
               offsets: Sequence[int]) -> List[int]:
        return self.sample_device(logits, params, seeds, offsets).cpu().tolist()

    def sample_device(self, logits: torch.Tensor, params: Sequence, seeds: Sequence[int],
                      offsets: Sequence[int]) -> torch.Tensor:
        """``logits``: float32 [R, V] on the device; ``params[i]`` has temperature, top_k and
        top_p; row i draws its uniform from (seeds[i], offsets[i]).  Returns int32 [R] on the
        device; nothing waits for the device."""
        R = logits.shape[0]
        if not (len(params) == len(seeds) == len(offsets) == R):
            raise ValueError("one set of sampling options per logits row is required")
        # int32 words: seeds (int64) | offsets (int64) | temperature | top_p | top_k
        st = self._staging(7 * R)
        words = st.host.numpy()[:7 * R]
        i64 = words[:4 * R].view(np.int64)
        f32 = words[4 * R:6 * R].view(np.float32)
        top_k = words[6 * R:]
        # whole arrays at once: with hundreds of rows a loop of scalar stores costs a millisecond
        mask = 2**64 - 1
        i64[:R] = np.fromiter((s & mask for s in seeds), dtype=np.uint64, count=R).view(np.int64)
        i64[R:] = offsets
        f32[:R] = [p.temperature for p in params]
        f32[R:] = [p.top_p for p in params]
        top_k[:] = [p.top_k for p in params]
        if any(p.temperature > 0 and (p.top_k > 0 or p.top_p < 1.0) for p in params):
            kind = "narrow"
        else:
            kind = "draw" if any(p.temperature > 0 for p in params) else "greedy"
        dev = torch.empty(7 * R, dtype=torch.int32, device=logits.device)
        dev.copy_(st.host[:7 * R], non_blocking=True)
        st.event.record()
        d64 = dev[:4 * R].view(torch.int64)
        d32 = dev[4 * R:6 * R].view(torch.float32)
        return ops.sample(logits, d32[:R], dev[6 * R:], d32[R:], d64[:R], d64[R:], kind=kind)
