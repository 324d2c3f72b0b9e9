"""Chooses the next token of every request that reached the end of its tokens in
a step (python/helios/exec/sampler.py:20-91).  One kernel launch per step samples
all rows on the device; one copy brings the token ids back."""
from __future__ import annotations

from typing import List, Sequence

import numpy as np
import torch

from ..csrc import ops


class Sampler:
    def sample(self, logits: torch.Tensor, params: Sequence, seeds: Sequence[int],
               offsets: Sequence[int]) -> List[int]:
        """``logits``: float32 [R, V] on the device; ``params[i]`` has temperature, top_k and
        top_p; row i draws its uniform from (seeds[i], offsets[i])."""
        R = logits.shape[0]
        if not (len(params) == len(seeds) == len(offsets) == R):
            raise ValueError("one set of sampling options per logits row is required")
        f = np.empty((2, R), np.float32)
        i32 = np.empty((R,), np.int32)
        i64 = np.empty((2, R), np.int64)
        for i, p in enumerate(params):
            f[0, i], f[1, i] = p.temperature, p.top_p
            i32[i] = p.top_k
            i64[0, i] = np.uint64(seeds[i] & (2**64 - 1)).astype(np.int64)
            i64[1, i] = offsets[i]
        dev = logits.device
        fd = torch.from_numpy(f).to(dev, non_blocking=True)
        kd = torch.from_numpy(i32).to(dev, non_blocking=True)
        sd = torch.from_numpy(i64).to(dev, non_blocking=True)
        out = ops.sample(logits, fd[0].contiguous(), kd, fd[1].contiguous(), sd[0].contiguous(),
                         sd[1].contiguous())
        return out.cpu().tolist()
