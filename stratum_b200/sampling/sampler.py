"""Picking next tokens on the device from the step's logits."""
from __future__ import annotations

from typing import List, Optional, Sequence

import numpy as np
import torch

from .. import kernels as K
from .params import SamplingParams
from .pcg32 import Pcg32


class Sampler:
    """Greedy or temperature/top-k/top-p sampling of one token per logits row.

    Every request owns a PCG32 stream (seed, request index); a row's uniform is drawn on the host
    and handed to the kernel, so the pick depends only on the row's logits and the request's own
    stream.
    """

    def __init__(self, device):
        self.device = torch.device(device)

    def pick(self, logits: torch.Tensor, params: SamplingParams, streams: Optional[Sequence[Pcg32]] = None,
             want_values: bool = False):
        """logits float32 [n, vocab] on the device -> (ids int32 [n] on the device, values or None)."""
        n = logits.shape[0]
        ids = torch.empty(n, dtype=torch.int32, device=self.device)
        values = torch.empty(n, dtype=torch.float32, device=self.device) if want_values else None
        if n == 0:
            return ids, values
        if params.greedy:
            K.argmax(logits, ids, values)
            return ids, values
        if streams is None or len(streams) != n:
            raise ValueError("sampling needs one random stream per row")
        host = np.empty((4, n), dtype=np.float32)
        host[0, :] = params.temperature
        host[1, :] = np.array([params.top_k], dtype=np.int32).view(np.float32)[0]
        host[2, :] = params.top_p
        host[3, :] = [s.uniform() for s in streams]
        dev = torch.from_numpy(host).to(self.device)
        # (with filters and many rows the kernel that gives a row one block is ahead: engine/graphs.py, pick_kind)
        many_filtered = n > 32 and (params.top_k > 0 or params.top_p < 1.0)
        K.sample(logits, dev[0], dev[1].view(torch.int32), dev[2], dev[3], ids, values,
                 one_block_per_row=many_filtered)
        return ids, values
