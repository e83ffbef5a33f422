"""Choosing the next token of every row of a step, on the device.

The reference copies each row's logits to the host and samples there (inferrs/src/sampler.rs:146-357).
Here the rows of a step are sampled together by two kernels (penalties, then selection); what crosses
to the host is one token id per row.
"""
from __future__ import annotations

from typing import List, Sequence

import numpy as np
import torch

from .. import kernels
from .params import SamplingParams, uniform_for


class Sampler:
    def __init__(self, device: torch.device, act_dtype: torch.dtype = torch.float32):
        self.device = device
        self.act_dtype = act_dtype

    def sample(self, logits: torch.Tensor, params: Sequence[SamplingParams], seeds: Sequence[int],
               histories: Sequence[Sequence[int]], pending: "int | Sequence[int]" = 0,
               pending_ids: "torch.Tensor | None" = None) -> torch.Tensor:
        """int32 token ids [rows] (on the device) for float32 ``logits`` [rows, vocab].

        ``histories[r]`` is all tokens of row r's request so far, prompt and generated: its length is the
        step index of the random draw and its tail is the penalties' window.  It may be a list of token ids
        or an object with ``n_tokens`` and ``tail(n)`` (the scheduler's requests, which keep prompt and
        output apart).  ``logits`` is changed in place where penalties apply.  ``pending`` (0 or 1, one for all
        rows or one per row): the request has one more token that is on its way but not in its history yet; it
        counts for the step index of the draw, and ``pending_ids`` (int32 on the device, one per row; ignored
        where nothing is pending) has it for the penalties' window.
        """
        r = logits.shape[0]
        out = torch.empty((r,), dtype=torch.int32, device=self.device)
        if r == 0:
            return out
        if all(p.is_greedy and not p.has_penalty for p in params):
            kernels.argmax(logits, out, self.act_dtype)
            return out
        pend = [int(pending)] * r if isinstance(pending, int) else [int(x) for x in pending]
        if len(pend) != r or any(x not in (0, 1) for x in pend):
            raise ValueError("pending: 0 or 1, one for all rows or one per row")
        length = [(h.n_tokens if hasattr(h, "n_tokens") else len(h)) + x for h, x in zip(histories, pend)]
        if any(p.has_penalty for p in params):
            if any(pend) and pending_ids is None:
                raise ValueError("penalties need the whole history: the one pending token must be given on the device")
            width = max(1, max(min(p.repeat_last_n, n) if p.has_penalty else 0 for p, n in zip(params, length)))
            prev = np.full((r, width), -1, dtype=np.int32)
            n_prev = np.zeros((r,), dtype=np.int32)
            for i, (p, h) in enumerate(zip(params, histories)):
                if p.has_penalty:
                    # the window's order does not matter: the pending token, if any, takes the first place
                    known = p.repeat_last_n - pend[i]
                    tail = (h.tail(known) if hasattr(h, "tail") else list(h[-known:])) if known > 0 else []
                    prev[i, pend[i]:pend[i] + len(tail)] = tail
                    n_prev[i] = len(tail) + pend[i]
            f = np.array([[p.repetition_penalty if p.has_penalty else 1.0 for p in params],
                          [p.frequency_penalty if p.has_penalty else 0.0 for p in params],
                          [p.presence_penalty if p.has_penalty else 0.0 for p in params]], dtype=np.float32)
            fd = torch.from_numpy(f).to(self.device)
            prev_dev = torch.from_numpy(prev).to(self.device)
            if all(pend):
                prev_dev[:, 0].copy_(pending_ids[:r])
            elif any(pend):
                mask = torch.tensor(pend, dtype=torch.bool).to(self.device)
                prev_dev[:, 0] = torch.where(mask, pending_ids[:r].to(torch.int32), prev_dev[:, 0])
            kernels.penalties(logits, prev_dev, torch.from_numpy(n_prev).to(self.device), fd[0], fd[1], fd[2],
                              self.act_dtype)
        f = np.array([[p.temperature for p in params], [p.top_p for p in params], [p.min_p for p in params],
                      [uniform_for(s, n) for s, n in zip(seeds, length)]], dtype=np.float32)
        fd = torch.from_numpy(f).to(self.device)
        top_k = torch.tensor([p.top_k for p in params], dtype=torch.int32).to(self.device)
        kernels.sample(logits, fd[0], top_k, fd[1], fd[2], fd[3], out, self.act_dtype)
        return out
