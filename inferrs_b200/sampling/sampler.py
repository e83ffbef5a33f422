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
from .params import SamplingParams, uniforms_for


class Sampler:
    STAGING = 4      # pinned buffers used in turn: a step's numbers may still be on their way when the next is filled

    def __init__(self, device: torch.device, act_dtype: torch.dtype = torch.float32):
        self.device = device
        self.act_dtype = act_dtype
        self._staging = []       # [pinned int32 buffer, event of its last copy or None]
        self._turn = 0

    def _upload(self, words: np.ndarray) -> torch.Tensor:
        """The step's numbers (int32 words, floats as their bits) to the device with one copy that the host does not
        wait for: from one of a few pinned buffers, each reused only after its last copy has been made."""
        n = int(words.shape[0])
        if self.device.type != "cuda":
            return torch.from_numpy(words).to(self.device)
        if len(self._staging) < self.STAGING:
            self._staging.append([torch.empty((max(n, 4096),), dtype=torch.int32).pin_memory(), None])
            slot = self._staging[-1]
        else:
            slot = self._staging[self._turn]
            self._turn = (self._turn + 1) % self.STAGING
            if slot[1] is not None:
                slot[1].synchronize()
            if slot[0].shape[0] < n:
                slot[0] = torch.empty((2 * n,), dtype=torch.int32).pin_memory()
        slot[0].numpy()[:n] = words
        dev = torch.empty((n,), dtype=torch.int32, device=self.device)
        dev.copy_(slot[0][:n], non_blocking=True)
        slot[1] = torch.cuda.Event()
        slot[1].record()
        return dev

    def sample(self, logits: torch.Tensor, params: Sequence[SamplingParams], seeds: Sequence[int],
               histories: Sequence[Sequence[int]], pending: "int | Sequence[int]" = 0,
               pending_ids: "torch.Tensor | None" = None, pending_from=None) -> torch.Tensor:
        """int32 token ids [rows] (on the device) for float32 ``logits`` [rows, vocab].

        ``histories[r]`` is all tokens of row r's request so far, prompt and generated: its length is the
        step index of the random draw and its tail is the penalties' window.  It may be a list of token ids
        or an object with ``n_tokens`` and ``tail(n)`` (the scheduler's requests, which keep prompt and
        output apart).  ``logits`` is changed in place where penalties apply.  ``pending`` (0 or 1, one for all
        rows or one per row): the request has one more token that is on its way but not in its history yet; it
        counts for the step index of the draw, and ``pending_ids`` (int32 on the device, one per row; ignored
        where nothing is pending) has it for the penalties' window.  Instead of ``pending_ids``, ``pending_from`` =
        (ids, places) names a tensor of token ids on the device and, per row, the place of the row's pending token
        in it (any valid place where nothing is pending): the look-up then goes to the device with everything else.

        Everything the two kernels need per row goes to the device as one block of words in one copy that the
        host does not wait for, so a step can be prepared while the one before it still runs.
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
        penalised = [p.has_penalty for p in params]
        width = 0
        if any(penalised):
            if any(pend) and pending_ids is None and pending_from is None:
                raise ValueError("penalties need the whole history: the one pending token must be given on the device")
            width = max(1, max(min(p.repeat_last_n, n) if on else 0 for p, n, on in zip(params, length, penalised)))
        # the block: seven rows of floats (as their bits), two of ints, the penalties' windows, the pending tokens' places
        look_up = width > 0 and any(pend) and pending_ids is None
        words = np.empty((9 * r + r * width + (r if look_up else 0),), dtype=np.int32)
        floats = words[:7 * r].view(np.float32).reshape(7, r)
        floats[0] = [p.temperature for p in params]
        floats[1] = [p.top_p for p in params]
        floats[2] = [p.min_p for p in params]
        floats[3] = uniforms_for(seeds, length)
        floats[4] = [p.repetition_penalty if on else 1.0 for p, on in zip(params, penalised)]
        floats[5] = [p.frequency_penalty if on else 0.0 for p, on in zip(params, penalised)]
        floats[6] = [p.presence_penalty if on else 0.0 for p, on in zip(params, penalised)]
        words[7 * r:8 * r] = [p.top_k for p in params]
        n_prev = words[8 * r:9 * r]
        n_prev[:] = 0
        if width:
            prev = words[9 * r:9 * r + r * width].reshape(r, width)
            prev[:] = -1
            for i, (p, h) in enumerate(zip(params, histories)):
                if penalised[i]:
                    # the window's order does not matter: the pending token, if any, takes the first place
                    known = p.repeat_last_n - pend[i]
                    tail = (h.tail(known) if hasattr(h, "tail") else list(h[-known:])) if known > 0 else []
                    prev[i, pend[i]:pend[i] + len(tail)] = tail
                    n_prev[i] = len(tail) + pend[i]
        if look_up:
            words[9 * r + r * width:] = list(pending_from[1])
        dev = self._upload(words)
        fd = dev[:7 * r].view(torch.float32).view(7, r)
        if width:
            prev_dev = dev[9 * r:9 * r + r * width].view(r, width)
            if look_up:
                pending_ids = pending_from[0].index_select(0, dev[9 * r + r * width:])
            if all(pend):
                prev_dev[:, 0].copy_(pending_ids[:r])
            elif any(pend):
                mask = self._upload(np.array(pend, dtype=np.int32)).to(torch.bool)
                prev_dev[:, 0] = torch.where(mask, pending_ids[:r].to(torch.int32), prev_dev[:, 0])
            kernels.penalties(logits, prev_dev, dev[8 * r:9 * r], fd[4], fd[5], fd[6], self.act_dtype)
        kernels.sample(logits, fd[0], dev[7 * r:8 * r], fd[1], fd[2], fd[3], out, self.act_dtype)
        return out
