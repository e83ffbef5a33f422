"""The engine's look at what the kernels report about themselves.

Waits inside the TMA and tcgen05 kernels are bounded; one that runs out leaves a code in a word on the device and
the kernel's rows unwritten, and a row whose position lies outside the rotation tables is left out and recorded
likewise.  Nothing on the device stops because of it, so the loop has to look: the words are asked for in stream
order every few steps and whenever a request has ended, and read from pinned memory when they have arrived, so
that looking costs no wait.  The reference ends a request whose step failed with an error
(inferrs/src/engine.rs:812-821); so does the engine when a word is set.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .. import kernels


class KernelHealth:
    def __init__(self, dtype: torch.dtype, every: int = 16):
        self.dtype = dtype
        self.every = every                   # steps between two looks when no request ends
        self.host = torch.zeros((8,), dtype=torch.int32).pin_memory()
        self.event: Optional[torch.cuda.Event] = None

    @property
    def pending(self) -> bool:
        return self.event is not None

    def queue(self):
        """Ask for the words behind everything launched so far."""
        kernels.error_words_async(self.host, self.dtype)
        self.event = torch.cuda.Event()
        self.event.record()

    def poll(self, wait: bool = False) -> Optional[Dict[str, int]]:
        """None while nothing was asked for or the answer is not there yet (``wait``: wait for it); else the
        words that were set as {name: code}, empty if all were zero."""
        if self.event is None:
            return None
        if not wait and not self.event.query():
            return None
        self.event.synchronize()
        self.event = None
        words = self.host[:len(kernels.ERROR_WORDS)].tolist()
        return {name: int(v) for name, v in zip(kernels.ERROR_WORDS, words) if v}

    def reset(self) -> Dict[str, int]:
        """Clear the words on the device (waits for it); returns what was set."""
        return kernels.reset_error_words(self.dtype)
