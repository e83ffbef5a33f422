"""Per-request sampling options, with the reference's names, meanings and defaults
(inferrs/src/sampler.rs:27-112)."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Tuple

GREEDY_EPS = 1e-5  # temperatures below this pick the largest logit (sampler.rs:114, :176-179)


@dataclass
class SamplingParams:
    temperature: float = 0.7
    top_p: float = 0.9
    top_k: int = 50                      # 0: off
    repetition_penalty: float = 1.1      # 1.0: off; logit / p if >= 0 else logit * p, once per distinct token
    repeat_last_n: int = 64              # window of previous tokens the penalties look at; 0: off
    frequency_penalty: float = 0.0       # logit -= f * (times seen in the window)
    presence_penalty: float = 0.0        # logit -= q for tokens seen in the window
    min_p: float = 0.0                   # keep p >= min_p * p_max; 0: off
    max_tokens: int = 2048
    stop_token_ids: Tuple[int, ...] = ()  # the reference's extra_stop_token_ids
    seed: Optional[int] = None           # None: a fresh random seed per request
    ignore_eos: bool = False             # the reference's bypass_stop_tokens

    def __post_init__(self):
        if self.temperature < 0:
            raise ValueError(f"temperature must be >= 0, got {self.temperature}")
        if not 0.0 < self.top_p <= 1.0:
            raise ValueError(f"top_p must be in (0, 1], got {self.top_p}")
        if self.top_k < 0:
            raise ValueError(f"top_k must be >= 0, got {self.top_k}")
        if not 0.0 <= self.min_p <= 1.0:
            raise ValueError(f"min_p must be in [0, 1], got {self.min_p}")
        if self.max_tokens <= 0:
            raise ValueError(f"max_tokens must be positive, got {self.max_tokens}")
        if self.repeat_last_n < 0:
            raise ValueError(f"repeat_last_n must be >= 0, got {self.repeat_last_n}")
        self.stop_token_ids = tuple(int(t) for t in self.stop_token_ids)

    @classmethod
    def greedy(cls, max_tokens: int = 2048, **kw) -> "SamplingParams":
        """Largest logit, no penalties."""
        return cls(temperature=0.0, top_p=1.0, top_k=0, repetition_penalty=1.0, max_tokens=max_tokens, **kw)

    @property
    def is_greedy(self) -> bool:
        return self.temperature < GREEDY_EPS

    @property
    def has_penalty(self) -> bool:
        return self.repeat_last_n > 0 and (self.repetition_penalty not in (1.0, 0.0) or self.frequency_penalty != 0.0
                                           or self.presence_penalty != 0.0)


_M64 = (1 << 64) - 1


def _splitmix(x: int) -> int:
    x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & _M64
    x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & _M64
    return x ^ (x >> 31)


def uniform_for(seed: int, step: int) -> float:
    """The random number in [0, 1) for a request's seed and ``step`` = number of tokens it holds so far
    (prompt and generated): the reference's stateless generator (sampler.rs:370-397).  Being a function
    of (seed, step) only, a request's draws do not depend on what else is in the batch."""
    x = _splitmix((int(seed) + 0x9E3779B97F4A7C15) & _M64)
    x = (x + ((int(step) + 1) * 0x9E3779B97F4A7C15)) & _M64
    x = _splitmix(x)
    if x == 0:
        x = 0x1234567890ABCDEF
    x ^= (x << 13) & _M64
    x ^= x >> 7
    x ^= (x << 17) & _M64
    u = ((x * 0x2545F4914F6CDD1D) & _M64) >> 32
    return u / 4294967296.0


def uniforms_for(seeds, steps):
    """:func:`uniform_for` for many (seed, step) pairs at once, with the same bits: 64-bit arithmetic that wraps
    around, in numpy.  Returns float32 [n]."""
    import numpy as np

    def splitmix(x):
        x = (x ^ (x >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
        x = (x ^ (x >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
        return x ^ (x >> np.uint64(31))

    with np.errstate(over="ignore"):
        golden = np.uint64(0x9E3779B97F4A7C15)
        x = splitmix(np.array([int(s) & _M64 for s in seeds], dtype=np.uint64) + golden)
        x = splitmix(x + (np.array([int(n) + 1 for n in steps], dtype=np.uint64) * golden))
        x = np.where(x == 0, np.uint64(0x1234567890ABCDEF), x)
        x ^= x << np.uint64(13)
        x ^= x >> np.uint64(7)
        x ^= x << np.uint64(17)
        u = (x * np.uint64(0x2545F4914F6CDD1D)) >> np.uint64(32)
    return (u.astype(np.float64) / 4294967296.0).astype(np.float32)

