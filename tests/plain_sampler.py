"""A plain sampler on the host, written from the reference's (inferrs/src/sampler.rs:146-397):
penalties, temperature, softmax, stable sort by probability, top-k, top-p, min-p, renormalise, walk.
It shares no code with the package (the random generator is restated here too)."""
import numpy as np

M64 = (1 << 64) - 1


def _mix(x):
    x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & M64
    x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & M64
    return x ^ (x >> 31)


def rand_f32(seed, step):
    """sampler.rs:370-397."""
    x = _mix((seed + 0x9E3779B97F4A7C15) & M64)
    x = _mix((x + (step + 1) * 0x9E3779B97F4A7C15) & M64)
    if x == 0:
        x = 0x1234567890ABCDEF
    x ^= (x << 13) & M64
    x ^= x >> 7
    x ^= (x << 17) & M64
    return np.float32((((x * 0x2545F4914F6CDD1D) & M64) >> 32) / 4294967296.0)


def sample_token(logits, previous, temperature=0.7, top_p=0.9, top_k=50, repetition_penalty=1.1, repeat_last_n=64,
                 frequency_penalty=0.0, presence_penalty=0.0, min_p=0.0, seed=0, precise=False):
    """sampler.rs:146-357; ``previous`` is every token of the request so far.

    The reference sums and walks in float32.  Over a list of many thousands of entries (no top-k, top-p = 1)
    its running subtraction ``u -= p`` drifts by about 1e-4 and may stop a few entries off the exact place;
    ``precise=True`` does the same steps on the same float32 probabilities with float64 sums, which is what a
    sampler without that drift gives."""
    l = np.asarray(logits, dtype=np.float32).copy()
    vocab = l.shape[0]
    window = [] if repeat_last_n == 0 else list(previous[-repeat_last_n:])
    has_penalty = (repetition_penalty != 1.0 or frequency_penalty != 0.0 or presence_penalty != 0.0) and window
    if temperature < 1e-5 and not has_penalty:
        return int(np.argmax(l))                                   # :176-179
    if repetition_penalty not in (1.0, 0.0) and window:            # :199-213
        p = np.float32(repetition_penalty)
        for t in dict.fromkeys(window):
            if t < vocab:
                l[t] = l[t] / p if l[t] >= 0 else l[t] * p
    if (frequency_penalty != 0.0 or presence_penalty != 0.0) and window:   # :217-233
        counts = {}
        for t in window:
            if t < vocab:
                counts[t] = counts.get(t, 0) + 1
        for t, c in counts.items():
            l[t] -= np.float32(frequency_penalty) * np.float32(c)
            l[t] -= np.float32(presence_penalty)
    temp = np.float32(max(temperature, 1e-5))                      # :236-243
    l = l / temp
    e = np.exp(l - l.max())                                        # :246-253
    probs = (e / e.sum(dtype=np.float32)).astype(np.float32)
    acc = np.float64 if precise else np.float32
    if precise:
        probs = e.astype(np.float64) / e.astype(np.float64).sum()
    order = np.argsort(-probs, kind="stable")                      # :256-257
    if 0 < top_k < len(order):                                     # :260-262
        order = order[:top_k]
    if top_p < 1.0:                                                # :265-276
        cum, cutoff = acc(0), len(order)
        for i, t in enumerate(order):
            cum += probs[t]
            if cum >= acc(np.float32(top_p)):
                cutoff = i + 1
                break
        order = order[:cutoff]
    if min_p > 0.0 and len(order):                                 # :281-287
        thr = probs[order[0]] * acc(np.float32(min_p))
        keep = sum(1 for t in order if probs[t] >= thr)
        if keep > 0:
            order = order[:keep]
    total = acc(sum(probs[t] for t in order))                      # :290
    if total <= 0:
        return int(order[0]) if len(order) else 0
    u = acc(rand_f32(seed, len(previous)))                         # :328-338
    chosen = order[-1]
    for t in order:
        norm = probs[t] / total
        if u < norm:
            chosen = t
            break
        u -= norm
    return int(chosen)
