"""TEST INFRASTRUCTURE: NumPy restatement of the reference's top-k / top-p sampling.

``kept_set`` follows TopKSampling.sample (src/rotor/generation.py:57-80) and
TopPSampling.sample (:104-137) up to the draw: temperature, the kept token set and its
probabilities.  The reference then draws with ``np.random.choice`` from NumPy's global
generator; the device sampler cannot follow that stream, so ``sample`` states the draw the
CUDA kernel makes instead: a uniform from SplitMix64(seed, counter) and an inverse-CDF
lookup over the kept tokens in vocabulary order.  Same distribution, a different (and
documented) mapping from random bits to tokens.

Only ``tests/`` may import this module.
"""
import numpy as np

MASK64 = (1 << 64) - 1


def splitmix64(x):
    x = (x + 0x9E3779B97F4A7C15) & MASK64
    x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & MASK64
    x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & MASK64
    return x ^ (x >> 31)


def uniform(seed, counter, row=0):
    """[0, 1) with 24 random bits, as the kernel derives it."""
    r = splitmix64(seed ^ splitmix64((counter + row) & MASK64))
    return np.float32(r >> 40) * np.float32(1.0 / 16777216.0)


def kept_set(logits, mode, top_k=50, top_p=0.9, temperature=1.0):
    """(token ids ascending, probabilities float64 summing to 1) of the set the reference samples from.
    mode 0: the k largest logits; mode 1: the shortest probability-sorted prefix whose mass reaches p."""
    x = np.asarray(logits, dtype=np.float32)
    if temperature != 1.0:
        x = x / np.float32(temperature)
    if mode == 0:
        k = min(top_k, x.size)
        idx = np.argpartition(x, -k)[-k:]
        e = np.exp((x[idx] - np.max(x[idx])).astype(np.float64))
        pr = e / e.sum()
    else:
        e = np.exp((x - np.max(x)).astype(np.float64))
        probs = e / e.sum()
        order = np.argsort(probs)[::-1]
        sp = probs[order]
        size = int(np.searchsorted(np.cumsum(sp), top_p) + 1)
        size = min(size, x.size)
        idx = order[:size]
        pr = sp[:size] / sp[:size].sum()
    o = np.argsort(idx)
    return idx[o].astype(np.int64), pr[o]


def sample(logits, mode, top_k=50, top_p=0.9, temperature=1.0, seed=0, counter=0, row=0):
    """The token the device sampler draws (up to float rounding at set and CDF boundaries)."""
    idx, pr = kept_set(logits, mode, top_k, top_p, temperature)
    u = float(uniform(seed, counter, row))
    cdf = np.cumsum(pr)
    j = int(np.searchsorted(cdf, u * cdf[-1], side="right"))
    return int(idx[min(j, len(idx) - 1)])
