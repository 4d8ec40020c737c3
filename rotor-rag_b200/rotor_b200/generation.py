"""Sampling strategies and the generation loop, mirroring ``src/rotor/generation.py``
(GreedySampling :28-42, TopKSampling :45-88, TopPSampling :91-145, TextGenerator :148-340).

With a rotor_b200 BitNetModel, greedy generation with the cache stays on the device:
the prompt is prefilled once, every later step is a replay of one CUDA graph whose
greedy pick feeds the next step, and token ids come back to the host only to test for
EOS and to feed the per-token callback.  Top-k / top-p strategies keep the logits on the
device as well and draw there (rotor_b200_sample: the reference's distribution from a seeded
counter-based stream instead of NumPy's global generator); only the drawn token id comes
back.  That is the default whenever the model can do it; a strategy built with
``device=False`` (or ``use_cache=False``) sends the logits of the last position to the host
each step and samples them with the reference's NumPy procedure, drawing from NumPy's global
stream as the reference does.
"""
from __future__ import annotations

from typing import Callable, Optional

import numpy as np


class SamplingStrategy:
    def sample(self, logits: np.ndarray, temperature: float = 1.0) -> int:
        raise NotImplementedError


class GreedySampling(SamplingStrategy):
    """argmax, lowest index on ties; temperature ignored (reference :31-42)."""

    def sample(self, logits: np.ndarray, temperature: float = 1.0) -> int:
        return int(np.argmax(logits))


def _softmax(x: np.ndarray) -> np.ndarray:
    e = np.exp(x - np.max(x))
    return e / np.sum(e)


class _DeviceDraw:
    """Device-side draw shared by the top-k / top-p strategies (``device=True``)."""
    mode = 0
    k, p = 50, 0.9

    def _init_device(self, device, seed):
        self.device = None if device is None else bool(device)  # None: on the device when the model can
        self.seed = int(np.random.randint(0, 2 ** 31 - 1)) if seed is None else int(seed)
        self.counter = 0

    def sample_device(self, logits, temperature: float = 1.0):
        """logits: CUDA float32 [rows, vocab]; returns a CUDA int64 tensor [rows] and advances the stream."""
        from . import ops
        out = ops.sample(logits, self.mode, top_k=self.k, top_p=self.p, temperature=temperature, seed=self.seed,
                         counter=self.counter)
        self.counter += logits.shape[0]
        return out


class TopKSampling(SamplingStrategy, _DeviceDraw):
    """Sample among the k largest logits (reference :45-88).  ``device=False``: draw on the host from
    NumPy's global stream (the reference's behaviour) instead of on the GPU."""
    mode = 0

    def __init__(self, k: int = 50, *, device: Optional[bool] = None, seed: Optional[int] = None):
        self.k = k
        self._init_device(device, seed)

    def sample(self, logits: np.ndarray, temperature: float = 1.0) -> int:
        if temperature != 1.0:
            logits = logits / temperature
        top = np.argpartition(logits, -self.k)[-self.k:]
        probs = _softmax(logits[top])
        return int(top[np.random.choice(len(top), p=probs)])


class TopPSampling(SamplingStrategy, _DeviceDraw):
    """Sample from the smallest set whose probability mass reaches p (reference :91-145).
    ``device=False``: draw on the host from NumPy's global stream instead of on the GPU."""
    mode = 1

    def __init__(self, p: float = 0.9, *, device: Optional[bool] = None, seed: Optional[int] = None):
        self.p = p
        self._init_device(device, seed)

    def sample(self, logits: np.ndarray, temperature: float = 1.0) -> int:
        if temperature != 1.0:
            logits = logits / temperature
        probs = _softmax(logits)
        order = np.argsort(probs)[::-1]
        sorted_probs = probs[order]
        size = np.searchsorted(np.cumsum(sorted_probs), self.p) + 1
        nucleus = sorted_probs[:size] / np.sum(sorted_probs[:size])
        return int(order[:size][np.random.choice(size, p=nucleus)])


NucleusSampling = TopPSampling


class TextGenerator:
    """Reference :148-340.  ``max_length`` bounds prompt + new tokens (:210); the EOS token
    is not appended (:228-229); the callback receives each new token's text (:236-238)."""

    def __init__(self, model, tokenizer, sampling_strategy: Optional[SamplingStrategy] = None,
                 temperature: float = 1.0, max_length: int = 100, use_cache: bool = True,
                 readback_chunk: int = 1):
        self.model = model
        self.tokenizer = tokenizer
        self.sampling_strategy = sampling_strategy or GreedySampling()
        self.temperature = temperature
        self.max_length = max_length
        self.use_cache = use_cache
        self.kv_cache = None
        # how many device-resident steps run between two looks at the tokens on the host;
        # 1 reproduces the reference's per-token EOS test and callback timing exactly
        self.readback_chunk = readback_chunk

    # ------------------------------------------------------------------------------------
    def _device_resident(self):
        return (self.use_cache and type(self.sampling_strategy) is GreedySampling
                and hasattr(self.model, "greedy_chunks"))

    def _plan(self, prompt, max_new_tokens, temperature):
        max_new_tokens = max_new_tokens or self.max_length
        temperature = temperature if temperature is not None else self.temperature
        token_ids = self.tokenizer.encode(prompt, add_special_tokens=True, return_numpy=True)
        ids = [int(t) for t in np.asarray(token_ids).tolist()]
        n = min(max_new_tokens, self.max_length - len(ids))
        return ids, n, temperature

    def _tokens(self, ids, n, temperature, stop_on_eos):
        """Yields new token ids one by one; stops before an EOS token."""
        eos = getattr(self.tokenizer, "eos_token_id", None)
        if self._device_resident():
            for new in self.model.greedy_chunks(ids, n, use_graph=True, chunk=self.readback_chunk):
                for tok in new:
                    if stop_on_eos and eos is not None and tok == eos:
                        return
                    yield tok
            return
        self.kv_cache = None
        seq = list(ids)
        on_device = isinstance(self.sampling_strategy, _DeviceDraw) and self.sampling_strategy.device is not False
        if self.use_cache and on_device and hasattr(self.model, "forward_last_logits_device"):
            # logits stay on the device; one token id per step comes back
            for step in range(n):
                feed = np.asarray(seq if step == 0 else seq[-1:], dtype=np.int64).reshape(1, -1)
                logits, self.kv_cache = self.model.forward_last_logits_device(feed, self.kv_cache)
                tok = int(self.sampling_strategy.sample_device(logits, temperature).cpu()[0])
                if stop_on_eos and eos is not None and tok == eos:
                    return
                seq.append(tok)
                yield tok
            return
        for step in range(n):
            logits = self._get_next_token_logits(np.asarray(seq, dtype=np.int64), is_first_step=(step == 0))
            tok = self.sampling_strategy.sample(logits, temperature)
            if stop_on_eos and eos is not None and tok == eos:
                return
            seq.append(tok)
            yield tok

    def _get_next_token_logits(self, token_ids: np.ndarray, is_first_step: bool = False) -> np.ndarray:
        """Reference :244-279, asking the model for the last position only."""
        kw = {"logits_positions": "last"} if hasattr(self.model, "greedy_chunks") else {}
        if self.use_cache:
            if is_first_step:
                logits, self.kv_cache = self.model.forward(token_ids.reshape(1, -1), use_cache=True, **kw)
            else:
                logits, self.kv_cache = self.model.forward(token_ids[-1:].reshape(1, -1),
                                                           past_kv_cache=self.kv_cache, use_cache=True, **kw)
        else:
            logits, _ = self.model.forward(token_ids.reshape(1, -1), use_cache=False, **kw)
        return logits[0, -1, :]

    # ------------------------------------------------------------------------------------
    def generate(self, prompt: str, max_new_tokens: Optional[int] = None, temperature: Optional[float] = None,
                 stop_on_eos: bool = True, callback: Optional[Callable[[str], None]] = None) -> str:
        ids, n, temperature = self._plan(prompt, max_new_tokens, temperature)
        if n <= 0:
            return self.tokenizer.decode(np.asarray(ids, dtype=np.int64), skip_special_tokens=True)
        for tok in self._tokens(list(ids), n, temperature, stop_on_eos):
            ids.append(tok)
            if callback:
                callback(self.tokenizer.decode([tok], skip_special_tokens=True))
        return self.tokenizer.decode(np.asarray(ids, dtype=np.int64), skip_special_tokens=True)

    def generate_streaming(self, prompt: str, max_new_tokens: Optional[int] = None,
                           temperature: Optional[float] = None, stop_on_eos: bool = True):
        """Reference :281-340: yields the prompt, then each new token's text."""
        ids, n, temperature = self._plan(prompt, max_new_tokens, temperature)
        yield prompt
        if n <= 0:
            return
        for tok in self._tokens(list(ids), n, temperature, stop_on_eos):
            yield self.tokenizer.decode([tok], skip_special_tokens=True)
