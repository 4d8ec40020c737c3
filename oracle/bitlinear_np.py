"""TEST INFRASTRUCTURE -- NumPy oracle for the ternary BitLinear decode path.

Only the test-suite, the smoke check and the CPU-baseline / reference leg of
the benchmark may import this module.  The product path never does: it fails
loudly when its CUDA library is missing.

Every function restates, in fresh functional code, what one piece of the
reference (BikerSam86/rotor-RAG) computes, with the reference path:line it
follows.  The restatement keeps NumPy's own dtype promotion, so under
NumPy >= 2 the data becomes float64 from the first attention onwards exactly
as it does in the reference (the score scaling divides a float32 array by a
float64 scalar).

Parity status: pinned.  ``tests/golden/make_golden.py`` imports the unmodified
reference, checks every function here against it on seeded inputs, and writes
the fixtures under ``tests/golden/`` that the CPU tests replay.

Two sets of semantics are expressed through :class:`Semantics`:

* ``REFERENCE`` -- what the reference code does when run: floating-point
  activations, ``gate * silu(clip(up, +-20))``, no positional encoding, no
  attention mask, eps 1e-6.
* ``BASELINE`` -- the published description of the BitNet-b1.58 path: per-token
  absmax int8 activations with exact int32 accumulation, ``relu(gate)^2 * up``,
  rotary embedding (theta 5e5), causal mask, eps 1e-5.  Each switch is a small
  patch of the reference flow and is documented where it applies.
"""
from __future__ import annotations

from dataclasses import dataclass, replace
from typing import Optional

import numpy as np


# --------------------------------------------------------------------------
# semantics switches
# --------------------------------------------------------------------------
@dataclass(frozen=True)
class Semantics:
    act_terms: int = 0            # 0: floating activations; n>=1: n-term int8 residual quantisation
    ffn_act: str = "silu_clip20"  # or "relu2"
    rope_theta: Optional[float] = None
    causal: bool = False
    eps: float = 1e-6
    # With int8 activations the glue between the products (norms, residual adds, LM head) is
    # float32, the dtype the embeddings arrive in.  glue64 runs that glue in float64 instead: a
    # second, equally valid evaluation of the same model, used by tests to find positions whose
    # logits hinge on a rounding tie of the quantiser (the two evaluations then disagree).
    glue64: bool = False


REFERENCE = Semantics()
BASELINE = Semantics(act_terms=1, ffn_act="relu2", rope_theta=500000.0, causal=True, eps=1e-5)


# --------------------------------------------------------------------------
# format: packed 2-bit <-> planes <-> int8      (vectorised NumPy)
# --------------------------------------------------------------------------
def encode(values):
    """flags (plus, minus) of ternary values; src/rotor/core.py:27-53."""
    v = np.asarray(values, dtype=np.int8)
    return (v == 1).astype(np.uint8), (v == -1).astype(np.uint8)


def decode(plus, minus):
    """value = plus - minus; src/rotor/core.py:56-72."""
    return plus.astype(np.int8) - minus.astype(np.int8)


def pack(plus, minus):
    """Four weights per byte, weight j of a byte in bits (2j+1, 2j) = (plus, minus);
    src/rotor/core.py:75-110."""
    plus = np.asarray(plus, dtype=np.uint8).reshape(-1, 4)
    minus = np.asarray(minus, dtype=np.uint8).reshape(-1, 4)
    sh = np.arange(4, dtype=np.uint8) * 2
    return (((plus << (sh + 1)) | (minus << sh)).sum(axis=1)).astype(np.uint8)


def unpack(packed, n):
    """Inverse of :func:`pack` for the first n weights; src/rotor/core.py:113-141."""
    packed = np.asarray(packed, dtype=np.uint8)[: (n + 3) // 4]
    fields = (packed[:, None] >> (np.arange(4, dtype=np.uint8) * 2)) & 3
    fields = fields.reshape(-1)[:n]
    return (fields >> 1).astype(np.uint8), (fields & 1).astype(np.uint8)


def pack_ternary_matrix(w):
    """int8 [out, in] in {-1,0,1} -> packed uint8 [out, in/4] (the on-disk layout that
    TernaryLinear.load_from_bitnet ingests; src/rotor/bitnet.py:263-300 restated
    without the per-element loop).  in must be a multiple of 4."""
    w = np.asarray(w, dtype=np.int8)
    out, inn = w.shape
    assert inn % 4 == 0
    field = np.where(w > 0, 2, np.where(w < 0, 1, 0)).astype(np.uint8).reshape(out, inn // 4, 4)
    sh = (np.arange(4, dtype=np.uint8) * 2)
    return (field << sh).sum(axis=2).astype(np.uint8)


def packed_fields(packed, cols=None):
    """uint8 [rows, cols/4] -> 2-bit fields [rows, cols]."""
    packed = np.asarray(packed, dtype=np.uint8)
    rows, nb = packed.shape
    cols = nb * 4 if cols is None else cols
    f = (packed[:, :, None] >> (np.arange(4, dtype=np.uint8) * 2)) & 3
    return f.reshape(rows, nb * 4)[:, :cols]


def packed_to_planes(packed, cols=None):
    """native/c/rotor_core.c:202-260 (bitnet_to_rotor): planes [rows, ceil(cols/8)],
    weight i at byte i//8 bit i%8; field 0b11 sets neither plane."""
    f = packed_fields(packed, cols)
    rows, cols = f.shape
    pad = (-cols) % 8
    plus = np.pad((f == 2).astype(np.uint8), ((0, 0), (0, pad)))
    minus = np.pad((f == 1).astype(np.uint8), ((0, 0), (0, pad)))
    return (np.packbits(plus, axis=1, bitorder="little"),
            np.packbits(minus, axis=1, bitorder="little"))


def planes_to_int8(plus, minus, rows, cols):
    """native/c/rotor_core.c:270-299 (rotor_unpack_weights)."""
    p = np.unpackbits(np.asarray(plus, np.uint8).reshape(rows, -1), axis=1, bitorder="little")[:, :cols]
    m = np.unpackbits(np.asarray(minus, np.uint8).reshape(rows, -1), axis=1, bitorder="little")[:, :cols]
    return p.astype(np.int8) - m.astype(np.int8)


def packed_to_int8(packed, cols=None):
    """The load path of TernaryLinear.load_from_bitnet (src/rotor/transformer.py:77-109):
    packed -> planes -> dense int8 cache."""
    packed = np.asarray(packed, dtype=np.uint8)
    cols = packed.shape[1] * 4 if cols is None else cols
    plus, minus = packed_to_planes(packed, cols)
    return planes_to_int8(plus, minus, packed.shape[0], cols)


def backend_codes(w):
    """The plug-in backend's own packing, code = w + 1 over the flattened matrix, four
    per byte LSB first; src/rotor/gpu_ternary.py:112-136."""
    flat = (np.asarray(w).astype(np.int16) + 1).astype(np.uint8).reshape(-1)
    pad = (-flat.size) % 4
    flat = np.pad(flat, (0, pad)).reshape(-1, 4)
    return (flat << (np.arange(4, dtype=np.uint8) * 2)).sum(axis=1).astype(np.uint8)


# --------------------------------------------------------------------------
# activation quantiser
# --------------------------------------------------------------------------
def quantize_tensor(x):
    """src/rotor/quantization.py:137-149, symmetric 8-bit, one scale for the whole
    array: s = max|x|/127 (1.0 when all zero), q = clip(round_half_even(x/s), -128, 127)."""
    max_val = np.max(np.abs(x))
    scale = max_val / 127 if max_val > 0 else 1.0
    q = np.clip(np.round(x / scale), -128, 127).astype(np.int8)
    return q, scale


def quantize_rows(x, terms=1):
    """The same quantiser applied to each token row, repeated ``terms`` times on the
    residual left by the previous term (term 1 alone is the published per-token absmax
    int8).  x: float32 [M, K].  Returns q int8 [M, terms, K], s float32 [M, terms].
    All arithmetic in float32 with one rounding per operation."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    m, k = x.shape
    q = np.zeros((m, terms, k), dtype=np.int8)
    s = np.ones((m, terms), dtype=np.float32)
    for r in range(m):
        resid = x[r].copy()
        for t in range(terms):
            qt, st = quantize_tensor(resid)
            st = np.float32(st)
            q[r, t] = qt
            s[r, t] = st
            resid = (resid - (qt.astype(np.float32) * st).astype(np.float32)).astype(np.float32)
    return q, s


# --------------------------------------------------------------------------
# BitLinear
# --------------------------------------------------------------------------
def bitlinear_float(x, w_int8, scale):
    """TernaryLinear.forward CPU branch, src/rotor/transformer.py:111-155:
    flatten leading dims, np.dot(x, W.T) * scale, restore shape."""
    lead = x.shape[:-1]
    flat = x.reshape(-1, x.shape[-1])
    y = np.dot(flat, w_int8.T) * scale
    return y.reshape(*lead, w_int8.shape[0])


def int_matmul(q, w_int8):
    """acc[m, t, o] = sum_k q[m, t, k] * w[o, k], exact int32.  Every partial sum is an integer of
    magnitude at most 128 * K; below 2^24 all of them are exact in float32 whatever the summation
    order, so the product can go through BLAS.  Wider layers take the integer einsum."""
    m, terms, k = q.shape
    if 128 * k < (1 << 24):
        accf = q.reshape(m * terms, k).astype(np.float32) @ w_int8.astype(np.float32).T
        return accf.astype(np.int32).reshape(m, terms, w_int8.shape[0])
    return np.einsum("mtk,ok->mto", q.astype(np.int32), w_int8.astype(np.int32), optimize=True).astype(np.int32)


def bitlinear_int(x, w_int8, scale, terms=1):
    """Quantised BitLinear: per-row n-term int8 activations, exact int32 accumulation
    against the cached int8 weights, then y = (sum_t s_t * acc_t) * scale in float32.
    Returns (y float32 [..., out], acc int32 [M, terms, out], q, s)."""
    lead = x.shape[:-1]
    flat = np.ascontiguousarray(x.reshape(-1, x.shape[-1]), dtype=np.float32)
    q, s = quantize_rows(flat, terms)
    acc = int_matmul(q, w_int8)
    y = np.zeros((flat.shape[0], w_int8.shape[0]), dtype=np.float32)
    for t in range(terms):
        y = (y + acc[:, t, :].astype(np.float32) * s[:, t:t + 1]).astype(np.float32)
    y = (y * np.float32(scale)).astype(np.float32)
    return y.reshape(*lead, w_int8.shape[0]), acc, q, s


def bitlinear(x, w_int8, scale, sem: Semantics):
    if sem.act_terms == 0:
        return bitlinear_float(x, w_int8, scale)
    return bitlinear_int(x, w_int8, scale, sem.act_terms)[0]


def backend_matvec(codes, scales, x, in_dim, out_dim):
    """Arithmetic of the plug-in kernel, src/rotor/gpu_ternary.py:12-45:
    out[r] = scales[r] * sum_i x[i] * (code(r*in+i) - 1)."""
    fields = (codes[:, None] >> (np.arange(4, dtype=np.uint8) * 2)) & 3
    w = fields.reshape(-1)[: in_dim * out_dim].astype(np.float32).reshape(out_dim, in_dim) - 1.0
    return (w @ x.astype(np.float32)) * scales.astype(np.float32)


# --------------------------------------------------------------------------
# transformer pieces
# --------------------------------------------------------------------------
def rmsnorm(x, weight, eps):
    """RMSNorm.forward, src/rotor/transformer.py:24-36."""
    norm = np.sqrt(np.mean(x ** 2, axis=-1, keepdims=True) + eps)
    return (x / norm) * weight


def silu_clip20(x):
    """GatedFFN._silu, src/rotor/transformer.py:343-351."""
    c = np.clip(x, -20, 20)
    return c / (1 + np.exp(-c))


def softmax(x, axis=-1):
    """MultiHeadAttention._softmax, src/rotor/transformer.py:294-298."""
    e = np.exp(x - np.max(x, axis=axis, keepdims=True))
    return e / np.sum(e, axis=axis, keepdims=True)


def rope(x, first_pos, theta):
    """Rotary embedding (half-split pairing: element i rotates with element i + D/2 by
    angle pos * theta^(-2i/D)).  The reference applies no positional encoding
    (src/rotor/transformer.py:234-247); this is the BASELINE switch.
    x: [B, H, S, D]; positions first_pos .. first_pos + S - 1."""
    d = x.shape[-1]
    half = d // 2
    inv = theta ** (-np.arange(half, dtype=np.float64) * 2.0 / d)
    ang = (first_pos + np.arange(x.shape[2], dtype=np.float64))[:, None] * inv[None, :]
    c, s = np.cos(ang), np.sin(ang)
    a, b = x[..., :half], x[..., half:]
    return np.concatenate([a * c - b * s, b * c + a * s], axis=-1)


def causal_mask(s, t):
    """Additive mask for s new queries over t total keys."""
    return np.triu(np.full((s, t), -np.inf), k=t - s + 1)


def ffn(x, lw, sem: Semantics):
    """GatedFFN.forward, src/rotor/transformer.py:320-341: gate, up, gating, sub-norm
    over d_ff, down."""
    gate = bitlinear(x, *lw["gate"], sem)
    up = bitlinear(x, *lw["up"], sem)
    if sem.ffn_act == "silu_clip20":
        gated = gate * silu_clip20(up)
    else:
        gated = np.maximum(gate, 0) ** 2 * up
    gated = rmsnorm(gated, lw["ffn_sub_norm"], sem.eps)
    return bitlinear(gated, *lw["down"], sem)


def attention(x, lw, cfg, sem: Semantics, kv_cache=None, use_cache=False):
    """MultiHeadAttention.forward, src/rotor/transformer.py:206-292.  x: [B, S, d].
    The sub-norm is applied after the output projection, as the reference does."""
    b, s, _ = x.shape
    h, hk = cfg["n_heads"], cfg["n_kv_heads"]
    d = cfg["d_model"] // h
    q = bitlinear(x, *lw["q"], sem).reshape(b, s, h, d).transpose(0, 2, 1, 3)
    k = bitlinear(x, *lw["k"], sem).reshape(b, s, hk, d).transpose(0, 2, 1, 3)
    v = bitlinear(x, *lw["v"], sem).reshape(b, s, hk, d).transpose(0, 2, 1, 3)
    past = 0 if kv_cache is None else kv_cache["k"].shape[2]
    if sem.rope_theta is not None:
        q = rope(q, past, sem.rope_theta)
        k = rope(k, past, sem.rope_theta)
    if kv_cache is not None:
        k = np.concatenate([kv_cache["k"], k], axis=2)
        v = np.concatenate([kv_cache["v"], v], axis=2)
    new_cache = {"k": k, "v": v} if use_cache else None
    if hk < h:
        k = np.repeat(k, h // hk, axis=1)
        v = np.repeat(v, h // hk, axis=1)
    scores = np.matmul(q, k.transpose(0, 1, 3, 2)) / np.sqrt(d)
    if sem.causal:
        scores = scores + causal_mask(s, k.shape[2])
    out = np.matmul(softmax(scores), v).transpose(0, 2, 1, 3).reshape(b, s, h * d)
    out = bitlinear(out, *lw["o"], sem)
    return rmsnorm(out, lw["attn_sub_norm"], sem.eps), new_cache


def block(x, lw, cfg, sem: Semantics, kv_cache=None, use_cache=False):
    """TransformerBlock.forward, src/rotor/transformer.py:383-413."""
    a, new_cache = attention(rmsnorm(x, lw["input_norm"], sem.eps), lw, cfg, sem, kv_cache, use_cache)
    x = x + a
    x = x + ffn(rmsnorm(x, lw["post_attn_norm"], sem.eps), lw, sem)
    return x, new_cache


def model_forward(model, input_ids, sem: Semantics = REFERENCE, past_kv_cache=None,
                  use_cache=False, return_logits=True):
    """BitNetModel.forward, src/rotor/bitnet_model.py:190-244: embedding gather, the
    blocks with a per-layer cache list, final norm, tied LM head over every position."""
    ids = np.asarray(input_ids)
    squeeze = ids.ndim == 1
    if squeeze:
        ids = ids[None, :]
    hcur = model["embed"][ids]
    if sem.glue64:
        hcur = hcur.astype(np.float64)
    caches = [] if use_cache else None
    for li, lw in enumerate(model["layers"]):
        past = None if past_kv_cache is None else past_kv_cache[li]
        hcur, c = block(hcur, lw, model["cfg"], sem, past, use_cache)
        if use_cache:
            caches.append(c)
    hcur = rmsnorm(hcur, model["norm"], sem.eps)
    out = np.dot(hcur, model["embed"].T) if return_logits else hcur
    return (out[0] if squeeze else out), caches


def greedy(logits):
    """GreedySampling.sample, src/rotor/generation.py:31-42 (lowest index on ties)."""
    return int(np.argmax(logits))


def generate_greedy(model, prompt_ids, n_new, sem: Semantics = REFERENCE, return_logits=False):
    """The cached loop of TextGenerator.generate, src/rotor/generation.py:179-279:
    one forward over the whole prompt, then one-token forwards that hand the cache back."""
    ids = [int(t) for t in prompt_ids]
    cache = None
    steps = []
    for step in range(n_new):
        feed = np.asarray(ids if step == 0 else ids[-1:], dtype=np.int64).reshape(1, -1)
        logits, cache = model_forward(model, feed, sem, past_kv_cache=cache, use_cache=True)
        last = logits[0, -1, :]
        if return_logits:
            steps.append(np.asarray(last))
        ids.append(greedy(last))
    return (ids, steps) if return_logits else ids


# --------------------------------------------------------------------------
# seeded synthetic parameters (shared by tests, smoke and the CPU baseline)
# --------------------------------------------------------------------------
def bf16_round(a):
    """Round float32 to the nearest bfloat16 (ties to even), returned as float32."""
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    u = (u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000
    return u.astype(np.uint32).view(np.float32)


def synth_ternary(rng, out, inn):
    """i.i.d. ternary weights, P = 1/3 each."""
    return rng.integers(-1, 2, size=(out, inn), dtype=np.int8)


SYNTH_SCALE = np.float32(0.015955)  # mean |N(0, 0.02)|


def synth_model(cfg, seed, random_norms=True, fast_embed=False):
    """Random-init model of the BitNet-b1.58 layout: ternary projections uniform over
    {-1,0,+1}, one float32 scale per matrix, bf16-representable N(0, 0.02) embeddings
    (tied LM head), norm weights near one."""
    rng = np.random.default_rng(seed)
    d, ff = cfg["d_model"], cfg["d_ff"]
    hd = d // cfg["n_heads"]
    dq, dkv = cfg["n_heads"] * hd, cfg["n_kv_heads"] * hd

    def norm_w(n):
        if not random_norms:
            return np.ones(n, dtype=np.float32)
        return bf16_round(1.0 + 0.1 * rng.standard_normal(n).astype(np.float32))

    def lin(o, i):
        w = synth_ternary(rng, o, i)
        sc = float(SYNTH_SCALE * np.float32(1.0 + 0.25 * rng.random()))
        return w, float(np.float32(sc))

    layers = []
    for _ in range(cfg["n_layers"]):
        layers.append({
            "input_norm": norm_w(d), "post_attn_norm": norm_w(d),
            "attn_sub_norm": norm_w(d), "ffn_sub_norm": norm_w(ff),
            "q": lin(dq, d), "k": lin(dkv, d), "v": lin(dkv, d), "o": lin(d, dq),
            "gate": lin(ff, d), "up": lin(ff, d), "down": lin(d, ff),
        })
    if fast_embed:
        # timing-only variant for full-size tables: float32 draws, bf16 by truncation, in place
        embed = rng.standard_normal((cfg["vocab_size"], d), dtype=np.float32)
        embed *= np.float32(0.02)
        embed.view(np.uint32)[...] &= np.uint32(0xFFFF0000)
    else:
        embed = bf16_round((0.02 * rng.standard_normal((cfg["vocab_size"], d))).astype(np.float32))
    return {"cfg": dict(cfg), "embed": embed, "norm": norm_w(d), "layers": layers}


def with_semantics(sem: Semantics, **kw) -> Semantics:
    return replace(sem, **kw)
