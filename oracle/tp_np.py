"""TEST INFRASTRUCTURE: NumPy restatement of the tensor-parallel split of the BitNet block.

The reference (BikerSam86/rotor-RAG) is single-device; there is no reference code for this
file to follow.  It restates, rank by rank, the split the CUDA library implements, so that
(a) the split itself can be checked against the single-device oracle
(``bitlinear_np.model_forward`` with one activation term) on CPU ranks, and (b) the GPU
ranks have a per-rank checker.  Collectives come in as callbacks:

    allreduce(array, op)   op in {"sum", "max"}; returns the reduced array on every rank

Only ``tests/`` may import this module.
"""
import numpy as np

from . import bitlinear_np as o


def quantize_rows_shared(x, row_absmax):
    """One-term absmax int8 quantiser with the row maximum given from outside (the global
    maximum over all ranks' slices of the row).  Same arithmetic as
    ``bitlinear_np.quantize_tensor`` per row."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    s = np.where(row_absmax > 0, row_absmax / np.float32(127), np.float32(1.0)).astype(np.float32)
    q = np.clip(np.round(x / s[:, None]), -128, 127).astype(np.int8)
    return q, s


def column_parallel(x, w, scale):
    """Rows of the weight matrix live here, the input row is whole: plain one-term BitLinear."""
    return o.bitlinear_int(x, w, scale, 1)[0]


def row_parallel(x_local, w_local, scale, allreduce):
    """Columns of the weight matrix live here, with the matching slice of the input row."""
    flat = np.ascontiguousarray(x_local.reshape(-1, x_local.shape[-1]), dtype=np.float32)
    amax = allreduce(np.max(np.abs(flat), axis=1).astype(np.float32), "max")
    q, s = quantize_rows_shared(flat, amax)
    acc = (q.astype(np.int32) @ w_local.astype(np.int32).T).astype(np.int32)
    acc = allreduce(acc, "sum")
    y = (acc.astype(np.float32) * s[:, None]).astype(np.float32)
    y = (y * np.float32(scale)).astype(np.float32)
    return y.reshape(*x_local.shape[:-1], w_local.shape[0])


def block_tp(x, sh, cfg, ld, sem, allreduce, kv_cache=None):
    """One block on one rank.  ``sh``: this rank's shard (rotor_b200.tensor_parallel.shard_layer),
    ``ld``: its local dimensions.  x: [B, S, d] (replicated).  Returns (x, cache)."""
    b, s, _ = x.shape
    h, hk, d = ld["n_heads"], ld["n_kv_heads"], ld["head_dim"]
    xn = o.rmsnorm(x, sh["input_norm"], sem.eps)
    q = column_parallel(xn, *sh["q"]).reshape(b, s, h, d).transpose(0, 2, 1, 3)
    k = column_parallel(xn, *sh["k"]).reshape(b, s, hk, d).transpose(0, 2, 1, 3)
    v = column_parallel(xn, *sh["v"]).reshape(b, s, hk, d).transpose(0, 2, 1, 3)
    past = 0 if kv_cache is None else kv_cache["k"].shape[2]
    if sem.rope_theta is not None:
        q = o.rope(q, past, sem.rope_theta)
        k = o.rope(k, past, sem.rope_theta)
    if kv_cache is not None:
        k = np.concatenate([kv_cache["k"], k], axis=2)
        v = np.concatenate([kv_cache["v"], v], axis=2)
    cache = {"k": k, "v": v}
    kk, vv = np.repeat(k, h // hk, axis=1), np.repeat(v, h // hk, axis=1)
    scores = np.matmul(q, kk.transpose(0, 1, 3, 2)) / np.sqrt(d)
    if sem.causal:
        scores = scores + o.causal_mask(s, kk.shape[2])
    att = np.matmul(o.softmax(scores), vv).transpose(0, 2, 1, 3).reshape(b, s, h * d)
    a = row_parallel(att.astype(np.float32), *sh["o"], allreduce)
    x = x + o.rmsnorm(a, sh["attn_sub_norm"], sem.eps)

    xn = o.rmsnorm(x, sh["post_attn_norm"], sem.eps)
    gate = column_parallel(xn, *sh["gate"])
    up = column_parallel(xn, *sh["up"])
    gated = gate * o.silu_clip20(up) if sem.ffn_act == "silu_clip20" else np.maximum(gate, 0) ** 2 * up
    gated = gated.astype(np.float32)
    ss = allreduce(np.sum(gated.astype(np.float32) ** 2, axis=-1).astype(np.float32), "sum")
    norm = np.sqrt(ss / np.float32(cfg["d_ff"]) + np.float32(sem.eps))[..., None]
    gated = ((gated / norm) * sh["ffn_sub_norm"]).astype(np.float32)
    x = x + row_parallel(gated, *sh["down"], allreduce)
    return x, cache


def model_forward_tp(model, shards, ld, rank, ids, sem, allreduce, caches=None):
    """Whole model on one rank.  Returns (logits of this rank's vocabulary slice
    [B, S, V/size], caches)."""
    ids = np.asarray(ids)
    if ids.ndim == 1:
        ids = ids[None, :]
    x = model["embed"][ids]
    new = []
    for li, sh in enumerate(shards):
        x, c = block_tp(x, sh, model["cfg"], ld, sem, allreduce, None if caches is None else caches[li])
        new.append(c)
    x = o.rmsnorm(x, model["norm"], sem.eps)
    vl = ld["vocab"]
    return np.dot(x, model["embed"][rank * vl:(rank + 1) * vl].T), new


def pick_tp(local_logits_row, rank, vl, allgather):
    """Greedy pick over vocabulary slices: best (value, global index) of every rank, then the
    highest value, lowest index on ties."""
    i = int(np.argmax(local_logits_row))
    pairs = allgather((float(np.float32(local_logits_row[i])), rank * vl + i))
    best = max(pairs, key=lambda p: (p[0], -p[1]))
    return best[1]
