"""Test helper: writes a small GGUF v3 file (metadata of every scalar kind, a string array, one
F32, one F16 and two ternary tensors in the 2-bit packed format) from seeded data."""
import struct

import numpy as np

from oracle import bitlinear_np as O

TQ1_0, TQ2_0, F32, F16 = 30, 31, 0, 1


def _s(text):
    b = text.encode("utf-8")
    return struct.pack("<Q", len(b)) + b


def synthetic_tensors(seed=321):
    rng = np.random.default_rng(seed)
    w_a = O.synth_ternary(rng, 48, 128)
    w_b = O.synth_ternary(rng, 32, 64)
    return {
        "blk.0.attn_q.weight": (TQ2_0, [48, 128], O.pack_ternary_matrix(w_a), w_a),
        "blk.0.ffn_up.weight": (TQ1_0, [32, 64], O.pack_ternary_matrix(w_b), w_b),
        "token_embd.weight": (F32, [10, 16], rng.standard_normal((10, 16)).astype(np.float32), None),
        "output_norm.weight": (F16, [16], rng.standard_normal(16).astype(np.float16), None),
    }


def write_gguf(path, seed=321):
    tensors = synthetic_tensors(seed)
    meta = [("general.architecture", 8, "bitnet"), ("general.alignment", 4, 32), ("bitnet.block_count", 4, 1),
            ("bitnet.rope.freq_base", 6, 500000.0), ("general.file_type", 5, -3), ("flag", 7, True),
            ("tiny", 0, 7), ("neg8", 1, -7), ("u16", 2, 65000), ("i16", 3, -1234), ("u64", 10, 1 << 40),
            ("i64", 11, -(1 << 40)), ("f64", 12, 2.5)]
    fmt = {0: "<B", 1: "<b", 2: "<H", 3: "<h", 4: "<I", 5: "<i", 6: "<f", 7: "<?", 10: "<Q", 11: "<q", 12: "<d"}
    out = b"GGUF" + struct.pack("<IQQ", 3, len(tensors), len(meta) + 1)
    for key, vt, val in meta:
        out += _s(key) + struct.pack("<I", vt) + (_s(val) if vt == 8 else struct.pack(fmt[vt], val))
    toks = ["<s>", "</s>", "hello"]
    out += _s("tokenizer.ggml.tokens") + struct.pack("<IIQ", 9, 8, len(toks)) + b"".join(_s(t) for t in toks)
    blobs, offset = [], 0
    for name, (tt, dims, data, _) in tensors.items():
        raw = np.ascontiguousarray(data).tobytes()
        out += _s(name) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims)
        out += struct.pack("<IQ", tt, offset)
        blobs.append((offset, raw))
        offset += -(-len(raw) // 32) * 32
    out += b"\0" * (-len(out) % 32)
    body = bytearray(offset)
    for off, raw in blobs:
        body[off:off + len(raw)] = raw
    with open(path, "wb") as f:
        f.write(out + bytes(body))
    return tensors
