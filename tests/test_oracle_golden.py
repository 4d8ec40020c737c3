"""CPU: the NumPy/C oracle replayed against the fixtures the unmodified reference produced
(tests/golden/make_golden.py) and against the known-answer vectors in the reference's own tests."""
import ctypes
import os
import subprocess

import numpy as np
import pytest

import golden_inputs as G
from oracle import bitlinear_np as O

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def rel_err(a, b):
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    return float(np.max(np.abs(a - b)) / np.sqrt(np.mean(b ** 2)))


@pytest.fixture(scope="module")
def coracle():
    subprocess.check_call(["make", "-s", "-C", os.path.join(ROOT, "oracle"), "all"])
    lib = ctypes.CDLL(os.path.join(ROOT, "oracle", "_build", "liboracle_rotor.so"))
    return lib


def _p(a):
    return a.ctypes.data_as(ctypes.c_void_p)


# ---- known-answer vectors held by the reference's tests --------------------------------
def test_encode_decode_vector():
    # tests/test_core.py:23-32
    v = np.array([1, -1, 0, 1, -1, 0, 0, 1])
    plus, minus = O.encode(v)
    assert plus.tolist() == [1, 0, 0, 1, 0, 0, 0, 1]
    assert minus.tolist() == [0, 1, 0, 0, 1, 0, 0, 0]
    assert np.array_equal(O.decode(plus, minus), v)


def test_pack_roundtrip_vector():
    # tests/test_core.py:89-105
    v = np.array([1, -1, 0, 1, -1, 0, 1, 0])
    plus, minus = O.encode(v)
    packed = O.pack(plus, minus)
    assert len(packed) == 2
    up, um = O.unpack(packed, 8)
    assert np.array_equal(up, plus) and np.array_equal(um, minus)


def test_byte_0x12():
    # tests/debug_bitnet_format.py:19-44: 0x12 -> [+1, 0, -1, 0], planes 0x01 / 0x04
    packed = np.array([[0x12]], dtype=np.uint8)
    plus, minus = O.packed_to_planes(packed)
    assert plus[0, 0] == 0b00000001 and minus[0, 0] == 0b00000100
    assert O.packed_to_int8(packed)[0].tolist() == [1, 0, -1, 0]


def test_docstring_vectors():
    # src/rotor/bitnet.py:95, 238-240, 274-276: 0b00_10_01_00 <-> [0, -1, +1, 0]
    assert O.packed_to_int8(np.array([[0b00100100]], dtype=np.uint8))[0].tolist() == [0, -1, 1, 0]
    assert O.pack_ternary_matrix(np.array([[0, -1, 1, 0]], dtype=np.int8))[0, 0] == 0b00100100
    # src/rotor/bitnet.py:171-174: planes 0x01/0x04 -> 0b00_01_00_10
    w = O.planes_to_int8(np.array([[1]], np.uint8), np.array([[4]], np.uint8), 1, 4)
    assert O.pack_ternary_matrix(w)[0, 0] == 0b00010010


def test_reserved_code_reads_zero():
    # field 0b11: src/rotor/core.py:233-247 flags it, the converters decode it as 0
    assert O.packed_to_int8(np.array([[0xFF]], dtype=np.uint8))[0].tolist() == [0, 0, 0, 0]


def test_all_ones_layer():
    # tests/test_optimized_model.py:124-157 runs a 4x8 all-(+1) layer on ones; value must be 8*scale... rows sum
    w = np.ones((4, 8), dtype=np.int8)
    y = O.bitlinear_float(np.ones((1, 8), np.float32), w, 0.5)
    assert y.tolist() == [[4.0, 4.0, 4.0, 4.0]]


# ---- fixtures produced by the reference --------------------------------------------------
def test_format_fixture(golden_dir, coracle):
    z = np.load(os.path.join(golden_dir, "format.npz"))
    w = G.format_matrix()
    packed = O.pack_ternary_matrix(w)
    plus, minus = O.packed_to_planes(packed)
    assert np.array_equal(plus, z["plus"]) and np.array_equal(minus, z["minus"])
    assert np.array_equal(O.planes_to_int8(plus, minus, *w.shape), z["weights"])
    assert np.array_equal(O.packed_to_planes(z["raw_packed"])[0], z["raw_plus"])
    assert np.array_equal(O.packed_to_planes(z["raw_packed"])[1], z["raw_minus"])
    assert np.array_equal(O.packed_to_int8(z["raw_packed"]), z["raw_weights"])
    assert np.array_equal(O.pack(*O.encode(z["vec"])), z["vec_packed"])
    # the C restatement agrees too
    rows, cols = w.shape
    cp = np.zeros_like(plus)
    cm = np.zeros_like(minus)
    coracle.oracle_packed_to_planes(_p(packed), ctypes.c_size_t(rows), ctypes.c_size_t(cols), _p(cp), _p(cm))
    assert np.array_equal(cp, z["plus"]) and np.array_equal(cm, z["minus"])
    cw = np.zeros((rows, cols), dtype=np.int8)
    coracle.oracle_planes_to_int8(_p(cp), _p(cm), ctypes.c_size_t(rows), ctypes.c_size_t(cols), _p(cw))
    assert np.array_equal(cw, z["weights"])
    raw = np.ascontiguousarray(z["raw_packed"])
    rp = np.zeros_like(z["raw_plus"])
    rm = np.zeros_like(z["raw_minus"])
    coracle.oracle_packed_to_planes(_p(raw), ctypes.c_size_t(5), ctypes.c_size_t(36), _p(rp), _p(rm))
    assert np.array_equal(rp, z["raw_plus"]) and np.array_equal(rm, z["raw_minus"])


def test_c_pack_unpack(coracle):
    rng = np.random.default_rng(5)
    v = rng.integers(-1, 2, size=64).astype(np.int8)
    plus = np.zeros(64, np.uint8)
    minus = np.zeros(64, np.uint8)
    coracle.oracle_encode(_p(v), ctypes.c_size_t(64), _p(plus), _p(minus))
    assert np.array_equal(plus, O.encode(v)[0]) and np.array_equal(minus, O.encode(v)[1])
    packed = np.zeros(16, np.uint8)
    coracle.oracle_pack(_p(plus), _p(minus), ctypes.c_size_t(64), _p(packed))
    assert np.array_equal(packed, O.pack(plus, minus))
    up = np.zeros(64, np.uint8)
    um = np.zeros(64, np.uint8)
    coracle.oracle_unpack(_p(packed), ctypes.c_size_t(64), _p(up), _p(um))
    assert np.array_equal(up, plus) and np.array_equal(um, minus)
    back = np.zeros(64, np.int8)
    coracle.oracle_decode(_p(up), _p(um), ctypes.c_size_t(64), _p(back))
    assert np.array_equal(back, v)


def test_quantize_fixture(golden_dir):
    z = np.load(os.path.join(golden_dir, "quantize.npz"))
    q, s = O.quantize_rows(G.quant_inputs(), 1)
    assert np.array_equal(q[:, 0, :], z["q"]) and np.array_equal(s[:, 0], z["s"])
    assert s[2, 0] == 1.0 and not q[2].any()


def test_bitlinear_fixture(golden_dir, coracle):
    z = np.load(os.path.join(golden_dir, "bitlinear_2560x6912.npz"))
    w, scale, x1, x16 = G.bitlinear_case()
    assert np.array_equal(O.bitlinear_float(x1, w, scale), z["y1"])
    assert np.array_equal(O.bitlinear_float(x16, w, scale), z["y16"])
    y3, acc, q, s = O.bitlinear_int(x1, w, scale, 3)
    assert rel_err(y3, z["y1"]) < 1e-5          # 3-term int8 is float32-faithful
    y1, acc1, q1, _ = O.bitlinear_int(x1, w, scale, 1)
    assert 1e-3 < rel_err(y1, z["y1"]) < 1e-1   # single-term int8 is a different numeric contract
    # C integer accumulation agrees with the NumPy one
    cacc = np.zeros((1, 6912), np.int32)
    qc = np.ascontiguousarray(q1[:, 0, :])
    coracle.oracle_bitlinear_acc(_p(qc), ctypes.c_size_t(1), _p(np.ascontiguousarray(w)), ctypes.c_size_t(6912),
                                 ctypes.c_size_t(2560), _p(cacc))
    assert np.array_equal(cacc, acc1[:, 0, :])


def test_small_ragged_fixture(golden_dir):
    z = np.load(os.path.join(golden_dir, "bitlinear_small.npz"))
    w, scale, x = G.small_linear_case()
    assert np.array_equal(O.bitlinear_float(x, w, scale), z["y"])


def test_ffn_fixture(golden_dir):
    z = np.load(os.path.join(golden_dir, "ffn_block.npz"))
    lw, x1, x16 = G.ffn_case()
    for tag, x in (("m1", x1), ("m16", x16)):
        y = O.ffn(O.rmsnorm(x, lw["post_attn_norm"], 1e-6), lw, O.REFERENCE)
        assert rel_err(y, z[tag]) < 1e-6


@pytest.mark.parametrize("name", list(G.TINY_MODELS))
def test_model_fixture(golden_dir, name):
    z = np.load(os.path.join(golden_dir, f"model_{name}.npz"))
    om, prompt = G.tiny_model(name)
    logits, caches = O.model_forward(om, prompt[None, :], O.REFERENCE, use_cache=True)
    assert rel_err(logits[0], z["prompt_logits"]) < 1e-9
    assert rel_err(caches[-1]["k"], z["last_k"]) < 1e-9
    lc, _ = O.model_forward(om, prompt[None, :], O.with_semantics(O.REFERENCE, causal=True))
    assert rel_err(lc[0], z["prompt_logits_causal"]) < 1e-9
    ids = O.generate_greedy(om, prompt, G.N_NEW, O.REFERENCE)
    assert ids == z["greedy_ids"].tolist()


def test_backend_code_matvec():
    # the plug-in kernel's arithmetic (src/rotor/gpu_ternary.py:12-45) equals the CPU branch
    rng = np.random.default_rng(3)
    w = O.synth_ternary(rng, 24, 40)
    x = rng.standard_normal(40).astype(np.float32)
    scales = np.full(24, 0.37, np.float32)
    y = O.backend_matvec(O.backend_codes(w), scales, x, 40, 24)
    assert rel_err(y, O.bitlinear_float(x[None, :], w, 0.37)[0]) < 1e-5


@pytest.mark.skipif(not os.path.isdir(os.path.join(os.environ.get("ROTOR_RAG_REF", ""), "src", "rotor")),
                    reason="set ROTOR_RAG_REF to a checkout of the reference to run this")
def test_oracle_against_live_reference(tmp_path):
    """Where the reference checkout exists, re-run the generator: it asserts oracle == reference."""
    env = dict(os.environ)
    subprocess.check_call(["make", "-s", "-C", os.path.join(ROOT, "oracle"), "_ref"])
    out = subprocess.run(["python", os.path.join(ROOT, "tests", "golden", "make_golden.py"), "--check-only"],
                         env=env, capture_output=True, text=True)
    assert out.returncode == 0, out.stdout + out.stderr


def test_sampling_kept_sets_match_reference_fixture(golden_dir):
    """Top-k / top-p: the set the reference's strategies draw from and its probabilities
    (fixture taken from the reference's own code with np.random.choice stood in for)."""
    from oracle import sampling_np as S
    z = np.load(os.path.join(golden_dir, "sampling.npz"))
    logits = G.sampling_logits()
    for ci, (mode, k, p, temp) in enumerate(G.SAMPLING_CASES):
        idx, pr = S.kept_set(logits, mode, k, p, temp)
        assert np.array_equal(idx, z[f"idx{ci}"])
        assert np.max(np.abs(pr - z[f"p{ci}"])) < 1e-6
    # the draw: deterministic in (seed, counter), inside the kept set, k = 1 is the argmax
    assert S.sample(logits, 0, top_k=1) == int(np.argmax(logits))
    a = [S.sample(logits, 1, top_p=0.9, seed=5, counter=c) for c in range(50)]
    assert a == [S.sample(logits, 1, top_p=0.9, seed=5, counter=c) for c in range(50)]
    assert set(a) <= set(S.kept_set(logits, 1, top_p=0.9)[0].tolist()) and len(set(a)) > 5
