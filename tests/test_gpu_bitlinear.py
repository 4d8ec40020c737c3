"""GPU: activation quantiser (a13) and BitLinear (a5/a14) through the C ABI.
Integer results are compared bit-for-bit; float32 outputs within 1e-3 of the output RMS
(max-abs), the tolerance stated for this path."""
import os

import numpy as np
import pytest

import golden_inputs as G
from oracle import bitlinear_np as O

pytestmark = pytest.mark.gpu
TOL = 1e-3  # max-abs error relative to the output RMS


def rel_err(a, b):
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    return float(np.max(np.abs(a - b)) / np.sqrt(np.mean(b ** 2)))


@pytest.fixture(scope="module")
def ops():
    from rotor_b200 import ops
    return ops


@pytest.fixture(scope="module")
def abi():
    from rotor_b200 import abi
    return abi


@pytest.mark.parametrize("terms", [1, 2, 3])
def test_quantize_rows_bit_exact(ops, golden_dir, terms):
    x = G.quant_inputs()
    xq, sx, xsum = ops.quantize_rows(x, terms)
    q, s = O.quantize_rows(x, terms)
    m, k = x.shape
    got = xq.cpu().numpy().reshape(m, terms, -1)
    assert np.array_equal(got[:, :, :k], q)
    assert not got[:, :, k:].any()
    assert np.array_equal(sx.cpu().numpy().reshape(m, terms), s)
    assert np.array_equal(xsum.cpu().numpy().reshape(m, terms), q.astype(np.int32).sum(axis=2))
    if terms == 1:
        z = np.load(os.path.join(golden_dir, "quantize.npz"))
        assert np.array_equal(got[:, 0, :k], z["q"]) and np.array_equal(sx.cpu().numpy(), z["s"])


@pytest.mark.parametrize("k", [8, 72, 2560, 6912, 28672])
def test_quantize_rows_sizes(ops, k):
    rng = np.random.default_rng(k)
    x = (rng.standard_normal((2, k)) * 3).astype(np.float32)
    xq, sx, xsum = ops.quantize_rows(x, 2)
    q, s = O.quantize_rows(x, 2)
    assert np.array_equal(xq.cpu().numpy().reshape(2, 2, -1)[:, :, :k], q)
    assert np.array_equal(sx.cpu().numpy().reshape(2, 2), s)


@pytest.mark.parametrize("variant", ["dp4a", "mma"])
@pytest.mark.parametrize("shape", [(16, 128, 1), (20, 72, 3), (6912, 2560, 1), (6912, 2560, 3), (2560, 6912, 2),
                                   (640, 2560, 1), (48, 1280, 8), (33, 260, 11)])
def test_integer_accumulators_bit_exact(ops, abi, variant, shape):
    out, inn, ncols = shape
    rng = np.random.default_rng(out + inn + ncols)
    w = O.synth_ternary(rng, out, inn)
    tiles = ops.int8_to_tiles(w)
    kpad = abi.lib.rotor_b200_in_padded(inn)
    q = np.zeros((ncols, kpad), dtype=np.int8)
    q[:, :inn] = rng.integers(-128, 128, size=(ncols, inn), dtype=np.int8)   # full int8 range incl. -128
    xq = ops.to_device(q)
    xsum = ops.to_device(q.astype(np.int32).sum(axis=1).astype(np.int32))
    v = abi.VARIANT_DP4A if variant == "dp4a" else abi.VARIANT_MMA
    acc = ops.bitlinear_acc(tiles, out, inn, xq, xsum, v).cpu().numpy()
    want = q[:, :inn].astype(np.int32) @ w.astype(np.int32).T
    assert np.array_equal(acc, want)
    abi.device_status()


@pytest.mark.parametrize("shape", [(6912, 2560, 130), (2560, 6912, 257), (48, 1280, 32), (33, 260, 300), (640, 2560, 1024),
                                   (400, 2560, 517), (3840, 384, 256), (272, 128, 700), (2560, 2560, 64), (528, 640, 100),
                                   (6912, 2560, 192)])
def test_many_column_product_bit_exact(ops, abi, shape):
    """Prefill-sized products (32 activation columns and more) take the tcgen05 kernel (TMA-fed token
    operand, weights decoded into shared memory, int32 accumulators in tensor memory); the mma.sync
    tiled GEMM remains behind ROTOR_B200_NO_TCGEN05.  Ragged token counts, row counts that do not fill
    the 256-row tile, and K that is not a multiple of the 128-wide weight tile."""
    out, inn, ncols = shape
    rng = np.random.default_rng(out * 3 + inn + ncols)
    w = O.synth_ternary(rng, out, inn)
    tiles = ops.int8_to_tiles(w)
    kpad = abi.lib.rotor_b200_in_padded(inn)
    q = np.zeros((ncols, kpad), dtype=np.int8)
    q[:, :inn] = rng.integers(-128, 128, size=(ncols, inn), dtype=np.int8)
    xq = ops.to_device(q)
    xsum = ops.to_device(q.astype(np.int32).sum(axis=1).astype(np.int32))
    acc = ops.bitlinear_acc(tiles, out, inn, xq, xsum, abi.VARIANT_AUTO).cpu().numpy()
    want = q[:, :inn].astype(np.int32) @ w.astype(np.int32).T
    assert np.array_equal(acc, want)
    # the column-chunked tensor-core GEMV gives the same integers
    acc2 = ops.bitlinear_acc(tiles, out, inn, xq, xsum, abi.VARIANT_MMA).cpu().numpy()
    assert np.array_equal(acc2, want)


def test_tcgen05_extreme_values(ops, abi):
    """-128 x -1 and 127 x +1 over K = 6912 on the tcgen05 path: sums stay exact in int32."""
    out, inn, ncols = 256, 6912, 256
    w = np.ones((out, inn), dtype=np.int8)
    w[::2] = -1
    tiles = ops.int8_to_tiles(w)
    q = np.full((ncols, inn), -128, dtype=np.int8)
    q[1::2] = 127
    xq, xsum = ops.to_device(q), ops.to_device(q.astype(np.int32).sum(axis=1).astype(np.int32))
    acc = ops.bitlinear_acc(tiles, out, inn, xq, xsum, abi.VARIANT_AUTO).cpu().numpy()
    assert np.array_equal(acc, q.astype(np.int32) @ w.astype(np.int32).T)
    abi.device_status()


def test_extreme_values_do_not_overflow(ops, abi):
    """All weights +1 and all activations -128 over the longest row the models use."""
    out, inn = 16, 28672
    w = np.ones((out, inn), dtype=np.int8)
    tiles = ops.int8_to_tiles(w)
    q = np.full((2, inn), -128, dtype=np.int8)
    q[1] = 127
    xq, xsum = ops.to_device(q), ops.to_device(q.astype(np.int32).sum(axis=1).astype(np.int32))
    for v in (abi.VARIANT_DP4A, abi.VARIANT_MMA):
        acc = ops.bitlinear_acc(tiles, out, inn, xq, xsum, v).cpu().numpy()
        assert (acc[0] == -128 * inn).all() and (acc[1] == 127 * inn).all()


@pytest.mark.parametrize("variant", ["dp4a", "mma"])
def test_config1_matches_reference_fixture(ops, abi, golden_dir, variant):
    """Config 1 (2560 -> 6912).  The fixture is what the unmodified reference returned."""
    z = np.load(os.path.join(golden_dir, "bitlinear_2560x6912.npz"))
    w, scale, x1, x16 = G.bitlinear_case()
    tiles = ops.packed_to_tiles(O.pack_ternary_matrix(w), 6912, 2560)
    v = abi.VARIANT_DP4A if variant == "dp4a" else abi.VARIANT_MMA
    # reference semantics: three-term activations reproduce the float path
    y = ops.bitlinear_forward(tiles, 6912, 2560, x1, 3, scale, variant=v).cpu().numpy()
    assert rel_err(y, z["y1"]) < TOL
    y16 = ops.bitlinear_forward(tiles, 6912, 2560, x16, 3, scale, variant=v).cpu().numpy()
    assert rel_err(y16, z["y16"]) < TOL
    # published semantics: single-term int8; the oracle quantises identically, so the
    # integers match exactly and the float32 output to rounding
    y_int = ops.bitlinear_forward(tiles, 6912, 2560, x16, 1, scale, variant=v).cpu().numpy()
    want, acc, _, _ = O.bitlinear_int(x16, w, scale, 1)
    assert np.array_equal(y_int, want)


def test_small_ragged_layer(ops, golden_dir):
    z = np.load(os.path.join(golden_dir, "bitlinear_small.npz"))
    w, scale, x = G.small_linear_case()
    tiles = ops.packed_to_tiles(O.pack_ternary_matrix(w), 20, 72)
    y = ops.bitlinear_forward(tiles, 20, 72, x, 3, scale).cpu().numpy()
    assert rel_err(y, z["y"]) < TOL


def test_per_row_scale_vector_and_host_seam(ops, abi):
    """The plug-in call shape: scales as a per-output vector, host arrays in and out
    (src/rotor/gpu_ternary.py:138-202)."""
    import ctypes
    rng = np.random.default_rng(8)
    w = O.synth_ternary(rng, 96, 384)
    tiles = ops.int8_to_tiles(w)
    x = rng.standard_normal(384).astype(np.float32)
    scales = rng.random(96).astype(np.float32) + 0.5
    y = np.zeros(96, dtype=np.float32)
    f32 = ctypes.POINTER(ctypes.c_float)
    st = abi.lib.rotor_b200_ternary_matmul_host(tiles.data_ptr(), scales.ctypes.data_as(f32),
                                                x.ctypes.data_as(f32), 384, 96, 3, y.ctypes.data_as(f32))
    assert st == 0
    want = O.backend_matvec(O.backend_codes(w), scales, x, 384, 96)
    assert rel_err(y, want) < TOL


def test_linearity_at_full_size(ops, abi):
    """Size-independent property at the XL shape (8192 -> 28672): acc(q1 + q2) = acc(q1) + acc(q2)."""
    out, inn = 28672, 8192
    rng = np.random.default_rng(77)
    w = O.synth_ternary(rng, out, inn)
    tiles = ops.int8_to_tiles(w)
    q = rng.integers(-60, 61, size=(2, inn), dtype=np.int8)
    q3 = np.concatenate([q, (q[0] + q[1])[None, :]], axis=0).astype(np.int8)
    xq, xsum = ops.to_device(q3), ops.to_device(q3.astype(np.int32).sum(axis=1).astype(np.int32))
    for v in (abi.VARIANT_DP4A, abi.VARIANT_MMA):
        acc = ops.bitlinear_acc(tiles, out, inn, xq, xsum, v).cpu().numpy()
        assert np.array_equal(acc[0] + acc[1], acc[2])
    # and a sampled exact check of 64 rows
    rows = rng.integers(0, out, size=64)
    want = q3.astype(np.int32) @ w[rows].astype(np.int32).T
    assert np.array_equal(acc[:, rows], want)


def test_errors_are_reported_not_swallowed(ops, abi):
    with pytest.raises(ValueError):
        ops.packed_to_tiles(np.zeros((4, 4), np.uint8), 16, 128)
    assert abi.lib.rotor_b200_bitlinear_acc(None, 16, 128, None, None, 1, None, 0, None) == 1
    import torch
    x = torch.zeros((1, 128), device="cuda")
    tiles = ops.int8_to_tiles(np.zeros((16, 128), np.int8))
    small = torch.empty(256, dtype=torch.uint8, device="cuda")
    y = torch.empty((1, 16), device="cuda")
    st = abi.lib.rotor_b200_bitlinear_forward(tiles.data_ptr(), 16, 128, x.data_ptr(), 1, 1, 1.0, None,
                                              y.data_ptr(), small.data_ptr(), 8, 0, None)
    assert st == 4   # workspace too small


def test_mma_sync_gemm_kept_as_comparison_path():
    """The mma.sync tiled GEMM (the pre-tcgen05 path) stays selectable with ROTOR_B200_NO_TCGEN05=1 and
    stays bit-exact.  The switch is read once per process, hence the child process."""
    import subprocess
    import sys
    code = r'''
import sys, numpy as np
sys.path[:0] = [%r, %r]
from oracle import bitlinear_np as O
from rotor_b200 import abi, ops
rng = np.random.default_rng(4)
for out, inn, ncols in ((640, 2560, 300), (6912, 384, 64)):
    w = O.synth_ternary(rng, out, inn)
    kpad = abi.lib.rotor_b200_in_padded(inn)
    q = np.zeros((ncols, kpad), dtype=np.int8)
    q[:, :inn] = rng.integers(-128, 128, size=(ncols, inn), dtype=np.int8)
    acc = ops.bitlinear_acc(ops.int8_to_tiles(w), out, inn, ops.to_device(q),
                            ops.to_device(q.astype(np.int32).sum(axis=1).astype(np.int32)), abi.VARIANT_AUTO).cpu().numpy()
    assert np.array_equal(acc, q[:, :inn].astype(np.int32) @ w.astype(np.int32).T)
print("ok")
''' % (os.path.dirname(os.path.dirname(os.path.abspath(__file__))),
       os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "rotor-rag_b200"))
    env = dict(os.environ, ROTOR_B200_NO_TCGEN05="1")
    r = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and r.stdout.strip().endswith("ok"), r.stderr[-2000:]
