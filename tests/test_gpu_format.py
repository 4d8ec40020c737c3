"""GPU: format kernels (a1-a4) through the C ABI, bit-exact against the oracle and the
fixtures the reference produced."""
import ctypes
import os

import numpy as np
import pytest

import golden_inputs as G
from oracle import bitlinear_np as O

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from rotor_b200 import ops
    return ops


def test_encode_decode_pack_unpack(ops):
    v = np.array([1, -1, 0, 1, -1, 0, 0, 1], dtype=np.int8)     # tests/test_core.py:23-32
    plus, minus = ops.encode(v)
    assert plus.cpu().numpy().tolist() == [1, 0, 0, 1, 0, 0, 0, 1]
    assert minus.cpu().numpy().tolist() == [0, 1, 0, 0, 1, 0, 0, 0]
    assert np.array_equal(ops.decode(plus, minus).cpu().numpy(), v)
    rng = np.random.default_rng(11)
    big = rng.integers(-1, 2, size=4096 * 4).astype(np.int8)
    plus, minus = ops.encode(big)
    packed = ops.pack(plus, minus)
    assert np.array_equal(packed.cpu().numpy(), O.pack(*O.encode(big)))
    up, um = ops.unpack(packed, big.size)
    assert np.array_equal(ops.decode(up, um).cpu().numpy(), big)
    # ragged unpack: fewer rotors than the bytes hold
    up, um = ops.unpack(packed, 13)
    assert np.array_equal(up.cpu().numpy(), O.unpack(packed.cpu().numpy(), 13)[0])


def test_empty_inputs(ops):
    from rotor_b200 import abi
    assert abi.lib.rotor_b200_encode(None, 0, None, None, None) == 0
    assert abi.lib.rotor_b200_packed_to_planes(None, 0, 0, None, None, None) == 0
    assert abi.lib.rotor_b200_pack(None, None, 6, None, None) == 1


def test_planes_and_int8_match_reference_fixture(ops, golden_dir):
    z = np.load(os.path.join(golden_dir, "format.npz"))
    w = G.format_matrix()
    packed = O.pack_ternary_matrix(w)
    plus, minus = ops.packed_to_planes(packed)
    assert np.array_equal(plus.cpu().numpy(), z["plus"]) and np.array_equal(minus.cpu().numpy(), z["minus"])
    assert np.array_equal(ops.planes_to_int8(plus, minus, *w.shape).cpu().numpy(), z["weights"])
    # reserved 0b11 fields and a column count that is not a multiple of 8
    plus, minus = ops.packed_to_planes(z["raw_packed"], 36)
    assert np.array_equal(plus.cpu().numpy(), z["raw_plus"]) and np.array_equal(minus.cpu().numpy(), z["raw_minus"])
    assert np.array_equal(ops.planes_to_int8(plus, minus, 5, 36).cpu().numpy(), z["raw_weights"])


def test_reference_named_host_entry_points(golden_dir):
    """bitnet_to_rotor / rotor_unpack_weights with the reference's ctypes calling convention
    (src/rotor/bitnet_fast.py:86-102, 138-154)."""
    from rotor_b200 import abi
    z = np.load(os.path.join(golden_dir, "format.npz"))
    w = G.format_matrix()
    packed = O.pack_ternary_matrix(w)
    rows, cols = w.shape
    bit0 = np.zeros((rows, (cols + 7) // 8), dtype=np.uint8)
    bit1 = np.zeros_like(bit0)
    u8 = ctypes.POINTER(ctypes.c_uint8)
    abi.lib.bitnet_to_rotor(packed.ctypes.data_as(u8), rows, cols, bit0.ctypes.data_as(u8), bit1.ctypes.data_as(u8))
    assert np.array_equal(bit0, z["plus"]) and np.array_equal(bit1, z["minus"])
    out = np.zeros((rows, cols), dtype=np.int8)
    abi.lib.rotor_unpack_weights(bit0.ctypes.data_as(u8), bit1.ctypes.data_as(u8), rows, cols,
                                 out.ctypes.data_as(ctypes.POINTER(ctypes.c_int8)))
    assert np.array_equal(out, z["weights"])


@pytest.mark.parametrize("shape", [(16, 128), (20, 72), (6912, 2560), (640, 2560), (2560, 6912), (33, 260)])
def test_tile_repack_roundtrip(ops, shape):
    out, inn = shape
    rng = np.random.default_rng(out * 7 + inn)
    w = O.synth_ternary(rng, out, inn)
    packed = O.pack_ternary_matrix(w)
    tiles = ops.packed_to_tiles(packed, out, inn)
    assert np.array_equal(ops.tiles_to_int8(tiles, out, inn).cpu().numpy(), w)
    tiles2 = ops.int8_to_tiles(w)
    assert bool((tiles == tiles2).all())


def test_tile_layout_is_the_documented_one(ops):
    """Byte-for-byte check of the layout in include/rotor_b200.h on one 16x128 tile."""
    rng = np.random.default_rng(1)
    w = O.synth_ternary(rng, 16, 128)
    tiles = ops.int8_to_tiles(w).cpu().numpy().view(np.uint32).reshape(32, 4)
    for lane in range(32):
        g, t = lane >> 2, lane & 3
        for i in range(4):
            word = 0
            for b in range(4):
                for j in range(4):
                    code = int(w[g + 8 * (i & 1), 32 * t + 8 * j + 4 * (i >> 1) + b]) + 1
                    word |= code << (8 * b + 2 * j)
            assert tiles[lane, i] == word


def test_reserved_field_becomes_zero_weight(ops):
    packed = np.full((16, 32), 0xFF, dtype=np.uint8)
    tiles = ops.packed_to_tiles(packed, 16, 128)
    assert not ops.tiles_to_int8(tiles, 16, 128).cpu().numpy().any()
