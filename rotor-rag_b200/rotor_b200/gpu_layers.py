"""The plug-in seam of the reference, served by the B200 library.

The reference's ``TernaryLinear`` asks ``rotor.gpu_layers.get_gpu()`` for a backend object
(src/rotor/transformer.py:70-75) and calls two methods on it:
``pack_ternary_weights(weights)`` at load (transformer.py:107-109) and
``ternary_matmul(packed, scales, input_vec, in_dim, out_dim)`` per token
(transformer.py:136-142; original implementation src/rotor/gpu_ternary.py:112-202).
``B200TernaryOps`` implements both on librotor_b200.so, so an unmodified reference
checkout runs its per-token GPU branch on a B200 by binding ``get_gpu`` to the one here.
Errors raise; nothing is recomputed on the CPU here.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import abi, ops
from .abi import check, lib

_instance = None


class PackedTernary:
    """Opaque result of pack_ternary_weights: the weight tiles on the device."""

    def __init__(self, tiles, out_dim, in_dim):
        self.tiles, self.out_dim, self.in_dim = tiles, out_dim, in_dim


class B200TernaryOps:
    def __init__(self, act_terms: int = 3):
        abi.require_cuda()
        self.act_terms = act_terms  # 3 = float32-faithful, like the reference's float kernel

    def pack_ternary_weights(self, weights: np.ndarray) -> PackedTernary:
        w = np.asarray(weights)
        if w.ndim != 2:
            raise ValueError("weights must be [out, in]")
        return PackedTernary(ops.int8_to_tiles(w.astype(np.int8)), w.shape[0], w.shape[1])

    def ternary_matmul(self, packed_weights: PackedTernary, scales: np.ndarray, input_vec: np.ndarray,
                       in_dim: int, out_dim: int) -> np.ndarray:
        if (packed_weights.out_dim, packed_weights.in_dim) != (out_dim, in_dim):
            raise ValueError("dimensions do not match the packed weights")
        scales = np.ascontiguousarray(scales, dtype=np.float32)
        x = np.ascontiguousarray(input_vec, dtype=np.float32)
        if scales.size != out_dim or x.size != in_dim:
            raise ValueError("scales / input length mismatch")
        y = np.empty(out_dim, dtype=np.float32)
        check(lib.rotor_b200_ternary_matmul_host(packed_weights.tiles.data_ptr(),
                                                 scales.ctypes.data_as(C.c_void_p), x.ctypes.data_as(C.c_void_p),
                                                 in_dim, out_dim, self.act_terms, y.ctypes.data_as(C.c_void_p)),
              "ternary_matmul")
        return y


def get_gpu():
    """Singleton accessor with the reference's name and behaviour (src/rotor/gpu_layers.py:14-25),
    except that a failed initialisation raises instead of silently selecting the CPU."""
    global _instance
    if _instance is None:
        _instance = B200TernaryOps()
    return _instance
