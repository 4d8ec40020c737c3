"""Host-side helper that writes the reference's packed wire format (for checkpoints and
tests).  This is data marshalling, not part of the compute path."""
import numpy as np


def pack_ternary_matrix(w):
    """int8 [out, in] in {-1,0,+1} -> uint8 [out, in/4]: weight 4k+j of a row in bits
    (2j+1, 2j) of byte k, 10 = +1, 01 = -1, 00 = 0 (reference src/rotor/core.py:97-108)."""
    w = np.asarray(w, dtype=np.int8)
    out, inn = w.shape
    if inn % 4:
        raise ValueError("in_features must be a multiple of 4")
    field = np.where(w > 0, 2, np.where(w < 0, 1, 0)).astype(np.uint8).reshape(out, inn // 4, 4)
    return (field << (np.arange(4, dtype=np.uint8) * 2)).sum(axis=2).astype(np.uint8)
