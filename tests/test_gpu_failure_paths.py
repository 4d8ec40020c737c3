"""GPU: what happens when a bounded device-side wait runs out.

The reference's plug-in call swallows every failure and silently recomputes on the CPU
(src/rotor/transformer.py:145-147).  Here a wait that gives up sets a status word the host reads,
later waits return at once instead of each burning their limit, and the library stays usable.
Nothing in this test faults, traps or hangs the GPU: the peer-memory all-reduce is run on one GPU
against a "peer" buffer that nothing writes, with a wait limit of about a millisecond.
"""
import ctypes as C

import numpy as np
import pytest

from oracle import bitlinear_np as O

pytestmark = pytest.mark.gpu


def test_exchange_wait_runs_out_then_library_still_works():
    import torch
    from rotor_b200 import abi, ops
    lib = abi.lib
    assert lib.rotor_b200_device_status() == 0
    status, ms = C.c_uint(0), C.c_float(-1.0)
    rc = lib.rotor_b200_selftest_exchange_timeout(2_000_000, C.byref(status), C.byref(ms))   # about 1 ms of SM cycles
    assert rc == 0, lib.rotor_b200_status_string(rc)
    assert status.value == (0x7E000000 | 1)            # gave up waiting for source rank 1
    # the second collective ran with a limit of about a second per source: it saw the status word and did not wait
    assert 0.0 <= ms.value < 100.0, ms.value
    # the host reads the code once, and the word is clear afterwards
    assert lib.rotor_b200_device_status() == (0x7E000000 | 1)
    assert lib.rotor_b200_device_status() == 0
    with pytest.raises(abi.RotorB200Error):
        lib.rotor_b200_selftest_exchange_timeout(1_000_000, C.byref(status), C.byref(ms))
        abi.device_status()                             # the Python wrapper turns a set word into an exception
    assert lib.rotor_b200_device_status() == 0
    # an ordinary call afterwards gives the right answer
    rng = np.random.default_rng(5)
    w = O.synth_ternary(rng, 640, 2560)
    x = rng.standard_normal((2, 2560)).astype(np.float32)
    tiles = ops.int8_to_tiles(w)
    y = ops.bitlinear_forward(tiles, 640, 2560, ops.to_device(x, torch.float32), 1, 0.02).cpu().numpy()
    assert np.array_equal(y, O.bitlinear_int(x, w, 0.02, 1)[0])
    abi.device_status()


def test_selftest_rejects_bad_limits():
    from rotor_b200 import abi
    status, ms = C.c_uint(0), C.c_float(0.0)
    assert abi.lib.rotor_b200_selftest_exchange_timeout(0, C.byref(status), C.byref(ms)) == 1
    assert abi.lib.rotor_b200_selftest_exchange_timeout(10 ** 12, C.byref(status), C.byref(ms)) == 1
    assert abi.lib.rotor_b200_selftest_exchange_timeout(1000, None, None) == 1
