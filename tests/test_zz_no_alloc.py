"""GPU: the allocation-free layer forward (rotor_b200_bitlinear_forward_static).

It serves hosts that cannot allocate device memory at call time -- a plug-in reached
through the reference's ternary_matmul(packed, scales, x, in, out) call, which has no
workspace argument, or a serving loop whose own pool already owns all free device memory
(cudaMalloc would fail there, and stalls every stream while it runs) -- by keeping its
scratch in a fixed array inside the library.  Checked here through the C ABI: same
results as the workspace-taking entry point, on two calls in a row that reuse the array
with different shapes, plus the size limit.  This file sorts last on purpose, so that a
run that stops at the first failure has already run every other test.
"""
import os
import subprocess
import sys

import numpy as np
import pytest

from oracle import bitlinear_np as O

pytestmark = pytest.mark.gpu


def _forward_both(abi, ops, torch, w, x, terms, scale, variant):
    out, inn = w.shape
    tiles = ops.int8_to_tiles(w)
    xd = ops.to_device(x, torch.float32)
    m = xd.shape[0]
    want = ops.bitlinear_forward(tiles, out, inn, xd, terms, scale, variant=variant)
    got = torch.full((m, out), float("nan"), dtype=torch.float32, device="cuda")
    st = abi.lib.rotor_b200_bitlinear_forward_static(tiles.data_ptr(), out, inn, xd.data_ptr(), m, terms,
                                                     float(scale), None, got.data_ptr(), variant, abi.stream())
    assert st == 0, abi.lib.rotor_b200_status_string(st)
    torch.cuda.synchronize()
    return want.cpu().numpy(), got.cpu().numpy()


def test_static_scratch_matches_workspace_entry_point_twice():
    import torch
    from rotor_b200 import abi, ops
    rng = np.random.default_rng(2024)
    # call 1: 2560 -> 6912, one row, one term (K fits one split: no accumulator clearing needed)
    w1 = O.synth_ternary(rng, 6912, 2560)
    x1 = rng.standard_normal((1, 2560)).astype(np.float32)
    want, got = _forward_both(abi, ops, torch, w1, x1, 1, 0.016, abi.VARIANT_DP4A)
    assert np.array_equal(got, want)
    assert np.array_equal(got, O.bitlinear_int(x1, w1, 0.016, 1)[0])      # and equal to the oracle
    # call 2, straight after: other shape, three terms, K split with atomics into accumulators that
    # still hold call 1's values unless the entry point clears them
    w2 = O.synth_ternary(rng, 640, 6912)
    x2 = rng.standard_normal((2, 6912)).astype(np.float32)
    want, got = _forward_both(abi, ops, torch, w2, x2, 3, 0.02, abi.VARIANT_MMA)
    assert np.array_equal(got, want)
    ref = O.bitlinear_float(x2, w2, 0.02)
    assert np.max(np.abs(got - ref)) / np.sqrt(np.mean(ref.astype(np.float64) ** 2)) < 1e-3
    # call 3 repeats call 1's shape: results do not depend on what the array held before
    want, got = _forward_both(abi, ops, torch, w1, x1, 1, 0.016, abi.VARIANT_AUTO)
    assert np.array_equal(got, want)
    abi.device_status()


_FRESH = r"""
import sys
import numpy as np, torch
from oracle import bitlinear_np as O
from rotor_b200 import abi, ops
rng = np.random.default_rng(7)
w = O.synth_ternary(rng, 6912, 2560)
x = rng.standard_normal((1, 2560)).astype(np.float32)
tiles = ops.int8_to_tiles(w)                      # load-time repack; no layer forward has run yet
xd = ops.to_device(x, torch.float32)
y = torch.empty((1, 6912), dtype=torch.float32, device="cuda")
def call():
    st = abi.lib.rotor_b200_bitlinear_forward_static(tiles.data_ptr(), 6912, 2560, xd.data_ptr(), 1, 1, 0.016, None,
                                                     y.data_ptr(), abi.VARIANT_DP4A, abi.stream())
    assert st == 0, st
    torch.cuda.synchronize()
call()                                            # first forward of the process: looks the array up, loads kernels
want = O.bitlinear_int(x, w, 0.016, 1)[0]
assert np.array_equal(y.cpu().numpy(), want)
y.zero_()                                         # (torch's own fill kernel is loaded now, not inside the window)
torch.cuda.synchronize()
free0 = torch.cuda.mem_get_info()[0]
torch_bytes0 = torch.cuda.memory_allocated()
call()
call()
free1 = torch.cuda.mem_get_info()[0]
assert free1 == free0, f"device memory in use changed across static calls: {free0} -> {free1}"
assert torch.cuda.memory_allocated() == torch_bytes0
assert np.array_equal(y.cpu().numpy(), want)
assert abi.lib.rotor_b200_device_status() == 0    # also reads the status word kept in the fixed array
print("FRESH_OK")
"""


def test_static_call_first_in_a_fresh_process_allocates_nothing():
    """The static entry point as the first layer forward of a new process (its set-up path), then two more
    calls across which neither the driver's free-memory figure nor torch's allocator moves."""
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ)
    env["PYTHONPATH"] = os.pathsep.join([root, os.path.join(root, "rotor-rag_b200"), env.get("PYTHONPATH", "")])
    r = subprocess.run([sys.executable, "-c", _FRESH], env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "FRESH_OK" in r.stdout, r.stdout + r.stderr


def test_static_scratch_size_limit_is_reported():
    import torch
    from rotor_b200 import abi, ops
    lib = abi.lib
    assert lib.rotor_b200_bitlinear_static_fits(6912, 2560, 1, 3) == 1
    # 64 rows x 3 terms x 28672 outputs of int32 accumulators is far beyond 4 MiB
    assert lib.rotor_b200_bitlinear_static_fits(28672, 8192, 64, 3) == 0
    tiles = ops.int8_to_tiles(np.zeros((16, 128), np.int8))
    x = torch.zeros((64, 8192), device="cuda")
    y = torch.zeros((64, 28672), device="cuda")
    st = lib.rotor_b200_bitlinear_forward_static(tiles.data_ptr(), 28672, 8192, x.data_ptr(), 64, 3, 1.0, None,
                                                 y.data_ptr(), 0, abi.stream())
    assert st == abi.ERR_TOO_LARGE
    assert b"scratch" in lib.rotor_b200_status_string(st)
    assert lib.rotor_b200_bitlinear_forward_static(None, 16, 128, None, 1, 1, 1.0, None, None, 0, None) == 1
