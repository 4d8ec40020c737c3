"""Tensor-level wrappers over the C ABI.  torch tensors are buffers only: every
function here allocates its outputs with torch and hands raw pointers to
librotor_b200.so on the current CUDA stream."""
from __future__ import annotations

import numpy as np

from . import abi
from .abi import lib, ptr, check


def _torch():
    return abi.require_cuda()


def to_device(a, dtype=None):
    """numpy array / tensor -> contiguous CUDA tensor."""
    torch = _torch()
    if isinstance(a, np.ndarray):
        a = torch.from_numpy(np.ascontiguousarray(a))
    if dtype is not None:
        a = a.to(dtype)
    return a.contiguous().cuda()


# ------------------------------------------------------------------ format
def encode(w):
    torch = _torch()
    w = to_device(w, torch.int8).reshape(-1)
    plus = torch.empty(w.numel(), dtype=torch.uint8, device="cuda")
    minus = torch.empty_like(plus)
    check(lib.rotor_b200_encode(ptr(w), w.numel(), ptr(plus), ptr(minus), abi.stream()), "encode")
    return plus, minus


def decode(plus, minus):
    torch = _torch()
    plus, minus = to_device(plus, torch.uint8).reshape(-1), to_device(minus, torch.uint8).reshape(-1)
    w = torch.empty(plus.numel(), dtype=torch.int8, device="cuda")
    check(lib.rotor_b200_decode(ptr(plus), ptr(minus), plus.numel(), ptr(w), abi.stream()), "decode")
    return w


def pack(plus, minus):
    torch = _torch()
    plus, minus = to_device(plus, torch.uint8).reshape(-1), to_device(minus, torch.uint8).reshape(-1)
    n = plus.numel()
    packed = torch.empty(n // 4, dtype=torch.uint8, device="cuda")
    check(lib.rotor_b200_pack(ptr(plus), ptr(minus), n, ptr(packed), abi.stream()), "pack")
    return packed


def unpack(packed, n):
    torch = _torch()
    packed = to_device(packed, torch.uint8).reshape(-1)
    if packed.numel() * 4 < n:
        raise ValueError("packed array shorter than n rotors")
    plus = torch.empty(n, dtype=torch.uint8, device="cuda")
    minus = torch.empty_like(plus)
    check(lib.rotor_b200_unpack(ptr(packed), n, ptr(plus), ptr(minus), abi.stream()), "unpack")
    return plus, minus


def packed_to_planes(packed, cols=None):
    torch = _torch()
    packed = to_device(packed, torch.uint8)
    rows, nb = packed.shape
    cols = nb * 4 if cols is None else cols
    plus = torch.empty((rows, (cols + 7) // 8), dtype=torch.uint8, device="cuda")
    minus = torch.empty_like(plus)
    check(lib.rotor_b200_packed_to_planes(ptr(packed), rows, cols, ptr(plus), ptr(minus), abi.stream()),
          "packed_to_planes")
    return plus, minus


def planes_to_int8(plus, minus, rows, cols):
    torch = _torch()
    plus, minus = to_device(plus, torch.uint8), to_device(minus, torch.uint8)
    w = torch.empty((rows, cols), dtype=torch.int8, device="cuda")
    check(lib.rotor_b200_planes_to_int8(ptr(plus), ptr(minus), rows, cols, ptr(w), abi.stream()), "planes_to_int8")
    return w


# ------------------------------------------------------------------ tiles
def packed_to_tiles(packed, out, inn):
    torch = _torch()
    packed = to_device(packed, torch.uint8)
    if tuple(packed.shape) != (out, (inn + 3) // 4):
        raise ValueError(f"packed shape {tuple(packed.shape)} does not match [{out}, {(inn + 3) // 4}]")
    tiles = torch.empty(lib.rotor_b200_tiles_bytes(out, inn), dtype=torch.uint8, device="cuda")
    check(lib.rotor_b200_packed_to_tiles(ptr(packed), out, inn, ptr(tiles), abi.stream()), "packed_to_tiles")
    return tiles


def int8_to_tiles(w):
    torch = _torch()
    w = to_device(w, torch.int8)
    out, inn = w.shape
    tiles = torch.empty(lib.rotor_b200_tiles_bytes(out, inn), dtype=torch.uint8, device="cuda")
    check(lib.rotor_b200_int8_to_tiles(ptr(w), out, inn, ptr(tiles), abi.stream()), "int8_to_tiles")
    return tiles


def tiles_to_int8(tiles, out, inn):
    torch = _torch()
    w = torch.empty((out, inn), dtype=torch.int8, device="cuda")
    check(lib.rotor_b200_tiles_to_int8(ptr(tiles), out, inn, ptr(w), abi.stream()), "tiles_to_int8")
    return w


# ------------------------------------------------------------------ quantiser / BitLinear
def quantize_rows(x, terms=1):
    """x float32 [M, K] (CUDA) -> xq int8 [M*terms, K128], sx float32 [M*terms], xsum int32 [M*terms]."""
    torch = _torch()
    x = to_device(x, torch.float32)
    m, k = x.shape
    kpad = lib.rotor_b200_in_padded(k)
    xq = torch.empty((m * terms, kpad), dtype=torch.int8, device="cuda")
    sx = torch.empty(m * terms, dtype=torch.float32, device="cuda")
    xsum = torch.empty(m * terms, dtype=torch.int32, device="cuda")
    check(lib.rotor_b200_quantize_rows(ptr(x), m, k, terms, ptr(xq), ptr(sx), ptr(xsum), abi.stream()),
          "quantize_rows")
    return xq, sx, xsum


def bitlinear_acc(tiles, out, inn, xq, xsum, variant=abi.VARIANT_AUTO):
    """Exact int32 accumulators [ncols, out]."""
    torch = _torch()
    ncols = xq.shape[0]
    acc = torch.empty((ncols, out), dtype=torch.int32, device="cuda")
    check(lib.rotor_b200_bitlinear_acc(ptr(tiles), out, inn, ptr(xq), ptr(xsum), ncols, ptr(acc), variant,
                                       abi.stream()), "bitlinear_acc")
    return acc


def bitlinear_forward(tiles, out, inn, x, terms, wscale=1.0, wscale_vec=None, variant=abi.VARIANT_AUTO,
                      workspace=None):
    """y float32 [M, out] = BitLinear(x float32 [M, in])."""
    torch = _torch()
    x = to_device(x, torch.float32)
    m = x.shape[0]
    need = lib.rotor_b200_bitlinear_workspace_bytes(out, inn, m, terms)
    if workspace is None or workspace.numel() < need:
        workspace = torch.empty(need, dtype=torch.uint8, device="cuda")
    y = torch.empty((m, out), dtype=torch.float32, device="cuda")
    check(lib.rotor_b200_bitlinear_forward(ptr(tiles), out, inn, ptr(x), m, terms, float(wscale),
                                           ptr(wscale_vec), ptr(y), ptr(workspace), workspace.numel(),
                                           variant, abi.stream()), "bitlinear_forward")
    return y


def sample(logits, mode, top_k=50, top_p=0.9, temperature=1.0, seed=0, counter=0):
    """One token per row of CUDA float32 logits [rows, vocab]; mode 0 top-k, 1 top-p.  Returns a CUDA int64 [rows]."""
    torch = _torch()
    rows, vocab = logits.shape
    out = torch.empty(rows, dtype=torch.int64, device="cuda")
    abi.check(abi.lib.rotor_b200_sample(abi.ptr(logits), rows, vocab, int(mode), int(top_k), float(top_p),
                                        float(temperature), int(seed) & (2 ** 64 - 1), int(counter) & (2 ** 64 - 1),
                                        abi.ptr(out), abi.stream()), "sample")
    return out
