"""ctypes binding of librotor_b200.so (declared in include/rotor_b200.h).

The library is the only compute path.  If it is missing or a call fails this
module raises; nothing falls back to NumPy.  torch tensors serve as device
buffers: every wrapper takes tensors (or raw pointers) and passes
``tensor.data_ptr()`` through the C ABI together with the current CUDA stream.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "librotor_b200.so")

OK = 0
VARIANT_AUTO, VARIANT_DP4A, VARIANT_MMA = 0, 1, 2
ERR_TOO_LARGE = 6
STATIC_SCRATCH_BYTES = 4 << 20


class RotorB200Error(RuntimeError):
    pass


def _load():
    if not os.path.exists(LIB_PATH):
        raise RotorB200Error(
            f"{LIB_PATH} not found: build it with `make -C rotor-rag_b200/csrc` "
            "(or __graft_entry__.build()); there is no CPU fallback")
    return C.CDLL(LIB_PATH)


lib = _load()

_p, _sz, _i, _f = C.c_void_p, C.c_size_t, C.c_int, C.c_float

_SIGNATURES = {
    "rotor_b200_version": (_i, []),
    "rotor_b200_status_string": (C.c_char_p, [_i]),
    "rotor_b200_device_status": (_i, []),
    "rotor_b200_launch_count": (C.c_ulonglong, []),
    "rotor_b200_launch_empty": (_i, [_p]),
    "rotor_b200_selftest_exchange_timeout": (_i, [C.c_longlong, _p, _p]),
    "rotor_b200_encode": (_i, [_p, _sz, _p, _p, _p]),
    "rotor_b200_decode": (_i, [_p, _p, _sz, _p, _p]),
    "rotor_b200_pack": (_i, [_p, _p, _sz, _p, _p]),
    "rotor_b200_unpack": (_i, [_p, _sz, _p, _p, _p]),
    "rotor_b200_packed_to_planes": (_i, [_p, _sz, _sz, _p, _p, _p]),
    "rotor_b200_planes_to_int8": (_i, [_p, _p, _sz, _sz, _p, _p]),
    "bitnet_to_rotor": (None, [_p, _sz, _sz, _p, _p]),
    "rotor_unpack_weights": (None, [_p, _p, _sz, _sz, _p]),
    "rotor_b200_tiles_bytes": (_sz, [_sz, _sz]),
    "rotor_b200_in_padded": (_sz, [_sz]),
    "rotor_b200_out_padded": (_sz, [_sz]),
    "rotor_b200_packed_to_tiles": (_i, [_p, _sz, _sz, _p, _p]),
    "rotor_b200_int8_to_tiles": (_i, [_p, _sz, _sz, _p, _p]),
    "rotor_b200_tiles_to_int8": (_i, [_p, _sz, _sz, _p, _p]),
    "rotor_b200_quantize_rows": (_i, [_p, _sz, _sz, _i, _p, _p, _p, _p]),
    "rotor_b200_bitlinear_acc": (_i, [_p, _sz, _sz, _p, _p, _sz, _p, _i, _p]),
    "rotor_b200_bitlinear_dequant": (_i, [_p, _p, _sz, _i, _sz, _f, _p, _p, _p]),
    "rotor_b200_bitlinear_workspace_bytes": (_sz, [_sz, _sz, _sz, _i]),
    "rotor_b200_bitlinear_forward": (_i, [_p, _sz, _sz, _p, _sz, _i, _f, _p, _p, _p, _sz, _i, _p]),
    "rotor_b200_ternary_matmul_host": (_i, [_p, _p, _p, _sz, _sz, _i, _p]),
    "rotor_b200_bitlinear_static_fits": (_i, [_sz, _sz, _sz, _i]),
    "rotor_b200_bitlinear_forward_static": (_i, [_p, _sz, _sz, _p, _sz, _i, _f, _p, _p, _i, _p]),
}


class ModelConfig(C.Structure):
    """rotor_b200_model_config"""
    _fields_ = [("vocab_size", C.c_int32), ("d_model", C.c_int32), ("n_layers", C.c_int32),
                ("n_heads", C.c_int32), ("n_kv_heads", C.c_int32), ("d_ff", C.c_int32),
                ("act_terms", C.c_int32), ("ffn_act", C.c_int32), ("causal", C.c_int32),
                ("rope_theta", C.c_float), ("eps", C.c_float),
                ("max_batch", C.c_int32), ("max_seq", C.c_int32), ("max_rows", C.c_int32),
                ("gemv_variant", C.c_int32), ("tp_size", C.c_int32), ("tp_rank", C.c_int32)]


class LayerWeights(C.Structure):
    """rotor_b200_layer_weights"""
    _fields_ = [("qkv_tiles", _p), ("o_tiles", _p), ("gate_up_tiles", _p), ("down_tiles", _p),
                ("q_scale", _f), ("k_scale", _f), ("v_scale", _f), ("o_scale", _f),
                ("gate_scale", _f), ("up_scale", _f), ("down_scale", _f),
                ("input_norm", _p), ("post_attn_norm", _p), ("attn_sub_norm", _p), ("ffn_sub_norm", _p),
                ("k_cache", _p), ("v_cache", _p)]


FFN_SILU_CLIP20, FFN_RELU2 = 0, 1
LOGITS_NONE, LOGITS_LAST, LOGITS_ALL = 0, 1, 2
_cfgp, _lwp = C.POINTER(ModelConfig), C.POINTER(LayerWeights)

_SIGNATURES.update({
    "rotor_b200_rmsnorm": (_i, [_p, _sz, _sz, _p, _f, _p, _p]),
    "rotor_b200_model_workspace_bytes": (_sz, [_cfgp]),
    "rotor_b200_model_create": (_i, [_cfgp, _lwp, _p, _p, _p, _sz, C.POINTER(_p)]),
    "rotor_b200_model_destroy": (None, [_p]),
    "rotor_b200_model_forward": (_i, [_p, _p, _i, _i, _i, _i, _p, _p, _p]),
    "rotor_b200_model_forward_hidden": (_i, [_p, _p, _i, _i, _i, _i, _i, _i, _p, _p]),
    "rotor_b200_model_decode_begin": (_i, [_p, _p, _i, _i, _p]),
    "rotor_b200_model_decode_steps": (_i, [_p, _i, _i, _p]),
    "rotor_b200_model_read_tokens": (_i, [_p, _i, _i, _p, _p]),
    "rotor_b200_model_position": (_i, [_p]),
    "rotor_b200_model_forward_ragged": (_i, [_p, _p, _i, _i, _p, _i, _p, _p, _p]),
    "rotor_b200_model_decode_begin_ragged": (_i, [_p, _p, _i, _p, _p]),
    "rotor_b200_block_workspace_bytes": (_sz, [_cfgp, _i]),
    "rotor_b200_set_pdl": (_i, [_i]),
    "rotor_b200_sample": (_i, [_p, _i, _i, _i, _i, C.c_float, C.c_float, C.c_uint64, C.c_uint64, _p, _p]),
    "rotor_b200_tp_unique_id": (_i, [_p]),
    "rotor_b200_tp_init": (_i, [_i, _i, _p, C.POINTER(_p)]),
    "rotor_b200_tp_destroy": (None, [_p]),
    "rotor_b200_model_set_tp": (_i, [_p, _p]),
    "rotor_b200_ffn_forward": (_i, [_cfgp, _lwp, _p, _p, _i, _p, _p, _sz, _p]),
    "rotor_b200_attention_forward": (_i, [_cfgp, _lwp, _p, _i, _i, _i, _p, _p, _sz, _p]),
})


def _declare(signatures):
    for name, (res, args) in signatures.items():
        fn = getattr(lib, name)  # AttributeError here = header and library out of step
        fn.restype = res
        fn.argtypes = args


_declare(_SIGNATURES)


def check(status: int, what: str = "librotor_b200 call"):
    if status != OK:
        raise RotorB200Error(f"{what}: {lib.rotor_b200_status_string(status).decode()} (status {status})")


def device_status():
    """Raise if a bounded device-side wait gave up since the last check."""
    check(lib.rotor_b200_device_status(), "device status")


def ptr(t):
    """Device (or host) address of a torch tensor / numpy array / int / None."""
    if t is None:
        return None
    if isinstance(t, int):
        return t
    if hasattr(t, "data_ptr"):
        return t.data_ptr()
    return t.ctypes.data


def stream():
    import torch
    return torch.cuda.current_stream().cuda_stream


def require_cuda():
    import torch
    if not torch.cuda.is_available():
        raise RotorB200Error("no CUDA device: the rotor_b200 path runs on a B200 only (no CPU fallback)")
    return torch


def set_pdl(enable: bool) -> bool:
    """Programmatic dependent launch for the decode chain (see rotor_b200_set_pdl)."""
    return bool(lib.rotor_b200_set_pdl(int(bool(enable))))


if os.environ.get("ROTOR_B200_PDL") is not None:
    set_pdl(os.environ["ROTOR_B200_PDL"] not in ("", "0"))
