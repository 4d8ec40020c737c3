"""GPU-backed mirror of the reference's transformer classes for this path.

Same class names, constructor arguments, attributes and ``forward`` signatures as
``src/rotor/transformer.py`` in the reference (RMSNorm :17-36, TernaryLinear :39-171,
MultiHeadAttention :174-298, GatedFFN :301-351, TransformerBlock :354-413).  Arrays
cross the API as NumPy, like the reference; every computation runs in
librotor_b200.so on the GPU.  There is no CPU branch: ``use_gpu=False`` raises.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import numpy as np

from . import abi, ops
from .abi import RotorB200Error, check, lib, ptr
from .semantics import REFERENCE, Semantics

_FFN_ACT = {"silu_clip20": abi.FFN_SILU_CLIP20, "relu2": abi.FFN_RELU2}


def _require_gpu_flag(use_gpu):
    if not use_gpu:
        raise RotorB200Error("this build has no CPU path: construct with use_gpu=True")


def _as_rows(x):
    x = np.asarray(x)
    return x.reshape(-1, x.shape[-1]), x.shape[:-1]


class RMSNorm:
    """x / sqrt(mean(x^2) + eps) * weight; reference src/rotor/transformer.py:17-36."""

    def __init__(self, dim: int, eps: float = 1e-6):
        self.eps = eps
        self.dim = dim
        self._weight = np.ones(dim, dtype=np.float32)
        self._dev = None

    @property
    def weight(self):
        return self._weight

    @weight.setter
    def weight(self, w):
        w = np.ascontiguousarray(np.asarray(w, dtype=np.float32).reshape(-1))
        if w.size != self.dim:
            raise ValueError(f"norm weight has {w.size} elements, expected {self.dim}")
        self._weight = w
        self._dev = None

    def device_weight(self):
        if self._dev is None:
            self._dev = ops.to_device(self._weight)
        return self._dev

    def forward(self, x: np.ndarray) -> np.ndarray:
        torch = abi.require_cuda()
        rows, lead = _as_rows(x)
        if rows.shape[0] == 0:  # empty input: empty output, like the NumPy reference
            return np.zeros((*lead, self.dim), dtype=np.float32)
        xd = ops.to_device(rows, torch.float32)
        y = torch.empty_like(xd)
        check(lib.rotor_b200_rmsnorm(ptr(xd), xd.shape[0], self.dim, ptr(self.device_weight()), float(self.eps),
                                     ptr(y), abi.stream()), "rmsnorm")
        return y.cpu().numpy().reshape(*lead, self.dim)


class TernaryLinear:
    """BitLinear layer: y = (x @ W.T) * scale with ternary W held in the GPU tile layout.

    Mirrors reference src/rotor/transformer.py:39-171.  ``load_from_bitnet`` takes the same
    packed uint8 [out, in/4] array and scale; the convert/decode/cache chain of the reference
    collapses into one repack kernel.  ``weights_cache`` (the reference's dense int8 copy) is
    produced on demand from the tiles.
    """

    def __init__(self, in_features: int, out_features: int, use_gpu: bool = True, *,
                 semantics: Semantics = REFERENCE, _tiles=None):
        _require_gpu_flag(use_gpu)
        self.in_features = in_features
        self.out_features = out_features
        self.use_gpu = True
        self.scale = 1.0
        self.semantics = semantics
        self.weight_shape = (out_features, in_features)
        self._tiles = _tiles          # device uint8 view, filled by load_from_bitnet
        self._loaded = False
        self._cache = None
        self._workspace = None

    # -- loading ---------------------------------------------------------------------------
    def _tile_buffer(self):
        if self._tiles is None:
            torch = abi.require_cuda()
            self._tiles = torch.empty(lib.rotor_b200_tiles_bytes(self.out_features, self.in_features),
                                      dtype=torch.uint8, device="cuda")
        return self._tiles

    def load_from_bitnet(self, packed_weights: np.ndarray, scale: float = 1.0):
        torch = abi.require_cuda()
        packed = ops.to_device(packed_weights, torch.uint8)
        want = (self.out_features, (self.in_features + 3) // 4)
        if tuple(packed.shape) != want:
            raise ValueError(f"packed weights have shape {tuple(packed.shape)}, expected {want}")
        check(lib.rotor_b200_packed_to_tiles(ptr(packed), self.out_features, self.in_features,
                                             ptr(self._tile_buffer()), abi.stream()), "packed_to_tiles")
        self.scale = float(scale)
        self._loaded = True
        self._cache = None

    def load_from_int8(self, weights, scale: float = 1.0):
        """Same as load_from_bitnet but from dense {-1,0,+1} values (host array or CUDA tensor)."""
        torch = abi.require_cuda()
        w = ops.to_device(weights, torch.int8)
        if tuple(w.shape) != (self.out_features, self.in_features):
            raise ValueError(f"weights have shape {tuple(w.shape)}, expected {self.weight_shape}")
        check(lib.rotor_b200_int8_to_tiles(ptr(w), self.out_features, self.in_features,
                                           ptr(self._tile_buffer()), abi.stream()), "int8_to_tiles")
        self.scale = float(scale)
        self._loaded = True
        self._cache = None

    @property
    def tiles(self):
        if not self._loaded:
            raise RotorB200Error("TernaryLinear has no weights: call load_from_bitnet first")
        return self._tiles

    @property
    def weights_cache(self):
        """Dense int8 [out, in] copy on the host, decoded from the tiles on first use."""
        if not self._loaded:
            return None
        if self._cache is None:
            self._cache = ops.tiles_to_int8(self._tiles, self.out_features, self.in_features).cpu().numpy()
        return self._cache

    # -- compute ---------------------------------------------------------------------------
    def forward_device(self, x):
        """x: CUDA float32 [M, in] -> CUDA float32 [M, out]."""
        torch = abi.require_cuda()
        m = x.shape[0]
        need = lib.rotor_b200_bitlinear_workspace_bytes(self.out_features, self.in_features, m,
                                                        self.semantics.act_terms)
        if self._workspace is None or self._workspace.numel() < need:
            self._workspace = torch.empty(need, dtype=torch.uint8, device="cuda")
        return ops.bitlinear_forward(self.tiles, self.out_features, self.in_features, x,
                                     self.semantics.act_terms, self.scale,
                                     variant=self.semantics.gemv_variant, workspace=self._workspace)

    def forward(self, x: np.ndarray) -> np.ndarray:
        torch = abi.require_cuda()
        rows, lead = _as_rows(x)
        if rows.shape[1] != self.in_features:
            raise ValueError(f"input has {rows.shape[1]} features, expected {self.in_features}")
        if rows.shape[0] == 0:  # empty input: empty output, like the NumPy reference
            return np.zeros((*lead, self.out_features), dtype=np.float32)
        y = self.forward_device(ops.to_device(rows, torch.float32))
        return y.cpu().numpy().reshape(*lead, self.out_features)


class KVCache:
    """Per-layer cache handle returned to callers in place of the reference's
    ``{'k': ..., 'v': ...}`` dict (src/rotor/transformer.py:250-257).  The data stays in a
    fixed device buffer; the handle records how many positions are valid.  ``cache['k']``
    / ``cache['v']`` copy the valid part to the host as [batch, n_kv, T, head_dim]."""

    def __init__(self, owner, length: int, batch: int):
        self.owner = owner
        self.length = length
        self.batch = batch

    def __getitem__(self, key):
        buf = {"k": self.owner.k_cache, "v": self.owner.v_cache}[key]
        return buf[: self.batch, :, : self.length, :].cpu().numpy()

    def __len__(self):
        return 2


class _BlockBase:
    """Device state shared by the attention and FFN halves of one block."""

    def _cfg_struct(self, sem: Semantics, max_batch: int, max_seq: int, rows: int):
        return abi.ModelConfig(vocab_size=1, d_model=self.d_model, n_layers=1, n_heads=self.n_heads,
                               n_kv_heads=self.n_kv_heads, d_ff=self.d_ff, act_terms=sem.act_terms,
                               ffn_act=_FFN_ACT[sem.ffn_act], causal=int(sem.causal),
                               rope_theta=float(sem.rope_theta or 0.0), eps=float(sem.eps),
                               max_batch=max_batch, max_seq=max_seq, max_rows=rows,
                               gemv_variant=sem.gemv_variant)

    def _workspace_for(self, cfg, rows):
        torch = abi.require_cuda()
        need = lib.rotor_b200_block_workspace_bytes(C.byref(cfg), rows)
        if need == 0:
            raise RotorB200Error("shape not supported by the GPU path (head_dim must be 32/64/128, "
                                 "projection widths multiples of 16)")
        ws = getattr(self, "_ws", None)
        if ws is None or ws.numel() < need:
            self._ws = torch.empty(need, dtype=torch.uint8, device="cuda")
        return self._ws


class MultiHeadAttention(_BlockBase):
    """Reference src/rotor/transformer.py:174-298: q/k/v projections, cache append, grouped-KV
    softmax attention, output projection, then the sub-norm."""

    def __init__(self, d_model: int, n_heads: int, n_kv_heads: Optional[int] = None,
                 head_dim: Optional[int] = None, use_gpu: bool = True, *, semantics: Semantics = REFERENCE,
                 max_seq: int = 2048, max_batch: int = 1, d_ff: int = 16):
        _require_gpu_flag(use_gpu)
        torch = abi.require_cuda()
        self.d_model = d_model
        self.n_heads = n_heads
        self.n_kv_heads = n_kv_heads if n_kv_heads is not None else n_heads
        self.head_dim = head_dim if head_dim is not None else d_model // n_heads
        if self.head_dim != d_model // n_heads:
            raise RotorB200Error("head_dim other than d_model // n_heads is not supported")
        self.d_q = self.n_heads * self.head_dim
        self.d_kv = self.n_kv_heads * self.head_dim
        self.d_ff = d_ff
        self.semantics = semantics
        self.max_seq, self.max_batch = max_seq, max_batch
        tb = lib.rotor_b200_tiles_bytes
        nq, nkv = tb(self.d_q, d_model), tb(self.d_kv, d_model)
        self.qkv_tiles = torch.empty(nq + 2 * nkv, dtype=torch.uint8, device="cuda")
        self.o_tiles = torch.empty(tb(d_model, self.d_q), dtype=torch.uint8, device="cuda")
        mk = lambda i, o, t: TernaryLinear(i, o, semantics=semantics, _tiles=t)
        self.q_proj = mk(d_model, self.d_q, self.qkv_tiles[:nq])
        self.k_proj = mk(d_model, self.d_kv, self.qkv_tiles[nq:nq + nkv])
        self.v_proj = mk(d_model, self.d_kv, self.qkv_tiles[nq + nkv:])
        self.o_proj = mk(self.d_q, d_model, self.o_tiles)
        self.attn_norm = RMSNorm(d_model, eps=semantics.eps)
        self.k_cache = None
        self.v_cache = None

    def ensure_cache(self, max_batch=None, max_seq=None):
        """Allocate (or grow, keeping the contents) the fixed K/V buffers
        [max_batch, n_kv_heads, max_seq, head_dim] float32."""
        torch = abi.require_cuda()
        mb, ms = max_batch or self.max_batch, max_seq or self.max_seq
        if self.k_cache is not None:
            mb, ms = max(mb, self.k_cache.shape[0]), max(ms, self.k_cache.shape[2])
        if self.k_cache is None or tuple(self.k_cache.shape[:3:2]) != (mb, ms):
            shape = (mb, self.n_kv_heads, ms, self.head_dim)
            k = torch.zeros(shape, dtype=torch.float32, device="cuda")
            v = torch.zeros(shape, dtype=torch.float32, device="cuda")
            if self.k_cache is not None:
                ob, os_ = self.k_cache.shape[0], self.k_cache.shape[2]
                k[:ob, :, :os_] = self.k_cache
                v[:ob, :, :os_] = self.v_cache
            self.k_cache, self.v_cache = k, v
        self.max_batch, self.max_seq = mb, ms
        return self.k_cache, self.v_cache

    def fill_layer_struct(self, lw: abi.LayerWeights):
        lw.qkv_tiles, lw.o_tiles = ptr(self.qkv_tiles), ptr(self.o_tiles)
        for p in (self.q_proj, self.k_proj, self.v_proj, self.o_proj):
            p.tiles  # raises if a projection was never loaded
        lw.q_scale, lw.k_scale, lw.v_scale, lw.o_scale = (self.q_proj.scale, self.k_proj.scale,
                                                          self.v_proj.scale, self.o_proj.scale)
        lw.attn_sub_norm = ptr(self.attn_norm.device_weight())
        k, v = self.ensure_cache()
        lw.k_cache, lw.v_cache = ptr(k), ptr(v)

    def forward(self, x: np.ndarray, mask: Optional[np.ndarray] = None, kv_cache: Optional[KVCache] = None,
                use_cache: bool = False):
        torch = abi.require_cuda()
        x = np.asarray(x)
        is_3d = x.ndim == 3
        if not is_3d:
            x = x[None, ...]
        batch, seq, _ = x.shape
        past = 0 if kv_cache is None else kv_cache.length
        sem = self.semantics
        if mask is not None:
            sem = _semantics_for_mask(sem, mask, seq, past + seq)
        self.ensure_cache(max(batch, self.max_batch), max(past + seq, self.max_seq))
        rows = batch * seq
        cfg = self._cfg_struct(sem, self.max_batch, self.max_seq, rows)
        lw = abi.LayerWeights()
        self.fill_layer_struct(lw)
        xd = ops.to_device(x.reshape(rows, self.d_model), torch.float32)
        y = torch.empty_like(xd)
        ws = self._workspace_for(cfg, rows)
        check(lib.rotor_b200_attention_forward(C.byref(cfg), C.byref(lw), ptr(xd), batch, seq, past, ptr(y),
                                               ptr(ws), ws.numel(), abi.stream()), "attention_forward")
        out = y.cpu().numpy().reshape(batch, seq, self.d_model)
        if not is_3d:
            out = out[0]
        return out, (KVCache(self, past + seq, batch) if use_cache else None)


def _semantics_for_mask(sem: Semantics, mask, seq, total):
    """The only additive mask the GPU path implements is the causal one."""
    mask = np.asarray(mask)
    causal = np.triu(np.full((seq, total), -np.inf), k=total - seq + 1)
    if mask.shape == causal.shape and np.array_equal(np.isinf(mask), np.isinf(causal)) and \
            not np.any(mask[np.isfinite(mask)]):
        return sem.with_(causal=True)
    raise NotImplementedError("only the causal additive mask is implemented on the GPU path")


def _scratch_heads(d_model):
    """A head count that makes d_model a legal attention width; a stand-alone FFN only needs it
    to size the scratch area it shares with the attention half."""
    for hd in (128, 64, 32):
        if d_model % hd == 0:
            return d_model // hd
    raise RotorB200Error("d_model must be a multiple of 32 on the GPU path")


class GatedFFN(_BlockBase):
    """Reference src/rotor/transformer.py:301-351: down(ffn_norm(gate(x) * silu(clip(up(x)))))."""

    def __init__(self, d_model: int, d_ff: int, use_gpu: bool = True, *, semantics: Semantics = REFERENCE):
        _require_gpu_flag(use_gpu)
        torch = abi.require_cuda()
        self.d_model, self.d_ff = d_model, d_ff
        self.n_heads = self.n_kv_heads = _scratch_heads(d_model)
        self.semantics = semantics
        tb = lib.rotor_b200_tiles_bytes
        n = tb(d_ff, d_model)
        self.gate_up_tiles = torch.empty(2 * n, dtype=torch.uint8, device="cuda")
        self.down_tiles = torch.empty(tb(d_model, d_ff), dtype=torch.uint8, device="cuda")
        self.gate_proj = TernaryLinear(d_model, d_ff, semantics=semantics, _tiles=self.gate_up_tiles[:n])
        self.up_proj = TernaryLinear(d_model, d_ff, semantics=semantics, _tiles=self.gate_up_tiles[n:])
        self.down_proj = TernaryLinear(d_ff, d_model, semantics=semantics, _tiles=self.down_tiles)
        self.ffn_norm = RMSNorm(d_ff, eps=semantics.eps)

    def fill_layer_struct(self, lw: abi.LayerWeights):
        for p in (self.gate_proj, self.up_proj, self.down_proj):
            p.tiles
        lw.gate_up_tiles, lw.down_tiles = ptr(self.gate_up_tiles), ptr(self.down_tiles)
        lw.gate_scale, lw.up_scale, lw.down_scale = self.gate_proj.scale, self.up_proj.scale, self.down_proj.scale
        lw.ffn_sub_norm = ptr(self.ffn_norm.device_weight())

    def forward_device(self, xd, pre_norm=None):
        """xd CUDA float32 [rows, d_model]; pre_norm: optional RMSNorm applied first on the device."""
        torch = abi.require_cuda()
        rows = xd.shape[0]
        sem = self.semantics
        cfg = self._cfg_struct(sem, 1, 1, rows)
        lw = abi.LayerWeights()
        self.fill_layer_struct(lw)
        y = torch.empty_like(xd)
        ws = self._workspace_for(cfg, rows)
        check(lib.rotor_b200_ffn_forward(C.byref(cfg), C.byref(lw),
                                         ptr(pre_norm.device_weight()) if pre_norm is not None else None,
                                         ptr(xd), rows, ptr(y), ptr(ws), ws.numel(), abi.stream()), "ffn_forward")
        return y

    def forward(self, x: np.ndarray) -> np.ndarray:
        torch = abi.require_cuda()
        rows, lead = _as_rows(x)
        if rows.shape[0] == 0:
            return np.zeros((*lead, self.d_model), dtype=np.float32)
        y = self.forward_device(ops.to_device(rows, torch.float32))
        return y.cpu().numpy().reshape(*lead, self.d_model)


class TransformerBlock:
    """Reference src/rotor/transformer.py:354-413: x + attn(input_norm(x)); x + ffn(post_attn_norm(x))."""

    def __init__(self, d_model: int, n_heads: int, d_ff: int, n_kv_heads: Optional[int] = None,
                 use_gpu: bool = True, *, semantics: Semantics = REFERENCE, max_seq: int = 2048,
                 max_batch: int = 1):
        _require_gpu_flag(use_gpu)
        self.d_model = d_model
        self.semantics = semantics
        self.input_norm = RMSNorm(d_model, eps=semantics.eps)
        self.post_attn_norm = RMSNorm(d_model, eps=semantics.eps)
        self.attention = MultiHeadAttention(d_model, n_heads, n_kv_heads, use_gpu=True, semantics=semantics,
                                            max_seq=max_seq, max_batch=max_batch, d_ff=d_ff)
        self.ffn = GatedFFN(d_model, d_ff, use_gpu=True, semantics=semantics)
        self.ffn.n_heads, self.ffn.n_kv_heads = self.attention.n_heads, self.attention.n_kv_heads
        self._solo = None

    def fill_layer_struct(self, lw: abi.LayerWeights):
        self.attention.fill_layer_struct(lw)
        self.ffn.fill_layer_struct(lw)
        lw.input_norm = ptr(self.input_norm.device_weight())
        lw.post_attn_norm = ptr(self.post_attn_norm.device_weight())

    def forward(self, x: np.ndarray, mask: Optional[np.ndarray] = None, kv_cache: Optional[KVCache] = None,
                use_cache: bool = False):
        """Stand-alone block call; inside a model the blocks run through the model handle."""
        from .bitnet_model import _SoloBlockRunner
        if self._solo is None:
            self._solo = _SoloBlockRunner(self)
        return self._solo.forward(x, mask, kv_cache, use_cache)
