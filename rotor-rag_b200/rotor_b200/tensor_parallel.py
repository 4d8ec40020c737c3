"""Tensor-parallel BitNet model: one process per GPU, BitLinear sharded Megatron-style.

The reference runs on one device.  For models whose decode step is worth spreading over
the GPUs of one box, every block is split as

* q / k / v, gate, up: by output rows (whole query heads with their KV heads, whole FFN
  channels), so each rank runs attention and the gating on its own heads / channels;
* o, down: by input columns; every rank quantises its slice of the input row with the
  row's GLOBAL absolute maximum (one float per row all-reduced with max), so the int32
  partial products add up, after an integer all-reduce, to exactly the single-GPU
  accumulator;
* the FFN sub-norm runs over the sharded row with an all-reduced sum of squares;
* the tied LM head by vocabulary rows; greedy picks all-gather one (value, index) pair.

Only the one-term activation quantiser (``act_terms == 1``, the published int8
behaviour) is supported: its scale depends on the row maximum alone.

The shard arithmetic (``shard_layer``) is plain NumPy and needs no GPU.
"""
from __future__ import annotations

import ctypes as C
from typing import Dict, Optional

import numpy as np

from . import abi, ops
from .abi import RotorB200Error, check, lib, ptr
from .semantics import BASELINE, Semantics

_FFN_ACT = {"silu_clip20": 0, "relu2": 1}


# ------------------------------------------------------------------------------ shard math
def local_dims(cfg: Dict, size: int) -> Dict:
    """Per-rank head / channel / vocabulary counts of a model split over ``size`` ranks."""
    h, hk, ff, v = cfg["n_heads"], cfg["n_kv_heads"], cfg["d_ff"], cfg["vocab_size"]
    if h % size or hk % size or ff % size or v % size:
        raise ValueError(f"heads {h}, KV heads {hk}, d_ff {ff} and vocabulary {v} must all divide by {size} ranks")
    hd = cfg["d_model"] // h
    return dict(n_heads=h // size, n_kv_heads=hk // size, d_ff=ff // size, vocab=v // size, head_dim=hd,
                dq=h // size * hd, dkv=hk // size * hd)


def shard_layer(lw: Dict, cfg: Dict, rank: int, size: int) -> Dict:
    """One rank's share of a block.  ``lw`` maps q/k/v/o/gate/up/down to (int8 matrix
    [out, in], scale) and the four norm names to float32 vectors.  Row-parallel matrices
    keep rows [rank*n, (rank+1)*n); o and down keep the matching columns; the FFN sub-norm
    weight is sliced like the channels; the other norms are replicated."""
    ld = local_dims(cfg, size)
    rq = slice(rank * ld["dq"], (rank + 1) * ld["dq"])
    rkv = slice(rank * ld["dkv"], (rank + 1) * ld["dkv"])
    rff = slice(rank * ld["d_ff"], (rank + 1) * ld["d_ff"])
    cut = lambda name, rows, cols: (np.ascontiguousarray(lw[name][0][rows, cols]), lw[name][1])
    every = slice(None)
    return {
        "q": cut("q", rq, every), "k": cut("k", rkv, every), "v": cut("v", rkv, every),
        "o": cut("o", every, rq),
        "gate": cut("gate", rff, every), "up": cut("up", rff, every), "down": cut("down", every, rff),
        "input_norm": lw["input_norm"], "post_attn_norm": lw["post_attn_norm"],
        "attn_sub_norm": lw["attn_sub_norm"],
        "ffn_sub_norm": np.ascontiguousarray(lw["ffn_sub_norm"][rff]),
    }


# ------------------------------------------------------------------------------ communicator
class TPGroup:
    """NCCL communicator owned by the C library.  ``torch.distributed`` (any backend)
    carries the 128-byte id from rank 0 to the others; the data path does not use it."""

    def __init__(self, rank: Optional[int] = None, size: Optional[int] = None):
        import torch
        import torch.distributed as dist
        abi.require_cuda()
        if not dist.is_initialized():
            raise RotorB200Error("torch.distributed must be initialised before a TPGroup is made")
        self.rank = dist.get_rank() if rank is None else rank
        self.size = dist.get_world_size() if size is None else size
        uid = torch.zeros(128, dtype=torch.uint8)
        if self.rank == 0:
            buf = (C.c_ubyte * 128)()
            check(lib.rotor_b200_tp_unique_id(buf), "tp_unique_id")
            uid = torch.tensor(list(buf), dtype=torch.uint8)
        if dist.get_backend() == "nccl":
            uid = uid.cuda()
        dist.broadcast(uid, src=0)
        raw = bytes(uid.cpu().tolist())
        comm = C.c_void_p()
        check(lib.rotor_b200_tp_init(self.rank, self.size, raw, C.byref(comm)), "tp_init")
        self.comm = comm

    def close(self):
        c, self.comm = getattr(self, "comm", None), None
        if c:
            lib.rotor_b200_tp_destroy(c)


# ------------------------------------------------------------------------------ model
class ShardedBitNetModel:
    """This rank's share of a BitNet model and the handle that runs it.

    ``forward`` returns logits of this rank's vocabulary slice
    ``[rank*V/size, (rank+1)*V/size)``; ``generate_greedy`` returns the same global token
    ids on every rank.
    """

    def __init__(self, config: Dict, group: TPGroup, *, semantics: Semantics = BASELINE, max_seq: int = 2048,
                 max_batch: int = 1, max_rows: Optional[int] = None):
        torch = abi.require_cuda()
        if semantics.act_terms != 1:
            raise RotorB200Error("tensor parallelism needs act_terms == 1 (one absmax scale per row)")
        self.config, self.group, self.semantics = dict(config), group, semantics
        self.ld = local_dims(config, group.size)
        self.d_model, self.n_layers, self.vocab_size = config["d_model"], config["n_layers"], config["vocab_size"]
        self.max_seq, self.max_batch = max_seq, max_batch
        self.max_rows = max_rows or min(max_seq, 512) * max_batch
        d, ld, tb = self.d_model, self.ld, lib.rotor_b200_tiles_bytes
        self._embed = torch.zeros((self.vocab_size, d), dtype=torch.bfloat16, device="cuda")
        self._final_norm = torch.ones(d, dtype=torch.float32, device="cuda")
        self._layers = []
        for _ in range(self.n_layers):
            nq, nkv, nff = tb(ld["dq"], d), tb(ld["dkv"], d), tb(ld["d_ff"], d)
            L = dict(qkv=torch.empty(nq + 2 * nkv, dtype=torch.uint8, device="cuda"),
                     o=torch.empty(tb(d, ld["dq"]), dtype=torch.uint8, device="cuda"),
                     gate_up=torch.empty(2 * nff, dtype=torch.uint8, device="cuda"),
                     down=torch.empty(tb(d, ld["d_ff"]), dtype=torch.uint8, device="cuda"),
                     scales=dict(q=1.0, k=1.0, v=1.0, o=1.0, gate=1.0, up=1.0, down=1.0),
                     input_norm=torch.ones(d, dtype=torch.float32, device="cuda"),
                     post_attn_norm=torch.ones(d, dtype=torch.float32, device="cuda"),
                     attn_sub_norm=torch.ones(d, dtype=torch.float32, device="cuda"),
                     ffn_sub_norm=torch.ones(ld["d_ff"], dtype=torch.float32, device="cuda"))
            L["views"] = dict(q=(L["qkv"][:nq], ld["dq"], d), k=(L["qkv"][nq:nq + nkv], ld["dkv"], d),
                              v=(L["qkv"][nq + nkv:], ld["dkv"], d), o=(L["o"], d, ld["dq"]),
                              gate=(L["gate_up"][:nff], ld["d_ff"], d), up=(L["gate_up"][nff:], ld["d_ff"], d),
                              down=(L["down"], d, ld["d_ff"]))
            self._layers.append(L)
        self._handle = None
        self._ws = None
        self._caches = None

    # -- loading ---------------------------------------------------------------------------
    def _set_matrix(self, L, name, w, scale):
        torch = abi.require_cuda()
        view, out, inn = L["views"][name]
        wd = ops.to_device(w, torch.int8)
        if tuple(wd.shape) != (out, inn):
            raise ValueError(f"{name}: shard has shape {tuple(wd.shape)}, expected {(out, inn)}")
        check(lib.rotor_b200_int8_to_tiles(ptr(wd), out, inn, ptr(view), abi.stream()), "int8_to_tiles")
        L["scales"][name] = float(scale)

    def load_from_params(self, params: Dict):
        """``params``: the whole model on the host (embed, norm, layers as for ``shard_layer``);
        each rank keeps its share."""
        torch = abi.require_cuda()
        self._embed.copy_(torch.from_numpy(np.ascontiguousarray(params["embed"])).to(torch.bfloat16))
        self._final_norm.copy_(torch.from_numpy(np.asarray(params["norm"], dtype=np.float32)))
        for L, lw in zip(self._layers, params["layers"]):
            sh = shard_layer(lw, self.config, self.group.rank, self.group.size)
            for name in ("q", "k", "v", "o", "gate", "up", "down"):
                self._set_matrix(L, name, *sh[name])
            for name in ("input_norm", "post_attn_norm", "attn_sub_norm", "ffn_sub_norm"):
                L[name].copy_(torch.from_numpy(np.asarray(sh[name], dtype=np.float32)))
        self._handle = None

    def load_random(self, seed: int = 0, scale: float = 0.015955):
        """Seeded random weights generated on the device: every rank draws the WHOLE matrix
        of each projection from the same generator state and keeps its share, so the ranks
        of any group size hold slices of one and the same model."""
        torch = abi.require_cuda()
        g = torch.Generator(device="cuda")
        g.manual_seed(seed)
        cfg, r, n, ld, d = self.config, self.group.rank, self.group.size, self.ld, self.d_model
        hd = ld["head_dim"]
        self._embed.copy_((0.02 * torch.randn(self._embed.shape, generator=g, device="cuda")).to(torch.bfloat16))
        rs = np.random.default_rng(seed)
        full = dict(q=(cfg["n_heads"] * hd, d), k=(cfg["n_kv_heads"] * hd, d), v=(cfg["n_kv_heads"] * hd, d),
                    o=(d, cfg["n_heads"] * hd), gate=(cfg["d_ff"], d), up=(cfg["d_ff"], d), down=(d, cfg["d_ff"]))
        for L in self._layers:
            for name in ("q", "k", "v", "o", "gate", "up", "down"):
                w = torch.randint(-1, 2, full[name], generator=g, device="cuda", dtype=torch.int8)
                _, out, inn = L["views"][name]
                if name in ("o", "down"):
                    w = w[:, r * inn:(r + 1) * inn].contiguous()
                else:
                    w = w[r * out:(r + 1) * out].contiguous()
                self._set_matrix(L, name, w, scale * (1.0 + 0.25 * rs.random()))
                del w
        self._handle = None

    # -- handle ----------------------------------------------------------------------------
    def _ensure_handle(self, batch=1, seq=1, total=1):
        torch = abi.require_cuda()
        grow = self._handle is not None and (batch > self.max_batch or total > self.max_seq
                                             or batch * seq > self.max_rows)
        if self._handle is not None and not grow:
            return self._handle
        if self._handle is not None:
            lib.rotor_b200_model_destroy(self._handle)
            self._handle = None
        self.max_batch, self.max_seq = max(self.max_batch, batch), max(self.max_seq, total)
        self.max_rows = max(self.max_rows, batch * seq)
        cfg, sem, ld = self.config, self.semantics, self.ld
        self._cfg = abi.ModelConfig(vocab_size=self.vocab_size, d_model=self.d_model, n_layers=self.n_layers,
                                    n_heads=cfg["n_heads"], n_kv_heads=cfg["n_kv_heads"], d_ff=cfg["d_ff"],
                                    act_terms=1, ffn_act=_FFN_ACT[sem.ffn_act], causal=int(sem.causal),
                                    rope_theta=float(sem.rope_theta or 0.0), eps=float(sem.eps),
                                    max_batch=self.max_batch, max_seq=self.max_seq, max_rows=self.max_rows,
                                    gemv_variant=sem.gemv_variant, tp_size=self.group.size, tp_rank=self.group.rank)
        shape = (self.max_batch, ld["n_kv_heads"], self.max_seq, ld["head_dim"])
        old = self._caches
        self._caches = []
        for i in range(self.n_layers):
            k = torch.zeros(shape, dtype=torch.float32, device="cuda")
            v = torch.zeros(shape, dtype=torch.float32, device="cuda")
            if old is not None:
                ob, os_ = old[i][0].shape[0], old[i][0].shape[2]
                k[:ob, :, :os_] = old[i][0]
                v[:ob, :, :os_] = old[i][1]
            self._caches.append((k, v))
        arr = (abi.LayerWeights * self.n_layers)()
        for lw, L, (k, v) in zip(arr, self._layers, self._caches):
            lw.qkv_tiles, lw.o_tiles = ptr(L["qkv"]), ptr(L["o"])
            lw.gate_up_tiles, lw.down_tiles = ptr(L["gate_up"]), ptr(L["down"])
            s = L["scales"]
            lw.q_scale, lw.k_scale, lw.v_scale, lw.o_scale = s["q"], s["k"], s["v"], s["o"]
            lw.gate_scale, lw.up_scale, lw.down_scale = s["gate"], s["up"], s["down"]
            lw.input_norm, lw.post_attn_norm = ptr(L["input_norm"]), ptr(L["post_attn_norm"])
            lw.attn_sub_norm, lw.ffn_sub_norm = ptr(L["attn_sub_norm"]), ptr(L["ffn_sub_norm"])
            lw.k_cache, lw.v_cache = ptr(k), ptr(v)
        need = lib.rotor_b200_model_workspace_bytes(C.byref(self._cfg))
        if need == 0:
            raise RotorB200Error("model shape not supported by the tensor-parallel GPU path")
        self._ws = torch.empty(need, dtype=torch.uint8, device="cuda")
        h = C.c_void_p()
        check(lib.rotor_b200_model_create(C.byref(self._cfg), arr, ptr(self._embed), ptr(self._final_norm),
                                          ptr(self._ws), need, C.byref(h)), "model_create")
        check(lib.rotor_b200_model_set_tp(h, self.group.comm), "model_set_tp")
        self._handle = h
        return h

    def __del__(self):
        h, self._handle = getattr(self, "_handle", None), None
        if h:
            lib.rotor_b200_model_destroy(h)

    # -- forward ---------------------------------------------------------------------------
    def forward(self, input_ids, past: int = 0, logits_positions: str = "all"):
        """Logits of this rank's vocabulary slice: [batch, seq or 1, vocab/size].  Collective:
        every rank must make the same call."""
        torch = abi.require_cuda()
        ids = np.asarray(input_ids, dtype=np.int64)
        if ids.ndim == 1:
            ids = ids[None, :]
        batch, seq = ids.shape
        h = self._ensure_handle(batch, seq, past + seq)
        allpos = logits_positions == "all"
        out = torch.empty((batch, seq if allpos else 1, self.ld["vocab"]), dtype=torch.float32, device="cuda")
        ids_d = ops.to_device(ids)
        check(lib.rotor_b200_model_forward(h, ptr(ids_d), batch, seq, past,
                                           abi.LOGITS_ALL if allpos else abi.LOGITS_LAST, ptr(out), None,
                                           abi.stream()), "model_forward")
        abi.device_status()
        return out.cpu().numpy()

    def forward_hidden(self, hidden, past: int = 0, layer_begin: int = 0, layer_end: Optional[int] = None,
                       final_norm: bool = False):
        """Blocks [layer_begin, layer_end) applied to replicated hidden rows [batch, seq, d_model];
        returns the (replicated) residual stream, or its normed form.  Collective."""
        torch = abi.require_cuda()
        x = np.asarray(hidden, dtype=np.float32)
        batch, seq, d = x.shape
        h = self._ensure_handle(batch, seq, past + seq)
        xd = ops.to_device(x.reshape(batch * seq, d), torch.float32)
        y = torch.empty_like(xd)
        check(lib.rotor_b200_model_forward_hidden(h, ptr(xd), batch, seq, past, layer_begin,
                                                  self.n_layers if layer_end is None else layer_end,
                                                  int(final_norm), ptr(y), abi.stream()), "model_forward_hidden")
        abi.device_status()
        return y.cpu().numpy().reshape(batch, seq, d)

    def generate_greedy(self, prompt_ids, max_new_tokens: int, use_graph: bool = False):
        """Device-resident greedy generation; returns the new global token ids (the same list
        on every rank).  Collective."""
        torch = abi.require_cuda()
        prompt = np.asarray(prompt_ids, dtype=np.int64).reshape(1, -1)
        n_prompt = prompt.shape[1]
        if max_new_tokens <= 0:
            return []
        h = self._ensure_handle(1, n_prompt, n_prompt + max_new_tokens)
        ids_d = ops.to_device(prompt)
        first = torch.empty(1, dtype=torch.int64, device="cuda")
        stream = torch.cuda.current_stream()
        if use_graph and stream.cuda_stream == 0:
            if getattr(self, "_stream", None) is None:
                self._stream = torch.cuda.Stream()
            self._stream.wait_stream(stream)
            stream = self._stream
        s = stream.cuda_stream
        out = []
        with torch.cuda.stream(stream):
            check(lib.rotor_b200_model_forward(h, ptr(ids_d), 1, n_prompt, 0, abi.LOGITS_NONE, None, ptr(first), s),
                  "prefill")
            out.append(int(first.cpu()[0]))
            remaining = max_new_tokens - 1
            if remaining > 0:
                check(lib.rotor_b200_model_decode_begin(h, ptr(first), 1, n_prompt, s), "decode_begin")
                check(lib.rotor_b200_model_decode_steps(h, remaining, int(use_graph), s), "decode_steps")
                buf = np.empty(remaining, dtype=np.int64)
                check(lib.rotor_b200_model_read_tokens(h, 0, remaining, buf.ctypes.data, s), "read_tokens")
                out += [int(t) for t in buf]
        abi.device_status()
        return out
