"""GPU-backed mirror of the reference's model container and loader.

``BitNetModel`` and ``load_bitnet_model`` keep the interface of
``src/rotor/bitnet_model.py`` (constructor :41-90, loader :92-188, forward :190-244,
load_bitnet_model :349-394): same config keys, same safetensors tensor names, same
``forward(input_ids, return_logits, past_kv_cache, use_cache) -> (logits, caches)``.
The forward pass runs through one C handle (rotor_b200_model_*); greedy generation can
stay on the device end to end (``generate_greedy``), which is what TextGenerator uses.
"""
from __future__ import annotations

import ctypes as C
import json
from pathlib import Path
from typing import Dict, Optional

import numpy as np

from . import abi, ops
from .abi import RotorB200Error, check, lib, ptr
from .semantics import REFERENCE, Semantics
from .transformer import (KVCache, RMSNorm, TransformerBlock, _FFN_ACT, _require_gpu_flag,
                          _semantics_for_mask)


class _Handle:
    """Owns one rotor_b200 model handle plus the device workspace it points into."""

    def __init__(self, blocks, embed, final_norm, vocab, sem: Semantics, max_batch, max_seq, max_rows):
        torch = abi.require_cuda()
        b0 = blocks[0]
        att = b0.attention
        self.cfg = abi.ModelConfig(vocab_size=vocab, d_model=b0.d_model, n_layers=len(blocks), n_heads=att.n_heads,
                                   n_kv_heads=att.n_kv_heads, d_ff=b0.ffn.d_ff, act_terms=sem.act_terms,
                                   ffn_act=_FFN_ACT[sem.ffn_act], causal=int(sem.causal),
                                   rope_theta=float(sem.rope_theta or 0.0), eps=float(sem.eps),
                                   max_batch=max_batch, max_seq=max_seq, max_rows=max_rows,
                                   gemv_variant=sem.gemv_variant)
        # every block's cache gets the same capacity (never smaller than what it already holds)
        for blk in blocks:
            if blk.attention.k_cache is not None:
                max_batch = max(max_batch, blk.attention.k_cache.shape[0])
                max_seq = max(max_seq, blk.attention.k_cache.shape[2])
        for blk in blocks:
            blk.attention.ensure_cache(max_batch, max_seq)
        self.cfg.max_batch, self.cfg.max_seq = max_batch, max_seq
        arr = (abi.LayerWeights * len(blocks))()
        for i, blk in enumerate(blocks):
            blk.fill_layer_struct(arr[i])
        need = lib.rotor_b200_model_workspace_bytes(C.byref(self.cfg))
        if need == 0:
            raise RotorB200Error("model shape not supported by the GPU path (head_dim 32/64/128, d_model a "
                                 "multiple of 256, projection widths multiples of 16)")
        self.workspace = torch.empty(need, dtype=torch.uint8, device="cuda")
        self.keep = (blocks, embed, final_norm)  # the handle points into these tensors
        h = C.c_void_p()
        check(lib.rotor_b200_model_create(C.byref(self.cfg), arr, ptr(embed), ptr(final_norm), ptr(self.workspace),
                                          need, C.byref(h)), "model_create")
        self.h = h

    def __del__(self):
        h, self.h = getattr(self, "h", None), None
        if h:
            lib.rotor_b200_model_destroy(h)


class BitNetModel:
    """Complete model: bf16 embedding table (tied LM head), n_layers blocks, final RMSNorm."""

    def __init__(self, config: Dict, use_gpu: bool = True, *, semantics: Semantics = REFERENCE,
                 max_seq: int = 2048, max_batch: int = 1, max_rows: Optional[int] = None, verbose: bool = False):
        _require_gpu_flag(use_gpu)
        torch = abi.require_cuda()
        self.config = config
        self.vocab_size = config['vocab_size']
        self.d_model = config['d_model']
        self.n_layers = config['n_layers']
        self.n_heads = config.get('n_heads', 20)
        self.n_kv_heads = config.get('n_kv_heads', 4)
        self.d_ff = config.get('d_ff', 6912)
        self.use_gpu = True
        self.semantics = semantics
        self.max_seq, self.max_batch = max_seq, max_batch
        self.max_rows = max_rows or min(max_seq, 512) * max_batch
        self._embed = torch.zeros((self.vocab_size, self.d_model), dtype=torch.bfloat16, device="cuda")
        self.layers = [TransformerBlock(self.d_model, self.n_heads, self.d_ff, self.n_kv_heads, use_gpu=True,
                                        semantics=semantics, max_seq=max_seq, max_batch=max_batch)
                       for _ in range(self.n_layers)]
        self.norm = RMSNorm(self.d_model, eps=semantics.eps)
        self.lm_head_weight = None  # tied to the embeddings, as in the reference
        self._handle = None
        self._norm_versions = None
        if verbose:
            print(f"Initialized BitNet model on GPU: vocab {self.vocab_size:,}, hidden {self.d_model}, "
                  f"{self.n_layers} layers, heads {self.n_heads} (KV {self.n_kv_heads}), FFN {self.d_ff}")

    # -- embeddings: device bf16, exposed as float32 NumPy like the reference attribute ------
    @property
    def embed_tokens(self):
        return self._embed.float().cpu().numpy()

    @embed_tokens.setter
    def embed_tokens(self, value):
        torch = abi.require_cuda()
        t = value if hasattr(value, "data_ptr") else torch.from_numpy(np.ascontiguousarray(value))
        if tuple(t.shape) != (self.vocab_size, self.d_model):
            raise ValueError(f"embedding shape {tuple(t.shape)} != {(self.vocab_size, self.d_model)}")
        self._embed.copy_(t.to(torch.bfloat16))

    # -- loader --------------------------------------------------------------------------
    def load_weights_from_safetensors(self, model_path: str):
        """Same tensor names as the reference loader (src/rotor/bitnet_model.py:105-185)."""
        import torch
        from safetensors import safe_open
        with safe_open(model_path, framework="pt") as f:
            self.embed_tokens = f.get_tensor("model.embed_tokens.weight")
            self.norm.weight = f.get_tensor("model.norm.weight").float().numpy()
            for i, layer in enumerate(self.layers):
                pre = f"model.layers.{i}"
                getn = lambda name: f.get_tensor(name).float().numpy()
                layer.input_norm.weight = getn(f"{pre}.input_layernorm.weight")
                layer.post_attn_norm.weight = getn(f"{pre}.post_attention_layernorm.weight")
                layer.attention.attn_norm.weight = getn(f"{pre}.self_attn.attn_sub_norm.weight")
                layer.ffn.ffn_norm.weight = getn(f"{pre}.mlp.ffn_sub_norm.weight")
                for proj, name in ((layer.attention.q_proj, "self_attn.q_proj"),
                                   (layer.attention.k_proj, "self_attn.k_proj"),
                                   (layer.attention.v_proj, "self_attn.v_proj"),
                                   (layer.attention.o_proj, "self_attn.o_proj"),
                                   (layer.ffn.gate_proj, "mlp.gate_proj"), (layer.ffn.up_proj, "mlp.up_proj"),
                                   (layer.ffn.down_proj, "mlp.down_proj")):
                    packed = f.get_tensor(f"{pre}.{name}.weight")
                    scale = f.get_tensor(f"{pre}.{name}.weight_scale").float().item()
                    proj.load_from_bitnet(packed, scale)
        self._handle = None

    # -- handle management ---------------------------------------------------------------
    def _norm_state(self):
        st = [id(self.norm._weight)]
        for l in self.layers:
            st += [id(l.input_norm._weight), id(l.post_attn_norm._weight), id(l.attention.attn_norm._weight),
                   id(l.ffn.ffn_norm._weight)]
            st += [p.scale for p in (l.attention.q_proj, l.attention.k_proj, l.attention.v_proj, l.attention.o_proj,
                                     l.ffn.gate_proj, l.ffn.up_proj, l.ffn.down_proj)]
        return st

    def _ensure_handle(self, batch=1, seq=1, total=1):
        state = self._norm_state()
        grow = self._handle is not None and (batch > self._handle.cfg.max_batch or total > self._handle.cfg.max_seq
                                             or batch * seq > self._handle.cfg.max_rows)
        if self._handle is None or state != self._norm_versions or grow:
            self.max_batch = max(self.max_batch, batch)
            self.max_seq = max(self.max_seq, total)
            self.max_rows = max(self.max_rows, batch * seq)
            self._handle = None
            self._handle = _Handle(self.layers, self._embed, self.norm.device_weight(), self.vocab_size,
                                   self.semantics, self.max_batch, self.max_seq, self.max_rows)
            self._norm_versions = state
        return self._handle

    # -- forward ---------------------------------------------------------------------------
    def forward(self, input_ids: np.ndarray, return_logits: bool = True, past_kv_cache: Optional[list] = None,
                use_cache: bool = False, logits_positions: str = "all"):
        """Reference src/rotor/bitnet_model.py:190-244.  ``logits_positions='last'`` returns
        logits of the last position only, shaped [batch, 1, vocab]."""
        torch = abi.require_cuda()
        ids = np.asarray(input_ids)
        squeeze = ids.ndim == 1
        if squeeze:
            ids = ids[None, :]
        batch, seq = ids.shape
        past = 0 if past_kv_cache is None else past_kv_cache[0].length
        h = self._ensure_handle(batch, seq, past + seq)
        ids_d = ops.to_device(ids.astype(np.int64))
        if return_logits:
            allpos = logits_positions == "all"
            npos = seq if allpos else 1
            logits = torch.empty((batch, npos, self.vocab_size), dtype=torch.float32, device="cuda")
            check(lib.rotor_b200_model_forward(h.h, ptr(ids_d), batch, seq, past,
                                               abi.LOGITS_ALL if allpos else abi.LOGITS_LAST, ptr(logits), None,
                                               abi.stream()), "model_forward")
            out = logits.cpu().numpy()
        else:
            emb = self._embed[ids_d.reshape(-1)].float().contiguous()
            hid = torch.empty_like(emb)
            check(lib.rotor_b200_model_forward_hidden(h.h, ptr(emb), batch, seq, past, 0, self.n_layers, 1,
                                                      ptr(hid), abi.stream()), "model_forward_hidden")
            out = hid.cpu().numpy().reshape(batch, seq, self.d_model)
        abi.device_status()
        if squeeze:
            out = out[0]
        caches = [KVCache(l.attention, past + seq, batch) for l in self.layers] if use_cache else None
        return out, caches

    def forward_last_logits_device(self, input_ids, past_kv_cache=None):
        """Like ``forward(..., use_cache=True, logits_positions='last')`` but the logits stay on the
        device: returns (CUDA float32 [batch, vocab], caches)."""
        torch = abi.require_cuda()
        ids = np.asarray(input_ids)
        if ids.ndim == 1:
            ids = ids[None, :]
        batch, seq = ids.shape
        past = 0 if past_kv_cache is None else past_kv_cache[0].length
        h = self._ensure_handle(batch, seq, past + seq)
        ids_d = ops.to_device(ids.astype(np.int64))
        logits = torch.empty((batch, self.vocab_size), dtype=torch.float32, device="cuda")
        check(lib.rotor_b200_model_forward(h.h, ptr(ids_d), batch, seq, past, abi.LOGITS_LAST, ptr(logits), None,
                                           abi.stream()), "model_forward")
        return logits, [KVCache(l.attention, past + seq, batch) for l in self.layers]

    # -- device-resident greedy generation ---------------------------------------------------
    def greedy_chunks(self, prompt_ids, max_new_tokens: int, use_graph: bool = True, chunk: int = 0):
        """Generator over lists of new token ids.  The prompt is prefilled once; every later
        step is a one-token forward whose greedy pick feeds the next step on the device.
        ``chunk`` > 0 hands tokens back every ``chunk`` steps (the first list holds the token
        picked after the prompt); 0 hands everything back at the end.  Stop iterating to stop
        generating."""
        torch = abi.require_cuda()
        prompt = np.asarray(prompt_ids, dtype=np.int64).reshape(1, -1)
        n_prompt = prompt.shape[1]
        if max_new_tokens <= 0:
            return
        h = self._ensure_handle(1, n_prompt, n_prompt + max_new_tokens)
        ids_d = ops.to_device(prompt)
        first = torch.empty(1, dtype=torch.int64, device="cuda")
        stream = torch.cuda.current_stream()
        if use_graph and stream.cuda_stream == 0:
            stream = self._side_stream()   # the legacy default stream cannot be captured
        s = stream.cuda_stream
        with torch.cuda.stream(stream):
            check(lib.rotor_b200_model_forward(h.h, ptr(ids_d), 1, n_prompt, 0, abi.LOGITS_NONE, None, ptr(first), s),
                  "prefill")
            first_host = [int(first.cpu()[0])]
        remaining = max_new_tokens - 1
        if chunk > 0 or remaining == 0:
            yield first_host
            first_host = []
        if remaining > 0:
            check(lib.rotor_b200_model_decode_begin(h.h, ptr(first), 1, n_prompt, s), "decode_begin")
            step = chunk if chunk > 0 else remaining
            buf = np.empty(step, dtype=np.int64)
            # The steps feed one another on the device, so the next chunk is launched BEFORE the current
            # one's tokens are read: the read goes through a second stream that waits for the chunk's own
            # event, and the device never idles for the host round trip.  A consumer that stops iterating
            # (EOS) leaves at most one chunk of surplus steps, which the close below waits out.
            copier = self._copy_stream()

            def launch(first_step):
                n = min(step, remaining - first_step)
                with torch.cuda.stream(stream):
                    check(lib.rotor_b200_model_decode_steps(h.h, n, int(use_graph), s), "decode_steps")
                    done_ev = torch.cuda.Event()
                    done_ev.record(stream)
                return first_step, n, done_ev

            try:
                queue = [launch(0)]
                launched = queue[0][1]
                while queue:
                    start, n, done_ev = queue.pop(0)
                    if launched < remaining:
                        queue.append(launch(launched))
                        launched += queue[-1][1]
                    copier.wait_event(done_ev)
                    check(lib.rotor_b200_model_read_tokens(h.h, start, n, buf.ctypes.data, copier.cuda_stream),
                          "read_tokens")
                    yield first_host + [int(t) for t in buf[:n]]
                    first_host = []
            finally:
                stream.synchronize()   # nothing of this generation is in flight when the handle is used again
        abi.device_status()

    def generate_greedy(self, prompt_ids, max_new_tokens: int, use_graph: bool = True, chunk: int = 0):
        """All new token ids of a device-resident greedy generation."""
        out = []
        for new in self.greedy_chunks(prompt_ids, max_new_tokens, use_graph, chunk):
            out += new
        return out

    def generate_greedy_batch(self, prompt_ids, max_new_tokens: int, use_graph: bool = True):
        """Device-resident greedy generation for a batch of prompts: one prefill, then every step
        advances all sequences at once.  ``prompt_ids`` is [batch, prompt_len] or a list of
        prompts of different lengths; those are right-padded for the prefill (a causal model
        never attends to the padding behind a token) and every sequence then continues from
        its own length.  Returns int64 [batch, max_new_tokens], row b holding what a
        single-prompt generation from prompt b gives."""
        torch = abi.require_cuda()
        rows = [np.asarray(p, dtype=np.int64).reshape(-1) for p in prompt_ids]
        batch = len(rows)
        if batch == 0:
            return np.zeros((0, max(max_new_tokens, 0)), dtype=np.int64)
        lens = np.array([len(r) for r in rows], dtype=np.int32)
        if lens.min() < 1:
            raise ValueError("every prompt needs at least one token")
        n_prompt = int(lens.max())
        ragged = bool((lens != n_prompt).any())
        if ragged and not self.semantics.causal:
            raise ValueError("prompts of different lengths need a causal model")
        prompts = np.zeros((batch, n_prompt), dtype=np.int64)
        for b, r in enumerate(rows):
            prompts[b, :len(r)] = r
        if max_new_tokens <= 0:
            return np.zeros((batch, 0), dtype=np.int64)
        h = self._ensure_handle(batch, n_prompt, n_prompt + max_new_tokens)
        ids_d = ops.to_device(prompts)
        first = torch.empty(batch, dtype=torch.int64, device="cuda")
        stream = torch.cuda.current_stream()
        if use_graph and stream.cuda_stream == 0:
            stream = self._side_stream()
        s = stream.cuda_stream
        out = np.empty((batch, max_new_tokens), dtype=np.int64)
        with torch.cuda.stream(stream):
            if ragged:
                check(lib.rotor_b200_model_forward_ragged(h.h, ptr(ids_d), batch, n_prompt, lens.ctypes.data,
                                                          abi.LOGITS_NONE, None, ptr(first), s), "prefill")
            else:
                check(lib.rotor_b200_model_forward(h.h, ptr(ids_d), batch, n_prompt, 0, abi.LOGITS_NONE, None,
                                                   ptr(first), s), "prefill")
            out[:, 0] = first.cpu().numpy()
            remaining = max_new_tokens - 1
            if remaining > 0:
                if ragged:
                    check(lib.rotor_b200_model_decode_begin_ragged(h.h, ptr(first), batch, lens.ctypes.data, s),
                          "decode_begin")
                else:
                    check(lib.rotor_b200_model_decode_begin(h.h, ptr(first), batch, n_prompt, s), "decode_begin")
                check(lib.rotor_b200_model_decode_steps(h.h, remaining, int(use_graph), s), "decode_steps")
                buf = np.empty((remaining, batch), dtype=np.int64)   # the token log is [step][sequence]
                check(lib.rotor_b200_model_read_tokens(h.h, 0, remaining, buf.ctypes.data, s), "read_tokens")
                out[:, 1:] = buf.T
        abi.device_status()
        return out

    def _copy_stream(self):
        torch = abi.require_cuda()
        if getattr(self, "_copier", None) is None:
            self._copier = torch.cuda.Stream()
        return self._copier

    def _side_stream(self):
        torch = abi.require_cuda()
        if getattr(self, "_stream", None) is None:
            self._stream = torch.cuda.Stream()
        self._stream.wait_stream(torch.cuda.current_stream())
        return self._stream


class _SoloBlockRunner:
    """Runs one TransformerBlock through a one-layer model handle (stand-alone block calls)."""

    def __init__(self, block: TransformerBlock):
        self.block = block
        self.handle = None
        self.key = None

    def forward(self, x, mask, kv_cache, use_cache):
        torch = abi.require_cuda()
        blk = self.block
        x = np.asarray(x)
        is_3d = x.ndim == 3
        if not is_3d:
            x = x[None, ...]
        batch, seq, d = x.shape
        past = 0 if kv_cache is None else kv_cache.length
        sem = blk.semantics
        if mask is not None:
            sem = _semantics_for_mask(sem, mask, seq, past + seq)
        att = blk.attention
        key = (sem, id(blk.input_norm._weight), id(blk.post_attn_norm._weight), id(att.attn_norm._weight),
               id(blk.ffn.ffn_norm._weight))
        cap_ok = self.handle is not None and batch <= self.handle.cfg.max_batch and \
            past + seq <= self.handle.cfg.max_seq and batch * seq <= self.handle.cfg.max_rows
        if self.handle is None or key != self.key or not cap_ok:
            torch_dummy = torch.zeros((1, d), dtype=torch.bfloat16, device="cuda")
            ones = torch.ones(d, dtype=torch.float32, device="cuda")
            self.handle = None
            self.handle = _Handle([blk], torch_dummy, ones, 1, sem, max(batch, att.max_batch),
                                  max(past + seq, att.max_seq), max(batch * seq, 64))
            self.key = key
        xd = ops.to_device(x.reshape(batch * seq, d), torch.float32)
        y = torch.empty_like(xd)
        check(lib.rotor_b200_model_forward_hidden(self.handle.h, ptr(xd), batch, seq, past, 0, 1, 0, ptr(y),
                                                  abi.stream()), "block forward")
        out = y.cpu().numpy().reshape(batch, seq, d)
        if not is_3d:
            out = out[0]
        return out, (KVCache(att, past + seq, batch) if use_cache else None)


def load_bitnet_model(model_dir: str, use_gpu: bool = True, *, semantics: Semantics = REFERENCE,
                      max_seq: int = 2048, max_batch: int = 1, verbose: bool = False) -> BitNetModel:
    """Reference src/rotor/bitnet_model.py:349-394: config.json (HF key names) +
    model.safetensors in ``model_dir``."""
    _require_gpu_flag(use_gpu)
    model_dir = Path(model_dir)
    with open(model_dir / "config.json", "r") as f:
        config = json.load(f)
    model_config = {
        'vocab_size': config['vocab_size'],
        'd_model': config['hidden_size'],
        'n_layers': config['num_hidden_layers'],
        'n_heads': config['num_attention_heads'],
        'n_kv_heads': config.get('num_key_value_heads', config['num_attention_heads']),
        'd_ff': config['intermediate_size'],
    }
    model = BitNetModel(model_config, use_gpu=True, semantics=semantics, max_seq=max_seq, max_batch=max_batch,
                        verbose=verbose)
    model.load_weights_from_safetensors(str(model_dir / "model.safetensors"))
    return model
