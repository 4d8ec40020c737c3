"""Synthetic, seeded parameters for the path: random-init models of the BitNet-b1.58 layout
on the device, a pass-through tokenizer, and a checkpoint writer that produces the
config.json + model.safetensors pair ``load_bitnet_model`` reads (tensor names as in the
reference loader, src/rotor/bitnet_model.py:105-185)."""
from __future__ import annotations

import json
import os

import numpy as np

from . import abi
from .bitnet_model import BitNetModel
from .semantics import REFERENCE, Semantics

SYNTH_SCALE = 0.015955  # mean |N(0, 0.02)|

BITNET_2B = dict(vocab_size=128256, d_model=2560, n_layers=30, n_heads=20, n_kv_heads=5, d_ff=6912)
XL_TP = dict(vocab_size=128256, d_model=8192, n_layers=80, n_heads=64, n_kv_heads=8, d_ff=28672)


class PassThroughTokenizer:
    """Token ids as space-separated integers; the three members TextGenerator uses
    (encode / decode / eos_token_id, reference src/rotor/generation.py:205,228,241)."""

    def __init__(self, eos_token_id=-1):
        self.eos_token_id = eos_token_id

    def encode(self, text, add_special_tokens=True, return_numpy=True):
        ids = np.array([int(t) for t in text.split()], dtype=np.int64)
        return ids if return_numpy else ids.tolist()

    def decode(self, ids, skip_special_tokens=True):
        return " ".join(str(int(t)) for t in np.asarray(ids).reshape(-1))


def random_model_on_device(cfg, seed=0, semantics: Semantics = REFERENCE, **kw) -> BitNetModel:
    """Random-init model generated on the GPU: ternary weights uniform over {-1,0,+1},
    per-tensor scales near mean|N(0,0.02)|, bf16 N(0,0.02) embeddings, unit norm weights."""
    torch = abi.require_cuda()
    g = torch.Generator(device="cuda")
    g.manual_seed(seed)
    model = BitNetModel(cfg, use_gpu=True, semantics=semantics, **kw)
    model._embed.copy_((0.02 * torch.randn(model._embed.shape, generator=g, device="cuda")).to(torch.bfloat16))
    rs = np.random.default_rng(seed)
    for layer in model.layers:
        a, f = layer.attention, layer.ffn
        for proj in (a.q_proj, a.k_proj, a.v_proj, a.o_proj, f.gate_proj, f.up_proj, f.down_proj):
            w = torch.randint(-1, 2, (proj.out_features, proj.in_features), generator=g, device="cuda",
                              dtype=torch.int8)
            proj.load_from_int8(w, SYNTH_SCALE * (1.0 + 0.25 * rs.random()))
    return model


def model_from_oracle_params(params, semantics: Semantics = REFERENCE, **kw) -> BitNetModel:
    """Build the GPU model from an oracle-style parameter dict (host NumPy), going through
    the same packed uint8 bytes and load_from_bitnet call the reference uses."""
    from .hostpack import pack_ternary_matrix
    model = BitNetModel(params["cfg"], use_gpu=True, semantics=semantics, **kw)
    model.embed_tokens = params["embed"]
    model.norm.weight = params["norm"]
    for layer, lw in zip(model.layers, params["layers"]):
        layer.input_norm.weight = lw["input_norm"]
        layer.post_attn_norm.weight = lw["post_attn_norm"]
        layer.attention.attn_norm.weight = lw["attn_sub_norm"]
        layer.ffn.ffn_norm.weight = lw["ffn_sub_norm"]
        a, f = layer.attention, layer.ffn
        for name, proj in (("q", a.q_proj), ("k", a.k_proj), ("v", a.v_proj), ("o", a.o_proj),
                           ("gate", f.gate_proj), ("up", f.up_proj), ("down", f.down_proj)):
            w, sc = lw[name]
            proj.load_from_bitnet(pack_ternary_matrix(w), sc)
    return model


def write_checkpoint(params, directory):
    """config.json (HF key names) + model.safetensors with the reference's tensor names."""
    import torch
    from safetensors.torch import save_file
    from .hostpack import pack_ternary_matrix
    os.makedirs(directory, exist_ok=True)
    cfg = params["cfg"]
    with open(os.path.join(directory, "config.json"), "w") as f:
        json.dump({"vocab_size": cfg["vocab_size"], "hidden_size": cfg["d_model"],
                   "num_hidden_layers": cfg["n_layers"], "num_attention_heads": cfg["n_heads"],
                   "num_key_value_heads": cfg["n_kv_heads"], "intermediate_size": cfg["d_ff"]}, f)
    t = {"model.embed_tokens.weight": torch.from_numpy(params["embed"]).to(torch.bfloat16),
         "model.norm.weight": torch.from_numpy(params["norm"]).to(torch.bfloat16)}
    names = {"q": "self_attn.q_proj", "k": "self_attn.k_proj", "v": "self_attn.v_proj", "o": "self_attn.o_proj",
             "gate": "mlp.gate_proj", "up": "mlp.up_proj", "down": "mlp.down_proj"}
    for i, lw in enumerate(params["layers"]):
        pre = f"model.layers.{i}"
        t[f"{pre}.input_layernorm.weight"] = torch.from_numpy(lw["input_norm"]).to(torch.bfloat16)
        t[f"{pre}.post_attention_layernorm.weight"] = torch.from_numpy(lw["post_attn_norm"]).to(torch.bfloat16)
        t[f"{pre}.self_attn.attn_sub_norm.weight"] = torch.from_numpy(lw["attn_sub_norm"]).to(torch.bfloat16)
        t[f"{pre}.mlp.ffn_sub_norm.weight"] = torch.from_numpy(lw["ffn_sub_norm"]).to(torch.bfloat16)
        for k, nm in names.items():
            w, sc = lw[k]
            t[f"{pre}.{nm}.weight"] = torch.from_numpy(pack_ternary_matrix(w))
            t[f"{pre}.{nm}.weight_scale"] = torch.tensor([sc], dtype=torch.float32)
    save_file(t, os.path.join(directory, "model.safetensors"))
