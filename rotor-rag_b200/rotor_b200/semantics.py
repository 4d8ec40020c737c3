"""Numeric contract switches of the path.

``REFERENCE`` reproduces what the reference code computes when it runs
(src/rotor/transformer.py): floating-point activations (here: three-term int8
residual quantisation, which is float32-faithful), gate * silu(clip(up, +-20)),
no positional encoding, no attention mask, eps 1e-6.

``BASELINE`` is the published BitNet-b1.58 description: one-term per-token absmax
int8 activations with exact int32 accumulation, relu(gate)^2 * up, rotary embedding
(theta 5e5), causal mask, eps 1e-5.
"""
from __future__ import annotations

from dataclasses import dataclass, replace
from typing import Optional


@dataclass(frozen=True)
class Semantics:
    act_terms: int = 3
    ffn_act: str = "silu_clip20"      # or "relu2"
    rope_theta: Optional[float] = None
    causal: bool = False
    eps: float = 1e-6
    gemv_variant: int = 0             # abi.VARIANT_*

    def with_(self, **kw) -> "Semantics":
        return replace(self, **kw)


REFERENCE = Semantics()
BASELINE = Semantics(act_terms=1, ffn_act="relu2", rope_theta=500000.0, causal=True, eps=1e-5)
