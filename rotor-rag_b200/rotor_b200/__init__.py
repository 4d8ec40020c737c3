"""B200-native ternary BitLinear decode path behind the rotor-RAG Python API.

Modules mirror the reference's layout for this path:
``transformer`` (RMSNorm, TernaryLinear, MultiHeadAttention, GatedFFN,
TransformerBlock), ``bitnet_model`` (BitNetModel, load_bitnet_model),
``generation`` (sampling strategies, TextGenerator), ``gpu_layers`` (get_gpu),
on top of ``abi`` (ctypes binding of librotor_b200.so) and ``ops`` (tensor-level
wrappers).  Importing the package loads the CUDA library and raises if it is
missing.
"""
from . import abi  # noqa: F401  (fails loudly when librotor_b200.so is absent)

__all__ = ["abi"]
