"""Seeded inputs behind the fixtures in tests/golden/.

The fixtures store only what the reference produced; the inputs are rebuilt
here from fixed seeds (NumPy's PCG64 stream is stable across releases), both
when the fixtures are generated and when the tests replay them.
"""
import numpy as np

from oracle import bitlinear_np as O

SEED_FORMAT = 42
SEED_QUANT = 7
SEED_LINEAR = 1234
SEED_SMALL = 99
SEED_FFN = 2025
N_NEW = 32

TINY_MODELS = {
    # head_dim 128 with grouped KV heads, like the 2B shape in miniature
    "hd128": dict(cfg=dict(vocab_size=1024, d_model=512, n_layers=3, n_heads=4, n_kv_heads=2, d_ff=1152),
                  seed=31337, prompt_len=8),
    # head_dim 64, 4 query heads per KV head
    "hd64": dict(cfg=dict(vocab_size=768, d_model=256, n_layers=2, n_heads=4, n_kv_heads=1, d_ff=640),
                 seed=4242, prompt_len=5),
}


def format_matrix():
    """64 x 256 ternary matrix, P = (0.3, 0.4, 0.3) -- the shape of the reference's own
    round-trip self-test (src/rotor/bitnet.py:367-381)."""
    rng = np.random.default_rng(SEED_FORMAT)
    return rng.choice(np.array([-1, 0, 1], dtype=np.int8), size=(64, 256), p=[0.3, 0.4, 0.3])


def quant_inputs():
    rng = np.random.default_rng(SEED_QUANT)
    x = rng.standard_normal((6, 2560)).astype(np.float32)
    x[1] *= 37.5
    x[2] = 0.0                     # all-zero row -> scale 1.0
    x[3, :5] = [0.5, 1.5, 2.5, -0.5, -1.5]
    x[4] = np.round(x[4] * 3)      # many exact .5 ties after scaling are possible
    return x


def bitlinear_case():
    """Config 1: in 2560, out 6912; x ~ N(0,1), batch 1 and 16."""
    rng = np.random.default_rng(SEED_LINEAR)
    w = O.synth_ternary(rng, 6912, 2560)
    x1 = rng.standard_normal((1, 2560)).astype(np.float32)
    x16 = rng.standard_normal((16, 2560)).astype(np.float32)
    return w, float(O.SYNTH_SCALE), x1, x16


def small_linear_case():
    """Ragged layer: out 20, in 72 (neither a multiple of 16 rows / 128 columns)."""
    rng = np.random.default_rng(SEED_SMALL)
    w = O.synth_ternary(rng, 20, 72)
    x = rng.standard_normal((3, 72)).astype(np.float32)
    return w, 0.731, x


def ffn_case():
    """Config 2 shape: RMSNorm(2560) -> gate/up 2560->6912 -> sub-norm(6912) -> down."""
    rng = np.random.default_rng(SEED_FFN)
    lw = {
        "post_attn_norm": O.bf16_round(1.0 + 0.1 * rng.standard_normal(2560).astype(np.float32)),
        "ffn_sub_norm": O.bf16_round(1.0 + 0.1 * rng.standard_normal(6912).astype(np.float32)),
        "gate": (O.synth_ternary(rng, 6912, 2560), 0.0171),
        "up": (O.synth_ternary(rng, 6912, 2560), 0.0163),
        "down": (O.synth_ternary(rng, 2560, 6912), 0.0148),
    }
    x1 = rng.standard_normal((1, 2560)).astype(np.float32)
    x16 = rng.standard_normal((16, 2560)).astype(np.float32)
    return lw, x1, x16


# FFN wider than 8192: the down projection's input row takes the shared-memory prologue of the
# generation-step kernels (no fixture from the reference: checked against the oracle only)
EXTRA_MODELS = {
    "wide_ffn": dict(cfg=dict(vocab_size=512, d_model=256, n_layers=2, n_heads=4, n_kv_heads=2, d_ff=9216),
                     seed=777, prompt_len=6),
    # per-rank FFN slice still wider than 8192 when split two ways
    "wide_tp": dict(cfg=dict(vocab_size=512, d_model=256, n_layers=2, n_heads=4, n_kv_heads=2, d_ff=18432),
                    seed=778, prompt_len=6),
    # four KV heads: shards four ways.  The seed is one whose one-term quantiser has no value within
    # float rounding of a .5 tie (checked by perturbing the oracle's norm sums): with one activation
    # term a single such tie moves the logits by several percent of their RMS.
    "tp4": dict(cfg=dict(vocab_size=1024, d_model=512, n_layers=2, n_heads=8, n_kv_heads=4, d_ff=2048),
                seed=9094, prompt_len=7),
}


def tiny_model(name):
    spec = TINY_MODELS.get(name) or EXTRA_MODELS[name]
    om = O.synth_model(spec["cfg"], spec["seed"])
    rng = np.random.default_rng(spec["seed"] + 1)
    prompt = rng.integers(0, spec["cfg"]["vocab_size"], size=spec["prompt_len"]).astype(np.int64)
    return om, prompt


# sampling: seeded logits with a peaked head and a long tail; (mode, k, p, temperature) cases
SAMPLING_CASES = [(0, 10, 0.0, 1.0), (0, 50, 0.0, 0.7), (0, 1, 0.0, 1.0), (1, 0, 0.9, 1.0), (1, 0, 0.5, 0.6),
                  (1, 0, 0.999, 1.3)]


def sampling_logits(vocab=2000, seed=99):
    rng = np.random.default_rng(seed)
    x = rng.standard_normal(vocab).astype(np.float32) * np.float32(1.5)
    x[rng.integers(0, vocab, size=12)] += np.float32(4.0)
    return x
