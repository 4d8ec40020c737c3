#!/usr/bin/env python
"""Regenerates the fixtures in this directory from the unmodified reference.

Run on a machine that has a checkout of BikerSam86/rotor-RAG:

    make -C oracle all _ref
    python tests/golden/make_golden.py [--ref /path/to/rotor-RAG]

The script imports the reference's own Python modules (read-only), hands its
loader the reference C library built by ``oracle/Makefile`` (target ``_ref``),
runs the reference on seeded inputs, checks this repo's NumPy oracle against
every result, and only then writes the ``.npz`` fixtures.  Inputs are never
stored: each fixture keeps the seed, and ``tests/golden_inputs.py`` rebuilds
the inputs from it, so the fixtures stay a few hundred KB.
"""
import argparse
import contextlib
import ctypes
import io
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

from oracle import bitlinear_np as O  # noqa: E402
import golden_inputs as G  # noqa: E402


def load_reference(ref_root):
    sys.path.insert(0, os.path.join(ref_root, "src"))
    import rotor.bitnet_fast as bf
    lib = os.path.join(ROOT, "oracle", "_ref", "librotor_core.so")
    bf._lib = ctypes.CDLL(lib)  # the stock search path is inside the read-only checkout
    assert bf.is_c_library_available()
    import rotor.transformer as tr
    import rotor.bitnet_model as bm
    import rotor.generation as gen
    import rotor.core as core
    import rotor.quantization as qz
    return bf, tr, bm, gen, core, qz


def quiet(fn, *a, **k):
    with contextlib.redirect_stdout(io.StringIO()):
        return fn(*a, **k)


def ref_linear(tr, w, scale):
    out, inn = w.shape
    lin = tr.TernaryLinear(inn, out)
    quiet(lin.load_from_bitnet, O.pack_ternary_matrix(w), scale)
    return lin


def ref_model(bm, om):
    """Reference BitNetModel filled from an oracle parameter dict through the reference's
    own load_from_bitnet (the pattern of examples/test_kv_cache.py:44-58)."""
    cfg = om["cfg"]
    model = quiet(bm.BitNetModel, cfg)
    model.embed_tokens = om["embed"].copy()
    model.norm.weight = om["norm"].copy()
    for layer, lw in zip(model.layers, om["layers"]):
        layer.input_norm.weight = lw["input_norm"].copy()
        layer.post_attn_norm.weight = lw["post_attn_norm"].copy()
        layer.attention.attn_norm.weight = lw["attn_sub_norm"].copy()
        layer.ffn.ffn_norm.weight = lw["ffn_sub_norm"].copy()
        for name, proj in (("q", layer.attention.q_proj), ("k", layer.attention.k_proj),
                           ("v", layer.attention.v_proj), ("o", layer.attention.o_proj),
                           ("gate", layer.ffn.gate_proj), ("up", layer.ffn.up_proj),
                           ("down", layer.ffn.down_proj)):
            w, sc = lw[name]
            quiet(proj.load_from_bitnet, O.pack_ternary_matrix(w), sc)
            assert np.array_equal(proj.weights_cache, w)
    return model


def rel_err(a, b):
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    return float(np.max(np.abs(a - b)) / (np.sqrt(np.mean(b ** 2)) + 1e-300))


class PassTokenizer:
    """ids as space-separated integers; the three members TextGenerator uses."""
    eos_token_id = -1

    def encode(self, text, add_special_tokens=True, return_numpy=True):
        return np.array([int(t) for t in text.split()], dtype=np.int64)

    def decode(self, ids, skip_special_tokens=True):
        return " ".join(str(int(t)) for t in ids)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", default=os.environ.get("ROTOR_RAG_REF"), required="ROTOR_RAG_REF" not in os.environ,
                    help="checkout of the reference (default: $ROTOR_RAG_REF)")
    ap.add_argument("--check-only", action="store_true", help="run every oracle-vs-reference check, write nothing")
    args = ap.parse_args()
    if args.check_only:
        np.savez_compressed = lambda *a, **k: None
    bf, tr, bm, gen, core, qz = load_reference(args.ref)
    report = []

    # ---------------------------------------------------------------- format
    w = G.format_matrix()
    packed = O.pack_ternary_matrix(w)
    p_ref, m_ref = bf.bitnet_to_rotor_fast(packed)
    w_ref = bf.rotor_unpack_weights_fast(p_ref, m_ref, *w.shape)
    assert np.array_equal(w_ref, w)
    p_o, m_o = O.packed_to_planes(packed)
    assert np.array_equal(p_o, p_ref) and np.array_equal(m_o, m_ref)
    assert np.array_equal(O.planes_to_int8(p_o, m_o, *w.shape), w_ref)
    # reserved field 0b11 and ragged column counts
    rng = np.random.default_rng(G.SEED_FORMAT + 1)
    raw = rng.integers(0, 256, size=(5, 9), dtype=np.uint8)   # all four field values occur
    p_raw, m_raw = bf.bitnet_to_rotor_fast(raw)
    w_raw = bf.rotor_unpack_weights_fast(p_raw, m_raw, 5, 36)
    assert np.array_equal(O.packed_to_planes(raw)[0], p_raw)
    assert np.array_equal(O.packed_to_int8(raw), w_raw)
    # 1-D pack/unpack (RotorCore) on a seeded vector
    v = rng.integers(-1, 2, size=64).astype(np.int8)
    b0, b1 = core.RotorCore.encode(v)
    pk = core.RotorCore.pack(b0, b1)
    assert np.array_equal(O.pack(*O.encode(v)), pk)
    u0, u1 = core.RotorCore.unpack(pk, 64)
    assert np.array_equal(O.unpack(pk, 64)[0], u0) and np.array_equal(O.unpack(pk, 64)[1], u1)
    np.savez_compressed(os.path.join(HERE, "format.npz"),
                        plus=p_ref, minus=m_ref, weights=w_ref,
                        raw_packed=raw, raw_plus=p_raw, raw_minus=m_raw, raw_weights=w_raw,
                        vec=v, vec_packed=pk)
    report.append("format: planes/int8/pack bit-exact vs reference")

    # ------------------------------------------------------------ quantiser
    xq = G.quant_inputs()
    q_ref, s_ref = zip(*[qz.quantize_activations(r) for r in xq])
    q_o, s_o = O.quantize_rows(xq, 1)
    assert np.array_equal(np.stack(q_ref), q_o[:, 0, :])
    assert np.array_equal(np.asarray(s_ref, dtype=np.float32), s_o[:, 0])
    np.savez_compressed(os.path.join(HERE, "quantize.npz"), q=np.stack(q_ref),
                        s=np.asarray(s_ref, dtype=np.float32))
    report.append("quantize_activations per row: bit-exact vs reference")

    # -------------------------------------------------- BitLinear, config 1
    w, scale, x1, x16 = G.bitlinear_case()
    lin = ref_linear(tr, w, scale)
    y1 = lin.forward(x1)
    y16 = lin.forward(x16)
    assert np.array_equal(O.bitlinear_float(x1, w, scale), y1)
    e3 = rel_err(O.bitlinear_int(x1, w, scale, 3)[0], y1)
    e1 = rel_err(O.bitlinear_int(x1, w, scale, 1)[0], y1)
    np.savez_compressed(os.path.join(HERE, "bitlinear_2560x6912.npz"), y1=y1, y16=y16)
    report.append(f"bitlinear 2560->6912: float oracle bit-exact; 3-term int8 {e3:.2e}, 1-term {e1:.2e} of RMS")

    # small ragged layer (out and in not multiples of the GPU tile)
    ws, ss, xs = G.small_linear_case()
    lin_s = ref_linear(tr, ws, ss)
    ys = lin_s.forward(xs)
    assert np.array_equal(O.bitlinear_float(xs, ws, ss), ys)
    np.savez_compressed(os.path.join(HERE, "bitlinear_small.npz"), y=ys)

    # ------------------------------------------------- FFN block, config 2 shape
    lw, xf1, xf16 = G.ffn_case()
    ffn = tr.GatedFFN(2560, 6912)
    norm = tr.RMSNorm(2560)
    norm.weight = lw["post_attn_norm"]
    ffn.ffn_norm.weight = lw["ffn_sub_norm"]
    for nm, proj in (("gate", ffn.gate_proj), ("up", ffn.up_proj), ("down", ffn.down_proj)):
        quiet(proj.load_from_bitnet, O.pack_ternary_matrix(lw[nm][0]), lw[nm][1])
    outs = {}
    for tag, xin in (("m1", xf1), ("m16", xf16)):
        yr = ffn.forward(norm.forward(xin))
        yo = O.ffn(O.rmsnorm(xin, lw["post_attn_norm"], 1e-6), lw, O.REFERENCE)
        assert rel_err(yo, yr) < 1e-6, rel_err(yo, yr)
        outs[tag] = yr
    np.savez_compressed(os.path.join(HERE, "ffn_block.npz"), **outs)
    report.append("ffn block 2560/6912 (reference semantics): oracle within 1e-6 of reference")

    # ---------------------------------------------------------- tiny models
    for name in G.TINY_MODELS:
        om, prompt = G.tiny_model(name)
        rm = ref_model(bm, om)
        logits_ref, caches_ref = rm.forward(prompt[None, :], use_cache=True)
        logits_o, caches_o = O.model_forward(om, prompt[None, :], O.REFERENCE, use_cache=True)
        assert logits_ref.dtype == logits_o.dtype, (logits_ref.dtype, logits_o.dtype)
        assert rel_err(logits_o, logits_ref) < 1e-9, rel_err(logits_o, logits_ref)
        assert rel_err(caches_o[-1]["k"], caches_ref[-1]["k"]) < 1e-9
        # cached greedy generation through the reference's own TextGenerator
        tg = gen.TextGenerator(rm, PassTokenizer(), max_length=len(prompt) + G.N_NEW, use_cache=True)
        text = tg.generate(" ".join(map(str, prompt)), max_new_tokens=G.N_NEW, stop_on_eos=False)
        ids_ref = [int(t) for t in text.split()]
        ids_o, step_logits = O.generate_greedy(om, prompt, G.N_NEW, O.REFERENCE, return_logits=True)
        assert ids_o == ids_ref, (ids_o, ids_ref)
        # causal variant through the reference's own mask plumbing (transformer.py:270-271, 386-403)
        h = rm.embed_tokens[prompt[None, :]]
        mask = O.causal_mask(len(prompt), len(prompt))
        for layer in rm.layers:
            h, _ = layer.forward(h, mask=mask)
        logits_causal = np.dot(rm.norm.forward(h), rm.embed_tokens.T)
        lo_c, _ = O.model_forward(om, prompt[None, :], O.with_semantics(O.REFERENCE, causal=True))
        assert rel_err(lo_c, logits_causal) < 1e-9
        step_logits = np.stack(step_logits)
        srt = np.sort(step_logits, axis=1)
        margin = (srt[:, -1] - srt[:, -2]) / np.sqrt(np.mean(step_logits ** 2, axis=1))
        np.savez_compressed(os.path.join(HERE, f"model_{name}.npz"),
                            prompt_logits=logits_ref[0].astype(np.float64),
                            prompt_logits_causal=logits_causal[0].astype(np.float64),
                            last_k=caches_ref[-1]["k"].astype(np.float64),
                            greedy_ids=np.asarray(ids_ref, dtype=np.int64),
                            step_logits=step_logits.astype(np.float64),
                            top2_margin=margin)
        report.append(f"model {name}: oracle logits within 1e-9, greedy ids identical "
                      f"({G.N_NEW} tokens, min top-2 margin {margin.min():.2e} of RMS)")

    # --- sampling: the set the reference's strategies draw from and its probabilities, read off the
    # reference's own code by standing in for np.random.choice (generation.py:78-80, 135-137)
    from oracle import sampling_np as S
    logits = G.sampling_logits()
    fx = {}
    for ci, (mode, k, p, temp) in enumerate(G.SAMPLING_CASES):
        strat = gen.TopKSampling(k) if mode == 0 else gen.TopPSampling(p)
        seen = {}
        real_choice = np.random.choice
        try:
            state = {"j": 0}

            def fake_choice(n, p=None):
                seen["n"], seen["p"] = n, np.array(p, dtype=np.float64)
                return state["j"]
            np.random.choice = fake_choice
            strat.sample(logits.copy(), temp)
            toks = []
            for j in range(seen["n"]):
                state["j"] = j
                toks.append(strat.sample(logits.copy(), temp))
        finally:
            np.random.choice = real_choice
        toks = np.asarray(toks, dtype=np.int64)
        order = np.argsort(toks)
        ref_idx, ref_p = toks[order], seen["p"][order]
        idx, pr = S.kept_set(logits, mode, k, p, temp)
        assert np.array_equal(idx, ref_idx), (ci, len(idx), len(ref_idx))
        assert np.max(np.abs(pr - ref_p)) < 1e-6
        fx[f"idx{ci}"], fx[f"p{ci}"] = ref_idx, ref_p
    np.savez_compressed(os.path.join(HERE, "sampling.npz"), **fx)
    report.append(f"sampling: kept sets and probabilities of {len(G.SAMPLING_CASES)} top-k / top-p cases identical")

    print("\n".join(report))


if __name__ == "__main__":
    main()
