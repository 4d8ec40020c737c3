"""GPU: parity at the shapes the benchmarks run, not at toy sizes.

 * 2B dimensions (d 2560, 20 query / 5 KV heads of 128, FFN 6912, vocabulary 128256), two layers.
   In the reference's float semantics (three int8 terms on the GPU): prompt logits at every
   position within 1e-3 of the logit RMS, identical greedy tokens, and the same tokens from every
   kernel route (captured graph, eager launches, the unfused batch path).
   In published int8 semantics (one term) a value that sits on a rounding tie of the quantiser is
   decided by float summation order, and at this width a single flipped tie in the down
   projection's input (squared-ReLU gating leaves most of its int8 values at 0 or +-1) moves the
   logits by percents of their RMS: the oracle's own float32 and float64 evaluations differ that
   much at some positions.  The checks there are tie-aware: the first position (no attention sum,
   hence nothing order dependent before the quantisers) is held to 1e-3; every teacher-forced
   generation step must pick the oracle's token unless the oracle's top-2 margin at that step is
   below twice the logit error measured at that step; no position may drift beyond what flipped
   ties explain.
 * One 2B-dimension block over a 1 x 2048 causal prompt (tcgen05 GEMM, tiled attention).
 * One block of the 80-layer tensor-parallel shape (d 8192, 64 / 8 heads, FFN 28672) as a
   generation step.

Reference path: src/rotor/bitnet_model.py:190-244, src/rotor/transformer.py:206-292,
src/rotor/generation.py:220-279.
"""
import numpy as np
import pytest

from oracle import bitlinear_np as O

pytestmark = pytest.mark.gpu
TOL = 1e-3
CFG_2B2 = dict(vocab_size=128256, d_model=2560, n_layers=2, n_heads=20, n_kv_heads=5, d_ff=6912)


def per_pos_err(got, want):
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    rms = np.sqrt(np.mean(want ** 2, axis=-1))
    return np.max(np.abs(got - want), axis=-1) / rms


@pytest.fixture(scope="module")
def rbm():
    import rotor_b200.synth as synth
    from rotor_b200 import semantics
    class NS: pass
    ns = NS()
    ns.synth, ns.sem = synth, semantics
    return ns


@pytest.fixture(scope="module")
def two_layer_2b():
    om = O.synth_model(CFG_2B2, 2026, fast_embed=True)
    prompt = np.random.default_rng(2027).integers(0, CFG_2B2["vocab_size"], size=16).astype(np.int64)
    return om, prompt


TIE_DRIFT = 0.3   # error / RMS that flipped ties explain at these widths (oracle vs oracle: up to 0.15)


def _check_tie_aware(got, want32, want64, what):
    """got / want*: [positions, vocab].  Position-wise: 1e-3 where the oracle's two evaluations agree
    and the GPU shows no flipped tie either; never beyond TIE_DRIFT."""
    err = per_pos_err(got, want32)
    sens = per_pos_err(want64, want32)
    assert np.all(err < TIE_DRIFT), (what, err.tolist())
    return err, sens


def _margins(step_logits):
    out = []
    for l in step_logits:
        l = np.asarray(l, np.float64)
        top2 = np.partition(l, -2)[-2:]
        out.append(float((top2[1] - top2[0]) / np.sqrt(np.mean(l ** 2))))
    return out


def _oracle_generation(om, prompt, n_new, sem):
    ids, steps = O.generate_greedy(om, prompt, n_new, sem, return_logits=True)
    return ids[len(prompt):], steps, _margins(steps)


def test_2b_dims_published_semantics(rbm, two_layer_2b):
    om, prompt = two_layer_2b
    sem32, sem64 = O.BASELINE, O.with_semantics(O.BASELINE, glue64=True)
    model = rbm.synth.model_from_oracle_params(om, semantics=rbm.sem.BASELINE, max_seq=64)
    # ---- prompt logits at every position
    want32, _ = O.model_forward(om, prompt[None, :], sem32)
    want64, _ = O.model_forward(om, prompt[None, :], sem64)
    got, cache = model.forward(prompt[None, :], use_cache=True)
    err, sens = _check_tie_aware(got[0], want32[0], want64[0], "prompt logits")
    assert err[0] < TOL, err[0]          # one key: no order-dependent sum in front of any quantiser
    print("2B dims, int8 semantics, prompt positions: logit error / RMS", np.round(err, 5).tolist(),
          "| oracle float32 vs float64 glue", np.round(sens, 5).tolist())
    # ---- 16 teacher-forced generation steps (fused step kernels): the oracle's token goes in, logits come out
    n_new = 16
    want_ids, steps, margins = _oracle_generation(om, prompt, n_new, sem32)
    picks, errs = [int(np.argmax(got[0, -1]))], [float(err[-1])]
    for i in range(n_new - 1):
        logits, cache = model.forward(np.array([[want_ids[i]]]), past_kv_cache=cache, use_cache=True)
        e = float(per_pos_err(logits[0, -1:], np.asarray(steps[i + 1])[None])[0])
        assert e < TIE_DRIFT, (i, e)
        picks.append(int(np.argmax(logits[0, -1])))
        errs.append(e)
    for i in range(n_new):
        assert picks[i] == want_ids[i] or margins[i] < 2 * max(errs[i], TOL), (i, picks[i], want_ids[i], margins[i], errs[i])
    print("teacher-forced steps: picks equal", sum(int(a == b) for a, b in zip(picks, want_ids)), "of", n_new,
          "| step error / RMS", np.round(errs, 5).tolist(), "| oracle top-2 margin / RMS", np.round(margins, 5).tolist())
    # ---- captured graph and eager launches run the same kernels: identical tokens
    free_graph = model.generate_greedy(prompt, 12, use_graph=True)
    free_eager = model.generate_greedy(prompt, 12, use_graph=False)
    assert free_graph == free_eager
    assert free_graph[0] == picks[0]


def test_2b_dims_reference_semantics(rbm, two_layer_2b):
    om, prompt = two_layer_2b
    prompt = prompt[:8]
    model = rbm.synth.model_from_oracle_params(om, semantics=rbm.sem.REFERENCE, max_seq=32, max_batch=5)
    want, _ = O.model_forward(om, prompt[None, :], O.REFERENCE)
    got, _ = model.forward(prompt[None, :])
    err = per_pos_err(got[0], want[0])
    assert np.all(err < TOL), err.tolist()
    n_new = 12
    want_ids, steps, margins = _oracle_generation(om, prompt, n_new, O.REFERENCE)
    assert min(margins) > 2 * TOL, margins      # the fixture leaves no step undecided at the tolerance
    got_ids = model.generate_greedy(prompt, n_new, use_graph=True)
    assert got_ids == want_ids, (got_ids, want_ids)
    assert model.generate_greedy(prompt, n_new, use_graph=False) == want_ids
    # five equal sequences take the batch path (separate stage kernels, tensor-core LM head)
    batch = model.generate_greedy_batch([prompt] * 5, n_new)
    for seq in batch:
        assert [int(t) for t in seq] == want_ids
    print("2B dims, reference semantics: prompt logit error / RMS", np.round(err, 7).tolist(),
          "| smallest top-2 margin / RMS over", n_new, "steps", min(margins))


def test_2b_block_prefill_2048(rbm):
    """One block of the 2B dimensions over a 1 x 2048 causal prompt: the tcgen05 GEMM path for every
    BitLinear and the tiled attention over 2048 positions, against the oracle's block.  Strict in the
    reference's float semantics (three int8 terms leave no rounding tie to decide).  With one int8
    term the attention sum over up to 2048 keys reaches the output projection's quantiser with
    rounding noise that decides ties in most rows (half of the oracle's own positions differ between
    its float32 and float64 evaluations); there the first position is held to the tolerance and the
    rest to the spread that flipped ties explain (95th percentile against the oracle's own)."""
    cfg = dict(CFG_2B2, n_layers=1, vocab_size=256)
    om = O.synth_model(cfg, 4048)
    rng = np.random.default_rng(4049)
    x = rng.standard_normal((1, 2048, cfg["d_model"])).astype(np.float32)
    mask = O.causal_mask(2048, 2048)
    ref_sem = rbm.sem.REFERENCE.with_(causal=True)
    model = rbm.synth.model_from_oracle_params(om, semantics=ref_sem, max_seq=2048, max_rows=2048)
    want, _ = O.block(x, om["layers"][0], cfg, O.with_semantics(O.REFERENCE, causal=True))
    got, _ = model.layers[0].forward(x, mask=mask)
    err = per_pos_err(got[0], want[0])
    assert np.all(err < TOL), (float(err.max()), int(np.argmax(err)))
    print("2B block, 2048 causal positions, float semantics: max error / RMS", float(err.max()))
    del model
    model = rbm.synth.model_from_oracle_params(om, semantics=rbm.sem.BASELINE, max_seq=2048, max_rows=2048)
    want32, _ = O.block(x, om["layers"][0], cfg, O.BASELINE)
    want64, _ = O.block(x.astype(np.float64), om["layers"][0], cfg, O.BASELINE)
    got, _ = model.layers[0].forward(x, mask=mask)
    err = per_pos_err(got[0], want32[0])
    sens = per_pos_err(want64[0], want32[0])
    assert err[0] < TOL, err[0]                    # one key: nothing order dependent in front of the quantisers
    assert err.max() < TIE_DRIFT, float(err.max())
    p95e, p95s = float(np.percentile(err, 95)), float(np.percentile(sens, 95))
    assert p95e <= max(2.0 * p95s, 0.1), (p95e, p95s)
    print("2B block, 2048 causal positions, int8 semantics: error / RMS median", float(np.median(err)), "p95", p95e,
          "max", float(err.max()), "| oracle float32 vs float64 glue: median", float(np.median(sens)), "p95", p95s,
          "max", float(sens.max()))


def test_xl_dims_one_layer_step(rbm):
    """The tensor-parallel benchmark's dimensions (d 8192, 64 query / 8 KV heads, FFN 28672) as one
    layer: prompt of 12 tokens, then generation steps (large-matrix variants of the step kernels,
    shared-memory prologue for the 28672-wide row).  Float semantics strict; int8 semantics tie-aware."""
    cfg = dict(vocab_size=4096, d_model=8192, n_layers=1, n_heads=64, n_kv_heads=8, d_ff=28672)
    om = O.synth_model(cfg, 8192)
    prompt = np.random.default_rng(8193).integers(0, cfg["vocab_size"], size=12).astype(np.int64)
    # ---- float semantics: prefill logits and 6 generated tokens
    model = rbm.synth.model_from_oracle_params(om, semantics=rbm.sem.REFERENCE, max_seq=32)
    want, _ = O.model_forward(om, prompt[None, :], O.REFERENCE)
    got, _ = model.forward(prompt[None, :])
    err = per_pos_err(got[0], want[0])
    assert np.all(err < TOL), err.tolist()
    want_ids, steps, margins = _oracle_generation(om, prompt, 6, O.REFERENCE)
    got_ids = model.generate_greedy(prompt, 6)
    for i in range(6):
        assert got_ids[i] == want_ids[i] or margins[i] < 2 * TOL, (i, got_ids, want_ids, margins)
        if got_ids[i] != want_ids[i]:
            break
    del model
    # ---- int8 semantics: first position strict, the rest bounded by what flipped ties explain
    model = rbm.synth.model_from_oracle_params(om, semantics=rbm.sem.BASELINE, max_seq=32)
    sem64 = O.with_semantics(O.BASELINE, glue64=True)
    want32, _ = O.model_forward(om, prompt[None, :], O.BASELINE)
    want64, _ = O.model_forward(om, prompt[None, :], sem64)
    got, cache = model.forward(prompt[None, :], use_cache=True)
    e8, sens = _check_tie_aware(got[0], want32[0], want64[0], "XL prompt logits")
    assert e8[0] < TOL, e8[0]
    want_ids, steps, margins = _oracle_generation(om, prompt, 4, O.BASELINE)
    for i in range(3):
        logits, cache = model.forward(np.array([[want_ids[i]]]), past_kv_cache=cache, use_cache=True)
        e = float(per_pos_err(logits[0, -1:], np.asarray(steps[i + 1])[None])[0])
        assert e < TIE_DRIFT, (i, e)
        assert int(np.argmax(logits[0, -1])) == want_ids[i + 1] or margins[i + 1] < 2 * max(e, TOL)
    print("XL dims: float-semantics error / RMS", np.round(err, 7).tolist(), "| int8-semantics", np.round(e8, 5).tolist())
