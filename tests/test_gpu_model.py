"""GPU: the decode path above BitLinear (a6-a12) through the reference-shaped Python API,
against the fixtures produced by the unmodified reference and against the oracle.
Tolerance for floating outputs: max-abs error below 1e-3 of the output RMS."""
import os

import numpy as np
import pytest

import golden_inputs as G
from oracle import bitlinear_np as O

pytestmark = pytest.mark.gpu
TOL = 1e-3


def rel_err(a, b):
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    return float(np.max(np.abs(a - b)) / np.sqrt(np.mean(b ** 2)))


@pytest.fixture(scope="module")
def rb():
    import rotor_b200.transformer as tr
    import rotor_b200.bitnet_model as bm
    import rotor_b200.generation as gen
    import rotor_b200.synth as synth
    from rotor_b200 import semantics
    class NS: pass
    ns = NS()
    ns.tr, ns.bm, ns.gen, ns.synth, ns.sem = tr, bm, gen, synth, semantics
    return ns


def o_sem(s):
    """rotor_b200 semantics -> oracle semantics (three-term int8 stands for the float path)."""
    return O.Semantics(act_terms=0 if s.act_terms == 3 else s.act_terms, ffn_act=s.ffn_act,
                       rope_theta=s.rope_theta, causal=s.causal, eps=s.eps)


def test_rmsnorm(rb):
    rng = np.random.default_rng(0)
    x = rng.standard_normal((3, 5, 2560)).astype(np.float32)
    n = rb.tr.RMSNorm(2560)
    n.weight = 1.0 + 0.1 * rng.standard_normal(2560).astype(np.float32)
    assert rel_err(n.forward(x), O.rmsnorm(x, n.weight, 1e-6)) < 1e-5


def test_ternary_linear_api(rb, golden_dir):
    """TernaryLinear with the reference's call pattern (examples/test_gpu_layer.py:34-46)."""
    z = np.load(os.path.join(golden_dir, "bitlinear_2560x6912.npz"))
    w, scale, x1, x16 = G.bitlinear_case()
    lin = rb.tr.TernaryLinear(2560, 6912, use_gpu=True)
    assert lin.weights_cache is None
    lin.load_from_bitnet(O.pack_ternary_matrix(w), scale)
    assert lin.in_features == 2560 and lin.out_features == 6912 and lin.scale == scale
    assert np.array_equal(lin.weights_cache, w)
    assert rel_err(lin.forward(x1), z["y1"]) < TOL
    y = lin.forward(x16.reshape(2, 8, 2560))          # 3-D input keeps its leading dims
    assert y.shape == (2, 8, 6912) and rel_err(y.reshape(16, -1), z["y16"]) < TOL
    with pytest.raises(Exception):
        rb.tr.TernaryLinear(8, 8, use_gpu=False)       # no CPU path
    with pytest.raises(Exception):
        rb.tr.TernaryLinear(128, 16).forward(np.zeros((1, 128), np.float32))   # never loaded
    with pytest.raises(ValueError):
        lin.load_from_bitnet(np.zeros((4, 4), np.uint8), 1.0)


@pytest.mark.parametrize("mode", ["reference", "baseline"])
def test_ffn_block_config2(rb, golden_dir, mode):
    """Config 2: RMSNorm(2560) -> gate/up -> gating -> sub-norm(6912) -> down, batch 1 and 16."""
    z = np.load(os.path.join(golden_dir, "ffn_block.npz"))
    lw, x1, x16 = G.ffn_case()
    sem = rb.sem.REFERENCE if mode == "reference" else rb.sem.BASELINE
    ffn = rb.tr.GatedFFN(2560, 6912, semantics=sem)
    pre = rb.tr.RMSNorm(2560, eps=sem.eps)
    pre.weight = lw["post_attn_norm"]
    ffn.ffn_norm.weight = lw["ffn_sub_norm"]
    for nm, proj in (("gate", ffn.gate_proj), ("up", ffn.up_proj), ("down", ffn.down_proj)):
        proj.load_from_bitnet(O.pack_ternary_matrix(lw[nm][0]), lw[nm][1])
    from rotor_b200 import ops
    import torch
    for tag, x in (("m1", x1), ("m16", x16)):
        y_fused = ffn.forward_device(ops.to_device(x, torch.float32), pre_norm=pre).cpu().numpy()
        y_api = ffn.forward(pre.forward(x))
        want = O.ffn(O.rmsnorm(x, lw["post_attn_norm"], sem.eps), lw, o_sem(sem))
        if mode == "reference":
            assert rel_err(y_fused, z[tag]) < TOL and rel_err(y_api, z[tag]) < TOL
        assert rel_err(y_fused, want) < TOL, (mode, tag, rel_err(y_fused, want))
        assert rel_err(y_api, want) < TOL


@pytest.mark.parametrize("rows", [1, 2, 3])
def test_ffn_large_matrix_variants(rb, rows):
    """An FFN big enough (2048 -> 2 x 20480 -> 2048) that the generation-step products take their
    large-matrix variants: the pipelined tile loop (eight or more weight tiles per warp) and, for the
    20480-wide input of the down projection, the shared-memory prologue.  One, two and three rows
    select the one-column DP4A, two-column DP4A and tensor-core tile products."""
    import torch
    from rotor_b200 import ops
    d, ff = 2048, 20480
    rng = np.random.default_rng(1000 + rows)
    lw = {"gate": (O.synth_ternary(rng, ff, d), 0.017), "up": (O.synth_ternary(rng, ff, d), 0.015),
          "down": (O.synth_ternary(rng, d, ff), 0.016),
          "ffn_sub_norm": (1.0 + 0.1 * rng.standard_normal(ff)).astype(np.float32)}
    pre_w = (1.0 + 0.1 * rng.standard_normal(d)).astype(np.float32)
    x = rng.standard_normal((rows, d)).astype(np.float32)
    sem = rb.sem.BASELINE
    ffn = rb.tr.GatedFFN(d, ff, semantics=sem)
    pre = rb.tr.RMSNorm(d, eps=sem.eps)
    pre.weight = pre_w
    ffn.ffn_norm.weight = lw["ffn_sub_norm"]
    for nm, proj in (("gate", ffn.gate_proj), ("up", ffn.up_proj), ("down", ffn.down_proj)):
        proj.load_from_int8(lw[nm][0], lw[nm][1])
    before = rb.tr.abi.lib.rotor_b200_launch_count()
    got = ffn.forward_device(ops.to_device(x, torch.float32), pre_norm=pre).cpu().numpy()
    assert rb.tr.abi.lib.rotor_b200_launch_count() - before == 2     # the fused two-launch route
    want = O.ffn(O.rmsnorm(x, pre_w, sem.eps), lw, o_sem(sem))
    assert rel_err(got, want) < TOL, rel_err(got, want)
    rb.tr.abi.device_status()


def _tiny(rb, name, sem, **kw):
    om, prompt = G.tiny_model(name)
    kw.setdefault("max_seq", 64)
    return om, prompt, rb.synth.model_from_oracle_params(om, semantics=sem, **kw)


@pytest.mark.parametrize("name", list(G.TINY_MODELS))
def test_attention_and_block_standalone(rb, name):
    om, prompt, model = _tiny(rb, name, rb.sem.REFERENCE)
    cfg, lw = om["cfg"], om["layers"][0]
    rng = np.random.default_rng(5)
    x = rng.standard_normal((1, 6, cfg["d_model"])).astype(np.float32)
    blk = model.layers[0]
    want, wc = O.attention(x, lw, cfg, O.REFERENCE, None, True)
    got, cache = blk.attention.forward(x, use_cache=True)
    assert rel_err(got, want) < TOL
    assert rel_err(cache["k"], wc["k"]) < TOL and rel_err(cache["v"], wc["v"]) < TOL
    # one more token against the cache
    x2 = rng.standard_normal((1, 1, cfg["d_model"])).astype(np.float32)
    want2, _ = O.attention(x2, lw, cfg, O.REFERENCE, wc, True)
    got2, cache2 = blk.attention.forward(x2, kv_cache=cache, use_cache=True)
    assert rel_err(got2, want2) < TOL and cache2.length == 7
    # whole block, 2-D input like the reference accepts
    wantb, _ = O.block(x, lw, cfg, O.REFERENCE)
    gotb, none = blk.forward(x[0])
    assert none is None and gotb.shape == x[0].shape and rel_err(gotb, wantb[0]) < TOL
    # causal mask through the mask argument
    mask = O.causal_mask(6, 6)
    wantc, _ = O.block(x, lw, cfg, O.with_semantics(O.REFERENCE, causal=True))
    gotc, _ = blk.forward(x, mask=mask)
    assert rel_err(gotc, wantc) < TOL
    with pytest.raises(NotImplementedError):
        blk.forward(x, mask=np.zeros((6, 6)) + 1.0)


@pytest.mark.parametrize("name", list(G.TINY_MODELS))
def test_model_forward_matches_reference_fixture(rb, golden_dir, name):
    z = np.load(os.path.join(golden_dir, f"model_{name}.npz"))
    om, prompt, model = _tiny(rb, name, rb.sem.REFERENCE)
    logits, caches = model.forward(prompt[None, :], use_cache=True)
    assert logits.shape == z["prompt_logits"][None].shape
    assert rel_err(logits[0], z["prompt_logits"]) < TOL
    assert len(caches) == om["cfg"]["n_layers"]
    assert rel_err(caches[-1]["k"], z["last_k"]) < TOL
    l1, _ = model.forward(prompt)                      # 1-D ids -> [S, V]
    assert l1.shape == z["prompt_logits"].shape and rel_err(l1, z["prompt_logits"]) < TOL
    last, _ = model.forward(prompt[None, :], logits_positions="last")
    assert rel_err(last[0, -1], z["prompt_logits"][-1]) < TOL
    hid, _ = model.forward(prompt[None, :], return_logits=False)
    want_h, _ = O.model_forward(om, prompt[None, :], O.REFERENCE, return_logits=False)
    assert rel_err(hid, want_h) < TOL
    mc = rb.synth.model_from_oracle_params(om, semantics=rb.sem.REFERENCE.with_(causal=True), max_seq=64)
    lc, _ = mc.forward(prompt[None, :])
    assert rel_err(lc[0], z["prompt_logits_causal"]) < TOL


@pytest.mark.parametrize("name", list(G.TINY_MODELS))
def test_greedy_generation_identical_to_reference(rb, golden_dir, name):
    """First 32 greedy tokens equal the reference's (TextGenerator, use_cache=True), through the
    device-resident graph path, the eager step path, and the host-sampling path."""
    z = np.load(os.path.join(golden_dir, f"model_{name}.npz"))
    om, prompt, model = _tiny(rb, name, rb.sem.REFERENCE)
    want = z["greedy_ids"].tolist()
    n_new = len(want) - len(prompt)
    assert n_new == G.N_NEW
    tok = rb.synth.PassThroughTokenizer()
    text = " ".join(map(str, prompt))
    tg = rb.gen.TextGenerator(model, tok, max_length=len(want), use_cache=True)
    seen = []
    out = tg.generate(text, max_new_tokens=n_new, stop_on_eos=False, callback=seen.append)
    assert [int(t) for t in out.split()] == want
    assert [int(t) for t in seen] == want[len(prompt):]
    assert model.generate_greedy(prompt, n_new, use_graph=False) == want[len(prompt):]
    assert model.generate_greedy(prompt, n_new, use_graph=True, chunk=0) == want[len(prompt):]
    # host-side sampling strategy object -> logits come back each step
    class Argmax(rb.gen.SamplingStrategy):
        def sample(self, logits, temperature=1.0):
            return int(np.argmax(logits))
    tg2 = rb.gen.TextGenerator(model, tok, sampling_strategy=Argmax(), max_length=len(want), use_cache=True)
    out2 = tg2.generate(text, max_new_tokens=n_new, stop_on_eos=False)
    assert [int(t) for t in out2.split()] == want
    # per-step logits stay within tolerance of the reference's
    logits, cache = model.forward(prompt[None, :], use_cache=True, logits_positions="last")
    assert rel_err(logits[0, -1], z["step_logits"][0]) < TOL
    l2, cache = model.forward(np.array([[want[len(prompt)]]]), past_kv_cache=cache, use_cache=True)
    assert rel_err(l2[0, -1], z["step_logits"][1]) < TOL


@pytest.mark.parametrize("name", list(G.TINY_MODELS))
def test_per_step_logits_against_fixture_margins(rb, golden_dir, name):
    """Every one of the 32 teacher-forced generation steps against the reference fixture: the logit error
    (max-abs over the vocabulary, in units of the step's logit RMS) stays below the tolerance AND below half
    the reference's own top-1 / top-2 margin at that step (stored with the fixture), which is what makes the
    greedy tokens identical rather than merely likely to be."""
    z = np.load(os.path.join(golden_dir, f"model_{name}.npz"))
    om, prompt, model = _tiny(rb, name, rb.sem.REFERENCE)
    want = z["greedy_ids"].tolist()
    logits, cache = model.forward(prompt[None, :], use_cache=True)
    cur = logits[0, -1]
    worst = 0.0
    for i in range(G.N_NEW):
        e = rel_err(cur, z["step_logits"][i])
        worst = max(worst, e)
        assert e < TOL, (i, e)
        assert 2 * e < z["top2_margin"][i], (i, e, float(z["top2_margin"][i]))
        assert int(np.argmax(cur)) == want[len(prompt) + i]
        if i + 1 < G.N_NEW:
            nxt, cache = model.forward(np.array([[want[len(prompt) + i]]]), past_kv_cache=cache, use_cache=True)
            cur = nxt[0, -1]
    print(f"{name}: worst per-step logit error {worst:.2e} of RMS, smallest margin {float(z['top2_margin'].min()):.2e}")


@pytest.mark.parametrize("name", list(G.TINY_MODELS))
def test_baseline_semantics_against_oracle(rb, name):
    """Published semantics (int8 activations, relu^2, rotary, causal, eps 1e-5) against the oracle that
    quantises identically.  A value on a rounding tie of the quantiser is decided by float summation
    order, so the check is tie-aware: the first position (one key, no order-dependent sum before a
    quantiser) within tolerance; every teacher-forced step picks the oracle's token unless the
    oracle's top-2 margin there is below twice the logit error measured at that step; no step
    drifts beyond what flipped ties explain."""
    om, prompt, model = _tiny(rb, name, rb.sem.BASELINE)
    want_logits, _ = O.model_forward(om, prompt[None, :], O.BASELINE)
    logits, cache = model.forward(prompt[None, :], use_cache=True)
    assert rel_err(logits[0, 0], want_logits[0, 0]) < TOL
    assert rel_err(logits, want_logits) < 0.3
    ids, steps = O.generate_greedy(om, prompt, 32, O.BASELINE, return_logits=True)
    want = ids[len(prompt):]
    cur = logits[0, -1]
    equal = 0
    for i in range(32):
        ref = np.asarray(steps[i], np.float64)
        e = rel_err(cur, ref)
        top2 = np.partition(ref, -2)[-2:]
        margin = float((top2[1] - top2[0]) / np.sqrt(np.mean(ref ** 2)))
        assert e < 0.3, (i, e)
        assert int(np.argmax(cur)) == want[i] or margin < 2 * max(e, TOL), (i, int(np.argmax(cur)), want[i], margin, e)
        equal += int(np.argmax(cur)) == want[i]
        if i < 31:
            nxt, cache = model.forward(np.array([[want[i]]]), past_kv_cache=cache, use_cache=True)
            cur = nxt[0, -1]
    assert equal >= 24, equal


def test_generation_loop_rules(rb):
    """max_length caps prompt + new tokens, EOS stops without being appended, streaming yields
    the prompt first (reference src/rotor/generation.py:210, 228-229, 315)."""
    om, prompt, model = _tiny(rb, "hd64", rb.sem.REFERENCE)
    tok = rb.synth.PassThroughTokenizer()
    text = " ".join(map(str, prompt))
    full = model.generate_greedy(prompt, 12)
    tg = rb.gen.TextGenerator(model, tok, max_length=len(prompt) + 4)
    assert len(tg.generate(text, max_new_tokens=50, stop_on_eos=False).split()) == len(prompt) + 4
    tg0 = rb.gen.TextGenerator(model, tok, max_length=len(prompt))
    assert tg0.generate(text) == text                      # nothing to generate
    tok_eos = rb.synth.PassThroughTokenizer(eos_token_id=full[3])
    tg_eos = rb.gen.TextGenerator(model, tok_eos, max_length=64)
    out = [int(t) for t in tg_eos.generate(text, max_new_tokens=12).split()]
    assert out == list(prompt) + full[:full.index(full[3])]
    pieces = list(rb.gen.TextGenerator(model, tok, max_length=64).generate_streaming(text, max_new_tokens=5,
                                                                                   stop_on_eos=False))
    assert pieces[0] == text and [int(p) for p in pieces[1:]] == full[:5]
    # top-k / top-p return valid ids on both routes: drawn on the device (the default with this model) and,
    # with device=False, from host logits with NumPy's global stream as in the reference
    np.random.seed(0)
    assert rb.gen.TopKSampling(k=5).device is None and rb.gen.TopPSampling(p=0.8, device=False).device is False
    for strat in (rb.gen.TopKSampling(k=5), rb.gen.TopPSampling(p=0.8), rb.gen.TopKSampling(k=5, device=False),
                  rb.gen.TopPSampling(p=0.8, device=False)):
        tgs = rb.gen.TextGenerator(model, tok, sampling_strategy=strat, temperature=0.7, max_length=64)
        ids = [int(t) for t in tgs.generate(text, max_new_tokens=4, stop_on_eos=False).split()]
        assert len(ids) == len(prompt) + 4 and all(0 <= t < om["cfg"]["vocab_size"] for t in ids)


def test_load_bitnet_model_from_checkpoint(rb, tmp_path, golden_dir):
    """load_bitnet_model(dir, use_gpu=True) on a synthetic config.json + model.safetensors."""
    z = np.load(os.path.join(golden_dir, "model_hd64.npz"))
    om, prompt = G.tiny_model("hd64")
    rb.synth.write_checkpoint(om, str(tmp_path))
    model = rb.bm.load_bitnet_model(str(tmp_path), use_gpu=True, max_seq=64)
    logits, _ = model.forward(prompt[None, :])
    assert rel_err(logits[0], z["prompt_logits"]) < TOL
    with pytest.raises(Exception):
        rb.bm.load_bitnet_model(str(tmp_path), use_gpu=False)


def test_plugin_backend_object(rb):
    """get_gpu() -> pack_ternary_weights / ternary_matmul with the reference's argument shapes
    (src/rotor/transformer.py:107-109, 136-142)."""
    from rotor_b200.gpu_layers import get_gpu
    gpu = get_gpu()
    assert gpu is get_gpu()
    rng = np.random.default_rng(12)
    w = O.synth_ternary(rng, 2560, 2560)
    packed = gpu.pack_ternary_weights(w)
    scales = np.full(2560, 1.2, dtype=np.float32)
    x = rng.standard_normal(2560).astype(np.float32)
    y = gpu.ternary_matmul(packed, scales, x, 2560, 2560)
    want = (w.astype(np.float32) @ x) * scales
    assert y.dtype == np.float32 and y.shape == (2560,)
    assert np.abs(y - want).max() < 1e-2          # the authors' own GPU-vs-CPU gate (gpu_layers.py:181)
    assert rel_err(y, want) < TOL
    with pytest.raises(ValueError):
        gpu.ternary_matmul(packed, scales, x, 2560, 100)


def test_batched_forward_and_cache_growth(rb):
    om, prompt, model = _tiny(rb, "hd64", rb.sem.REFERENCE, max_batch=1)
    rng = np.random.default_rng(3)
    ids = rng.integers(0, om["cfg"]["vocab_size"], size=(3, 7))
    want, _ = O.model_forward(om, ids, O.REFERENCE)
    got, caches = model.forward(ids, use_cache=True)        # batch 3 > max_batch 1: handle regrows
    assert rel_err(got, want) < TOL and caches[0]["k"].shape[0] == 3
    long_ids = rng.integers(0, om["cfg"]["vocab_size"], size=(1, 90))   # > max_seq 64
    want2, _ = O.model_forward(om, long_ids, O.REFERENCE)
    got2, _ = model.forward(long_ids)
    assert rel_err(got2, want2) < TOL


def test_prefill_and_stepwise_decode_agree(rb):
    """Size-independent property of the cached path (causal semantics): the last-position logits
    of one forward over n+1 tokens equal those of a forward over n tokens followed by a one-token
    step.  The prefill side runs the tiled tensor-core GEMM (>= 32 columns), the step the fused
    generation kernels."""
    om, prompt, model = _tiny(rb, "hd128", rb.sem.BASELINE, max_rows=64)
    rng = np.random.default_rng(17)
    ids = rng.integers(0, om["cfg"]["vocab_size"], size=(1, 41))
    full, _ = model.forward(ids, logits_positions="last")
    _, cache = model.forward(ids[:, :40], use_cache=True, logits_positions="last")
    step, _ = model.forward(ids[:, 40:], past_kv_cache=cache, use_cache=True, logits_positions="last")
    # int8 rounding decisions can differ between the two routes only through float32 summation order
    assert rel_err(step[0, -1], full[0, -1]) < 2e-2
    ref = rb.synth.model_from_oracle_params(om, semantics=rb.sem.REFERENCE.with_(causal=True), max_seq=64)
    full_r, _ = ref.forward(ids, logits_positions="last")
    _, cache_r = ref.forward(ids[:, :40], use_cache=True, logits_positions="last")
    step_r, _ = ref.forward(ids[:, 40:], past_kv_cache=cache_r, use_cache=True, logits_positions="last")
    assert rel_err(step_r[0, -1], full_r[0, -1]) < TOL


@pytest.mark.parametrize("name", list(G.TINY_MODELS))
@pytest.mark.parametrize("causal", [False, True])
def test_tiled_prefill_attention(rb, name, causal):
    """Prompts of 16 positions and more take the tiled attention kernel: ragged lengths (not a
    multiple of the 64-key tile or of the query tile), batch 2, then a second chunk attending
    over the cached keys of the first."""
    sem = rb.sem.REFERENCE.with_(causal=causal)
    osem = O.with_semantics(O.REFERENCE, causal=causal)
    om, prompt, model = _tiny(rb, name, sem, max_seq=256, max_batch=2)
    cfg, lw = om["cfg"], om["layers"][0]
    rng = np.random.default_rng(23)
    att = model.layers[0].attention
    x = rng.standard_normal((2, 150, cfg["d_model"])).astype(np.float32)
    mask = O.causal_mask(150, 150) if causal else None
    want, wc = O.attention(x, lw, cfg, osem, None, True)
    got, cache = att.forward(x, mask=mask, use_cache=True)
    assert rel_err(got, want) < TOL
    x2 = rng.standard_normal((2, 37, cfg["d_model"])).astype(np.float32)
    mask2 = O.causal_mask(37, 187) if causal else None
    want2, _ = O.attention(x2, lw, cfg, osem, wc, True)
    got2, cache2 = att.forward(x2, mask=mask2, kv_cache=cache, use_cache=True)
    assert rel_err(got2, want2) < TOL and cache2.length == 187


def test_prefill_qkv_epilogue_cache_rows(rb):
    """Prompt-sized calls in published semantics (one activation term, head_dim 128, 256 rows and more): the
    q/k/v product dequantises, rotates and appends to the cache in its read-back.  The cache rows (a direct
    function of the quantised input: rotary angles, positions, per-sequence offsets) and the attention
    output against the oracle, for a first chunk of 2 x 150 positions and a second of 2 x 140 behind it."""
    om, prompt, model = _tiny(rb, "hd128", rb.sem.BASELINE, max_seq=320, max_batch=2)
    cfg, lw = om["cfg"], om["layers"][0]
    rng = np.random.default_rng(77)
    att = model.layers[0].attention
    x = rng.standard_normal((2, 150, cfg["d_model"])).astype(np.float32)
    want, wc = O.attention(x, lw, cfg, O.BASELINE, None, True)
    got, cache = att.forward(x, mask=O.causal_mask(150, 150), use_cache=True)
    assert rel_err(cache["k"], wc["k"]) < TOL and rel_err(cache["v"], wc["v"]) < TOL
    assert rel_err(got, want) < 5e-3   # one-term int8 output projection: a flipped rounding tie moves a row
    x2 = rng.standard_normal((2, 140, cfg["d_model"])).astype(np.float32)
    want2, wc2 = O.attention(x2, lw, cfg, O.BASELINE, wc, True)
    got2, cache2 = att.forward(x2, mask=O.causal_mask(140, 290), kv_cache=cache, use_cache=True)
    assert cache2.length == 290
    assert rel_err(cache2["k"], wc2["k"]) < TOL and rel_err(cache2["v"], wc2["v"]) < TOL
    assert rel_err(got2, want2) < 5e-3


def test_wide_ffn_generation_step(rb):
    """d_ff above 8192: the down projection's prologue stages its input row in shared memory.
    Logits within tolerance and the same 32 greedy tokens as the oracle, published semantics."""
    om, prompt, model = _tiny(rb, "wide_ffn", rb.sem.BASELINE)
    osem = o_sem(rb.sem.BASELINE)
    want, _ = O.model_forward(om, prompt[None, :], osem)
    got, _ = model.forward(prompt[None, :])
    assert rel_err(got, want) < TOL
    ids = O.generate_greedy(om, prompt, G.N_NEW, osem)[len(prompt):]
    before = rb.tr.abi.lib.rotor_b200_launch_count()
    assert model.generate_greedy(prompt, G.N_NEW, use_graph=False) == ids
    per_step = (rb.tr.abi.lib.rotor_b200_launch_count() - before) / G.N_NEW
    assert per_step <= 5 * om["cfg"]["n_layers"] + 2     # the five-launch block (the unfused path takes 8 per block)
    assert model.generate_greedy(prompt, G.N_NEW, use_graph=True) == ids


@pytest.mark.parametrize("name", list(G.TINY_MODELS))
@pytest.mark.parametrize("max_seq,n_prompt", [(1100, 1040), (2100, 2040)])
def test_long_cache_generation_step(rb, name, max_seq, n_prompt):
    """Caches of 1024 and of 2048 and more positions: one-token attention keeps a slice of the cache in
    shared memory per CTA, eight slices per KV head while they fit, sixteen (a 16-CTA cluster where the
    device places one) beyond.  Last-position logits after the prompt and the next 8 greedy tokens against
    the oracle, float semantics."""
    om, _, model = _tiny(rb, name, rb.sem.REFERENCE, max_seq=max_seq)
    rng = np.random.default_rng(5150)
    prompt = rng.integers(0, om["cfg"]["vocab_size"], size=n_prompt).astype(np.int64)
    ids, steps = O.generate_greedy(om, prompt, 8, O.REFERENCE, return_logits=True)
    want = ids[len(prompt):]
    logits, cache = model.forward(prompt[None, :], use_cache=True, logits_positions="last")
    assert rel_err(logits[0, -1], steps[0]) < TOL
    nxt, _ = model.forward(np.array([[want[0]]]), past_kv_cache=cache, use_cache=True)
    assert rel_err(nxt[0, -1], steps[1]) < TOL
    assert model.generate_greedy(prompt, 8, use_graph=False) == want
    assert model.generate_greedy(prompt, 8, use_graph=True) == want


def test_empty_and_single_element_inputs(rb):
    """Zero token rows give empty outputs (the reference's NumPy path does the same); one row of one
    sequence is the smallest real call."""
    lin = rb.tr.TernaryLinear(64, 48)
    lin.load_from_int8(np.ones((48, 64), dtype=np.int8), 0.5)
    assert lin.forward(np.zeros((0, 64), dtype=np.float32)).shape == (0, 48)
    assert lin.forward(np.zeros((2, 0, 64), dtype=np.float32)).shape == (2, 0, 48)
    y = lin.forward(np.ones((1, 64), dtype=np.float32))
    assert y.shape == (1, 48) and np.allclose(y, 32.0, rtol=1e-5)
    norm = rb.tr.RMSNorm(64)
    assert norm.forward(np.zeros((0, 64), dtype=np.float32)).shape == (0, 64)
    ffn = rb.tr.GatedFFN(64, 128)
    assert ffn.gate_proj.in_features == 64
    for p in (ffn.gate_proj, ffn.up_proj, ffn.down_proj):
        p.load_from_int8(np.ones((p.out_features, p.in_features), dtype=np.int8), 0.1)
    assert ffn.forward(np.zeros((0, 64), dtype=np.float32)).shape == (0, 64)


@pytest.mark.parametrize("batch", [2, 9, 17])
def test_batched_decode_step(rb, batch):
    """One-token steps for several sequences at once against the oracle run sequence by sequence.
    Sixteen sequences and more take the tiled attention kernel instead of the split decode kernel."""
    om, prompt, model = _tiny(rb, "hd128", rb.sem.REFERENCE, max_batch=batch)
    rng = np.random.default_rng(40 + batch)
    vocab = om["cfg"]["vocab_size"]
    ids = rng.integers(0, vocab, size=(batch, 6))
    nxt = rng.integers(0, vocab, size=(batch, 1))
    _, caches = model.forward(ids, use_cache=True)
    got, caches2 = model.forward(nxt, past_kv_cache=caches, use_cache=True)
    assert caches2[0].length == 7
    for b in range(batch):
        _, oc = O.model_forward(om, ids[b:b + 1], O.REFERENCE, use_cache=True)
        want, _ = O.model_forward(om, nxt[b:b + 1], O.REFERENCE, past_kv_cache=oc, use_cache=True)
        assert rel_err(got[b], want[0]) < TOL, (b, rel_err(got[b], want[0]))


def test_wide_ffn_many_rows(rb):
    """70 rows through an FFN whose hidden width (9216) exceeds 8192: the gating / sub-norm / quantise
    stage takes the 512-thread register-resident kernel."""
    import torch
    from rotor_b200 import ops
    d, ff, rows = 256, 9216, 70
    rng = np.random.default_rng(77)
    lw = {"gate": (O.synth_ternary(rng, ff, d), 0.02), "up": (O.synth_ternary(rng, ff, d), 0.018),
          "down": (O.synth_ternary(rng, d, ff), 0.015),
          "ffn_sub_norm": (1.0 + 0.1 * rng.standard_normal(ff)).astype(np.float32)}
    pre_w = (1.0 + 0.1 * rng.standard_normal(d)).astype(np.float32)
    x = rng.standard_normal((rows, d)).astype(np.float32)
    sem = rb.sem.REFERENCE
    ffn = rb.tr.GatedFFN(d, ff, semantics=sem)
    pre = rb.tr.RMSNorm(d, eps=sem.eps)
    pre.weight = pre_w
    ffn.ffn_norm.weight = lw["ffn_sub_norm"]
    for nm, proj in (("gate", ffn.gate_proj), ("up", ffn.up_proj), ("down", ffn.down_proj)):
        proj.load_from_int8(lw[nm][0], lw[nm][1])
    got = ffn.forward_device(ops.to_device(x, torch.float32), pre_norm=pre).cpu().numpy()
    want = O.ffn(O.rmsnorm(x, pre_w, sem.eps), lw, o_sem(sem))
    assert rel_err(got, want) < TOL, rel_err(got, want)


@pytest.mark.parametrize("batch", [3, 6])
def test_batched_greedy_generation(rb, batch):
    """Equal-length prompts generated together give, sequence by sequence, the oracle's tokens
    (three sequences: fused generation step; six: the unfused one)."""
    om, prompt, model = _tiny(rb, "hd64", rb.sem.REFERENCE, max_batch=batch)
    rng = np.random.default_rng(60 + batch)
    prompts = rng.integers(0, om["cfg"]["vocab_size"], size=(batch, 5))
    got = model.generate_greedy_batch(prompts, 12)
    assert got.shape == (batch, 12)
    for b in range(batch):
        want = O.generate_greedy(om, prompts[b], 12, O.REFERENCE)[5:]
        assert list(got[b]) == want, b
    assert np.array_equal(model.generate_greedy_batch(prompts, 12, use_graph=False), got)


@pytest.mark.parametrize("lens", [[3, 7, 5], [9, 2, 6, 4, 9, 1], [30, 17, 40], list(range(4, 21))])
def test_batched_greedy_generation_ragged(rb, lens):
    """Prompts of different lengths generated together: every sequence gives the tokens of its
    own single-prompt generation by the oracle (3 sequences: fused step; 6: unfused; 30/17/40:
    tiled prefill attention over padded rows; 17 sequences: tiled attention in the steps)."""
    import dataclasses
    batch = len(lens)
    sem, osem = dataclasses.replace(rb.sem.REFERENCE, causal=True), dataclasses.replace(O.REFERENCE, causal=True)
    om, prompt, model = _tiny(rb, "hd64", sem, max_batch=batch)
    rng = np.random.default_rng(70 + batch + lens[0])
    prompts = [rng.integers(0, om["cfg"]["vocab_size"], size=n) for n in lens]
    new = 8
    got = model.generate_greedy_batch(prompts, new)
    assert got.shape == (batch, new)
    for b in range(batch):
        want = O.generate_greedy(om, prompts[b], new, osem)[lens[b]:]
        assert list(got[b]) == want, b
    assert np.array_equal(model.generate_greedy_batch(prompts, new, use_graph=False), got)
    with pytest.raises(ValueError):  # without a causal mask a row would attend to its padding
        _tiny(rb, "hd64", rb.sem.REFERENCE, max_batch=batch)[2].generate_greedy_batch(prompts, new)
