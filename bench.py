#!/usr/bin/env python
"""Benchmark of the ternary BitLinear decode path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference]

Workload (N = 1 and, as independent replicas, N > 1): random-init BitNet-b1.58-2B
architecture (30 layers, hidden 2560, 20 query / 5 KV heads, FFN 6912, vocab 128256,
bf16 tied embeddings, ternary projections), greedy decode, batch 1, 128-token seeded
prompt, published semantics (int8 absmax activations, relu^2 gating, rotary, causal).
A step is one generated token.  The prompt prefill is not timed; W warm-up tokens are
generated, then exactly K tokens are timed with CUDA events on the launching stream
(barrier + synchronize on both sides, max over ranks).

One JSON line is printed by rank 0:
  value        tokens/s of the whole job, weights and KV cache resident in HBM
  e2e          the same through TextGenerator.generate(): host prompt string in, token ids
               back on the host every step
  roofline     the ternary GEMV kernel on config 1 (2560 -> 6912, batch 1): 64 distinct
               matrices (283 MB > L2) back to back in one CUDA graph, algorithmic bytes per
               launch / mean launch time, against the measured HBM copy bandwidth; beside it
               the per-launch floor of a chain of empty kernels in the same harness and the
               single-matrix (L2-resident) figure
  roofline_step  the generation-step product kernel: its algorithmic bytes per token over its
               share of the step (share from the committed launch list under profiles/)
  parity       the GPU path against the CPU oracle on the same seeded weights (2B dimensions,
               two layers, full vocabulary), measured in this run
  ffn_block / prefill_2b / xl   (N = 1) the other configurations: FFN block of the 2B shape at
               1 and 16 rows, prefill of 8 x 2048 tokens, the 80-layer d 8192 shape decoding at
               batch 1 and 64 after a 1024-token prompt
  xl_tp        (N > 1) that 80-layer shape sharded tensor-parallel over the N GPUs of the launch
               (strong scaling), batch 1 / 8 / 64 after a 1024-token prompt
  cpu_baseline the NumPy oracle port of the reference's path on this box's host cores,
               bounded sample (N = 1 only)
--impl reference times the reference itself on the host cores (its installed copy under baseline/_ref,
through its own TextGenerator.generate; the port stands in where the copy is absent).
--workload / --only select one section alone (profiling aids; they print their own line).
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for _p in (ROOT, os.path.join(ROOT, "rotor-rag_b200")):
    if _p not in sys.path:
        sys.path.insert(0, _p)

METRIC = "BitNet-2B-shape greedy decode tokens/s (batch 1); roofline = ternary GEMV HBM GB/s"
UNIT = "tokens/s"
CFG_2B = dict(vocab_size=128256, d_model=2560, n_layers=30, n_heads=20, n_kv_heads=5, d_ff=6912)
PROMPT_LEN = 128
XL_PROMPT_LEN = 1024
WORKLOAD = ("BitNet-b1.58-2B-shape random-init model (30 layers, d 2560, 20q/5kv heads, ffn 6912, vocab 128256), "
            "greedy decode batch 1 after a 128-token prompt")
SEM_GPU = "published int8 semantics: per-token absmax int8 activations, relu^2 gating, rotary, causal"
SEM_CPU = ("the reference's own float semantics (float activations x int8 weight cache, no rotary, no mask): "
           "the only path its NumPy code has; same shapes, same bytes of weights per token")


def algorithmic_bytes_per_token(cfg, context, kv_bytes=4):
    """Bytes one decode step has to read: ternary tiles, bf16 LM head, norm weights, one
    embedding row, and the KV cache at `context` positions."""
    d, ff, L = cfg["d_model"], cfg["d_ff"], cfg["n_layers"]
    hd = d // cfg["n_heads"]
    dq, dkv = cfg["n_heads"] * hd, cfg["n_kv_heads"] * hd
    ternary = L * ((dq + 2 * dkv) * d + d * dq + 2 * ff * d + d * ff) // 4
    lm = cfg["vocab_size"] * d * 2
    norms = L * (3 * d + ff) * 4 + d * 4
    kv = L * 2 * dkv * context * kv_bytes
    return ternary + lm + norms + d * 2 + kv


# ----------------------------------------------------------------------------- clocks
class ClockSampler:
    """nvidia-smi clock / throttle-reason samples taken while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), [c.strip() for c in line.split(",")]))

    def stop(self, t0, t1):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        rows = [r for (t, r) in self.rows if t0 - 0.05 <= t <= t1 + 0.15 and len(r) >= 7] or \
               [r for (_, r) in self.rows if len(r) >= 7]
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        sm = [float(r[0]) for r in rows]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(r[3 + i].lower().startswith("active") for r in rows)]
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": float(rows[0][1]), "reasons": reasons,
                "samples": len(rows)}


def measured_peak_gbs():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


# ----------------------------------------------------------------------------- CPU port
def cpu_decode_sample(n_tokens, n_warm, seed=0, budget_s=None):
    """The oracle's restatement of the reference path (NumPy + its int8 weight cache) on the
    host cores: 2B-shape model, KV cache pre-filled with N(0,1) at 128 positions (timing is
    the same as after a real prefill), greedy one-token steps.  Returns tokens/s and notes."""
    import numpy as np
    from oracle import bitlinear_np as O
    try:
        from threadpoolctl import threadpool_info
        threads = max([p.get("num_threads", 1) for p in threadpool_info()] or [os.cpu_count() or 1])
    except Exception:
        threads = os.cpu_count() or 1
    cfg = CFG_2B
    model = O.synth_model(cfg, seed, random_norms=False, fast_embed=True)
    rng = np.random.default_rng(seed + 1)
    hd = cfg["d_model"] // cfg["n_heads"]
    cache = [{"k": rng.standard_normal((1, cfg["n_kv_heads"], PROMPT_LEN, hd)).astype(np.float32),
              "v": rng.standard_normal((1, cfg["n_kv_heads"], PROMPT_LEN, hd)).astype(np.float32)}
             for _ in range(cfg["n_layers"])]
    tok = int(rng.integers(0, cfg["vocab_size"]))
    times = []
    t_start = time.perf_counter()
    for i in range(n_warm + n_tokens):
        t0 = time.perf_counter()
        logits, cache = O.model_forward(model, np.array([[tok]]), O.REFERENCE, past_kv_cache=cache, use_cache=True)
        tok = O.greedy(logits[0, -1])
        dt = time.perf_counter() - t0
        if i >= n_warm:
            times.append(dt)
        if budget_s is not None and i >= n_warm and time.perf_counter() - t_start > budget_s:
            break
    per_tok = sum(times) / len(times)
    return 1.0 / per_tok, threads, len(times)


class _PassTokenizer:
    """ids as space-separated integers; the three members the reference's TextGenerator uses."""
    eos_token_id = -1

    def encode(self, text, add_special_tokens=True, return_numpy=True):
        import numpy as np
        return np.array([int(t) for t in text.split()], dtype=np.int64)

    def decode(self, ids, skip_special_tokens=True):
        return " ".join(str(int(t)) for t in ids)


class _BudgetSpent(Exception):
    pass


def reference_decode_sample(n_tokens, n_warm, seed=0, budget_s=None):
    """The unmodified reference (its installed copy under baseline/_ref, made by `make -C oracle refpy`)
    on the host cores: BitNetModel of the 2B shape with random ternary weights placed in its int8 weight
    caches, its own TextGenerator.generate (greedy, use_cache=True) on a 128-token prompt; per-token times
    from the callback, the first token (prefill) left out.  None if the copy is absent or does not import."""
    import contextlib
    import io
    import numpy as np
    ref_root = os.path.join(ROOT, "baseline", "_ref")
    if not (os.path.isdir(os.path.join(ref_root, "src", "rotor")) and
            os.path.exists(os.path.join(ref_root, "native", "build", "librotor_core.so"))):
        return None
    try:
        from oracle import bitlinear_np as O
        sys.path.insert(0, os.path.join(ref_root, "src"))
        quiet = io.StringIO()
        with contextlib.redirect_stdout(quiet):
            import rotor.bitnet_model as bm
            import rotor.generation as gen
            cfg = CFG_2B
            om = O.synth_model(cfg, seed, random_norms=False, fast_embed=True)
            model = bm.BitNetModel(dict(cfg))
            model.embed_tokens = np.asarray(om["embed"], dtype=np.float32)
            model.norm.weight = np.asarray(om["norm"], dtype=np.float32)
            for layer, lw in zip(model.layers, om["layers"]):
                layer.input_norm.weight = lw["input_norm"]
                layer.post_attn_norm.weight = lw["post_attn_norm"]
                layer.attention.attn_norm.weight = lw["attn_sub_norm"]
                layer.ffn.ffn_norm.weight = lw["ffn_sub_norm"]
                for name, proj in (("q", layer.attention.q_proj), ("k", layer.attention.k_proj),
                                   ("v", layer.attention.v_proj), ("o", layer.attention.o_proj),
                                   ("gate", layer.ffn.gate_proj), ("up", layer.ffn.up_proj),
                                   ("down", layer.ffn.down_proj)):
                    w, sc = lw[name]
                    proj.weights_cache = w      # what load_from_bitnet leaves behind (int8 [out, in])
                    proj.scale = float(sc)
        try:
            from threadpoolctl import threadpool_info
            threads = max([p.get("num_threads", 1) for p in threadpool_info()] or [os.cpu_count() or 1])
        except Exception:
            threads = os.cpu_count() or 1
        rng = np.random.default_rng(seed + 1)
        prompt = " ".join(str(int(t)) for t in rng.integers(0, cfg["vocab_size"], size=PROMPT_LEN))
        total = n_warm + n_tokens + 1           # + the token that comes out of the prefill
        g = gen.TextGenerator(model, _PassTokenizer(), max_length=PROMPT_LEN + total + 1, use_cache=True)
        stamps = []
        t_start = time.perf_counter()

        def on_token(_text):
            stamps.append(time.perf_counter())
            if budget_s is not None and len(stamps) > n_warm + 1 and stamps[-1] - t_start > budget_s:
                raise _BudgetSpent()
        try:
            with contextlib.redirect_stdout(quiet):
                g.generate(prompt, max_new_tokens=total, stop_on_eos=False, callback=on_token)
        except _BudgetSpent:
            pass
        steps = [b - a for a, b in zip(stamps[:-1], stamps[1:])][n_warm:]
        if not steps:
            return None
        return len(steps) / sum(steps), threads, len(steps)
    except Exception as e:  # the port below stands in; say why on stderr
        print(f"reference copy under baseline/_ref not usable ({type(e).__name__}: {e}); timing the port", file=sys.stderr)
        return None


def run_reference(args, rank):
    """Reference arm: the reference's CPU implementation of the path.  Where its installed copy
    (baseline/_ref) is present, the unmodified reference itself through TextGenerator.generate (kind
    "reference"); otherwise the NumPy port under oracle/ (kind "port"): the same
    np.dot(x, int8_cache.T) * scale, RMSNorm, attention and LM-head statements, asserted equal to the
    reference by the fixture generator.  Same step and warm-up counts as the GPU arm, within a
    wall-clock limit."""
    if rank != 0:
        return
    n_tok, n_warm = args.steps, max(args.warmup, 3)
    t0 = time.perf_counter()
    real = reference_decode_sample(n_tok, n_warm, budget_s=240.0)
    kind = "reference" if real else "port"
    tps, threads, done = real if real else cpu_decode_sample(n_tok, n_warm, budget_s=240.0)
    sample = (f"{done} timed one-token steps (+{n_warm} warm-up) of the full 30-layer 2B-shape model on the host, " +
              (f"the reference's TextGenerator.generate after its own prefill of the {PROMPT_LEN}-token prompt" if real
               else f"KV cache pre-filled at {PROMPT_LEN} positions"))
    line = {"metric": METRIC, "value": tps, "unit": UNIT, "impl": "reference", "n_gpus": args.gpus,
            "steps": done, "warmup": n_warm, "ms_per_step": 1000.0 / tps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f64 (NumPy promotion) over int8 weight cache",
            "data": "synthetic", "semantics": SEM_CPU,
            "config": {"workload": WORKLOAD, "global_batch": args.gpus, "prompt_len": PROMPT_LEN},
            "cpu_baseline": {"value": tps, "unit": UNIT, "cores": threads, "kind": kind, "sample": sample},
            "e2e": {"value": tps, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0, "wall_s": time.perf_counter() - t0}
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------- GPU arm
def gemv_roofline(torch, abi, nmat=64, iters=20, out=6912, inn=2560, distinct=True):
    """Config 1: ternary GEMV 2560 -> 6912, batch 1 (int8 activations), 64 distinct matrices
    back to back in one CUDA graph so that weights come from HBM, not L2.  With other
    out/inn the same measurement on another shape; distinct=False launches ONE matrix nmat
    times (L2-resident after the first launch)."""
    lib = abi.lib
    tb = lib.rotor_b200_tiles_bytes(out, inn)
    tiles = torch.randint(0, 256, (nmat, tb), dtype=torch.uint8, device="cuda")
    tiles &= 0xAA  # codes {0, 2}: valid weights -1/+1; timing does not depend on the values
    kpad = lib.rotor_b200_in_padded(inn)
    xq = torch.randint(-127, 128, (1, kpad), dtype=torch.int8, device="cuda")
    xsum = xq.to(torch.int32).sum(1).to(torch.int32)
    acc = torch.empty((nmat, 1, out), dtype=torch.int32, device="cuda")
    st = torch.cuda.Stream()
    with torch.cuda.stream(st):
        s = st.cuda_stream

        def body():
            for i in range(nmat):
                w = tiles[i if distinct else 0]
                abi.check(lib.rotor_b200_bitlinear_acc(w.data_ptr(), out, inn, xq.data_ptr(), xsum.data_ptr(),
                                                       1, acc[i].data_ptr(), abi.VARIANT_AUTO, s), "gemv")
        body()
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=st):
            body()
        for _ in range(3):
            g.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(st)
        for _ in range(iters):
            g.replay()
        e1.record(st)
        torch.cuda.synchronize()
        sec = e0.elapsed_time(e1) * 1e-3 / (iters * nmat)
    alg = out * inn // 4 + inn + 4 * out + 4   # packed weights + int8 activations + int32 outputs + scale
    return alg, sec


def launch_floor(torch, abi, nlaunch=64, iters=20):
    """Seconds per launch of a chain of `nlaunch` empty kernels captured in one CUDA graph: what a chain
    of dependent launches costs on this device before any kernel does work (same launch attributes as
    the GEMV chain)."""
    lib = abi.lib
    st = torch.cuda.Stream()
    with torch.cuda.stream(st):
        s = st.cuda_stream

        def body():
            for _ in range(nlaunch):
                abi.check(lib.rotor_b200_launch_empty(s), "empty launch")
        body()
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=st):
            body()
        for _ in range(3):
            g.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(st)
        for _ in range(iters):
            g.replay()
        e1.record(st)
        torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e-3 / (iters * nlaunch)


def profile_figure(name, key):
    """A number recorded in a committed ncu summary under profiles/ as a line `key: value` (None if
    the file or the line is missing)."""
    path = os.path.join(ROOT, "profiles", name)
    try:
        with open(path) as f:
            for line in f:
                if line.strip().startswith(key + ":"):
                    return float(line.split(":", 1)[1].split()[0])
    except (OSError, ValueError):
        pass
    return None


def gemm_throughput(torch, abi, out=13824, inn=2560, m=16384, iters=5):
    """Config 4's dominant product: the stacked gate/up BitLinear of the 2B shape as an
    [m x inn] x [inn x out] ternary x int8 GEMM.  Returns (int8 ops per launch, seconds per launch)."""
    lib = abi.lib
    tiles = torch.randint(0, 256, (lib.rotor_b200_tiles_bytes(out, inn),), dtype=torch.uint8, device="cuda") & 0xAA
    kpad = lib.rotor_b200_in_padded(inn)
    xq = torch.randint(-127, 128, (m, kpad), dtype=torch.int8, device="cuda")
    xsum = xq.to(torch.int32).sum(1).to(torch.int32)
    acc = torch.empty((m, out), dtype=torch.int32, device="cuda")
    st = torch.cuda.Stream()
    with torch.cuda.stream(st):
        s = st.cuda_stream
        run = lambda: abi.check(lib.rotor_b200_bitlinear_acc(tiles.data_ptr(), out, inn, xq.data_ptr(), xsum.data_ptr(),
                                                             m, acc.data_ptr(), abi.VARIANT_AUTO, s), "gemm")
        for _ in range(3):
            run()
        st.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(st)
        for _ in range(iters):
            run()
        e1.record(st)
        st.synchronize()
    abi.device_status()
    return 2.0 * out * inn * m, e0.elapsed_time(e1) * 1e-3 / iters


def time_decode(torch, abi, handle, batch, prompt, W, K, graph, barrier, local):
    """Prefill `prompt` ([batch, len] int64), W warm-up steps, K timed steps on a private stream.
    Returns (seconds for the K steps, launches in the timed region, clocks, token checksum)."""
    import numpy as np
    n_prompt = prompt.shape[1]
    st = torch.cuda.Stream()
    with torch.cuda.stream(st):
        s = st.cuda_stream
        ids_d = torch.from_numpy(prompt).cuda()
        first = torch.empty(batch, dtype=torch.int64, device="cuda")
        abi.check(abi.lib.rotor_b200_model_forward(handle, ids_d.data_ptr(), batch, n_prompt, 0, abi.LOGITS_NONE, None,
                                                   first.data_ptr(), s), "prefill")
        abi.check(abi.lib.rotor_b200_model_decode_begin(handle, first.data_ptr(), batch, n_prompt, s), "begin")
        abi.check(abi.lib.rotor_b200_model_decode_steps(handle, W, int(graph), s), "warmup")
        barrier()
        sampler = ClockSampler(local)
        sampler.start()
        time.sleep(0.25)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        before = abi.lib.rotor_b200_launch_count()
        t0 = time.time()
        e0.record(st)
        abi.check(abi.lib.rotor_b200_model_decode_steps(handle, K, int(graph), s), "timed steps")
        e1.record(st)
        st.synchronize()
        barrier()
        t1 = time.time()
        clocks = sampler.stop(t0, t1)
        launches = abi.lib.rotor_b200_launch_count() - before
        sec = e0.elapsed_time(e1) * 1e-3
        toks = np.empty((W + K) * batch, dtype=np.int64)
        abi.check(abi.lib.rotor_b200_model_read_tokens(handle, 0, W + K, toks.ctypes.data, s), "read_tokens")
    abi.device_status()
    return sec, int(launches), clocks, int(toks.sum() % 1000003)


def measure_parity():
    """The GPU path against the CPU oracle on the same seeded weights: 2B dimensions, two layers, full
    vocabulary.  Float semantics (three int8 terms on the GPU): worst prompt-logit error over the
    logit RMS and greedy tokens equal.  Int8 semantics: the first position (nothing order dependent
    in front of a quantiser) and the worst position (rounding ties of the quantiser flip with float
    summation order; the oracle's own float32 and float64 evaluations are given beside it)."""
    import numpy as np
    from oracle import bitlinear_np as O
    from rotor_b200 import semantics
    from rotor_b200.synth import model_from_oracle_params
    cfg = dict(CFG_2B, n_layers=2)
    om = O.synth_model(cfg, 2026, fast_embed=True)
    prompt = np.random.default_rng(2027).integers(0, cfg["vocab_size"], size=8).astype(np.int64)

    def err(got, want):
        got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
        return np.max(np.abs(got - want), axis=-1) / np.sqrt(np.mean(want ** 2, axis=-1))
    model = model_from_oracle_params(om, semantics=semantics.REFERENCE, max_seq=32)
    want, _ = O.model_forward(om, prompt[None, :], O.REFERENCE)
    got, _ = model.forward(prompt[None, :])
    e_ref = err(got[0], want[0])
    n_new = 8
    want_ids = O.generate_greedy(om, prompt, n_new, O.REFERENCE)[len(prompt):]
    got_ids = model.generate_greedy(prompt, n_new)
    del model
    model = model_from_oracle_params(om, semantics=semantics.BASELINE, max_seq=32)
    w32, _ = O.model_forward(om, prompt[None, :], O.BASELINE)
    w64, _ = O.model_forward(om, prompt[None, :], O.with_semantics(O.BASELINE, glue64=True))
    g8, _ = model.forward(prompt[None, :])
    e8, s8 = err(g8[0], w32[0]), err(w64[0], w32[0])
    del model
    return {"config": "2B dimensions, 2 layers, vocabulary 128256, 8-token seeded prompt, same weights on both sides",
            "float_semantics": {"max_rel_err": float(e_ref.max()), "tolerance": 1e-3,
                                "greedy_tokens_equal": int(sum(a == b for a, b in zip(got_ids, want_ids))),
                                "greedy_tokens": n_new},
            "int8_semantics": {"first_position_rel_err": float(e8[0]), "worst_position_rel_err": float(e8.max()),
                               "oracle_float32_vs_float64_glue_worst": float(s8.max())}}


def measure_ffn_block(torch, with_cpu):
    """Config 2: the 2B-shape FFN block (pre-norm, gate/up BitLinear 2560 -> 6912, squared-ReLU gating,
    sub-norm over 6912, down BitLinear 6912 -> 2560) for 1 and 16 token rows.  64 blocks with distinct
    weights (850 MB > L2) run back to back in one CUDA graph."""
    from rotor_b200 import semantics
    from rotor_b200.transformer import GatedFFN, RMSNorm
    d, ff, nblk = 2560, 6912, 64
    blocks = []
    for i in range(nblk):
        f = GatedFFN(d, ff, semantics=semantics.BASELINE)
        for p in (f.gate_proj, f.up_proj, f.down_proj):
            p.load_from_int8(torch.randint(-1, 2, (p.out_features, p.in_features), device="cuda", dtype=torch.int8), 0.016)
        blocks.append(f)
    pre = RMSNorm(d, eps=semantics.BASELINE.eps)
    peak, peak_kind = measured_peak_gbs()
    out = {"metric": "2B-shape FFN block time", "unit": "us per block", "higher_is_better": False, "data": "synthetic",
           "config": {"workload": "RMSNorm + gate/up 2560->6912 + relu^2 gating + sub-norm + down 6912->2560, "
                                  "64 distinct blocks per graph replay"}, "rows": {}}
    st = torch.cuda.Stream()
    for m in (1, 16):
        x = torch.randn(m, d, device="cuda")
        with torch.cuda.stream(st):
            for f in blocks:          # every block once outside the capture: device copies of the norm weights
                f.forward_device(x, pre_norm=pre)
            st.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=st):
                for f in blocks:
                    y = f.forward_device(x, pre_norm=pre)
            for _ in range(3):
                g.replay()
            st.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(st)
            for _ in range(10):
                g.replay()
            e1.record(st)
            st.synchronize()
        us = e0.elapsed_time(e1) * 1e3 / (10 * nblk)
        alg = 3 * d * ff // 4 + (2 * d + ff) * 4 + 2 * m * d * 4    # tiles + norm weights + rows in and out
        out["rows"][str(m)] = {"us_per_block": us, "algorithmic_bytes": alg, "achieved_gbs": alg / us / 1e3,
                               "frac_of_peak": alg / us / 1e3 / peak}
    out["peak_kind"] = peak_kind
    if with_cpu:
        out["cpu_baseline"] = cpu_layer_samples()
    return out


def measure_prefill(torch, abi, model, B, S, K, W, local=0):
    """Prompt prefill of the 2B shape through the whole model: tiled tensor-core BitLinear products,
    tiled attention, LM head on the last position."""
    import numpy as np
    cfg = model.config
    h = model._ensure_handle(B, S, S).h
    ids = torch.from_numpy(np.random.default_rng(5).integers(0, cfg["vocab_size"], size=(B, S))).cuda()
    nxt = torch.empty(B, dtype=torch.int64, device="cuda")
    st = torch.cuda.Stream()
    with torch.cuda.stream(st):
        s = st.cuda_stream
        run = lambda: abi.check(abi.lib.rotor_b200_model_forward(h, ids.data_ptr(), B, S, 0, abi.LOGITS_NONE, None,
                                                                 nxt.data_ptr(), s), "prefill")
        for _ in range(W):
            run()
        st.synchronize()
        sampler = ClockSampler(local)
        sampler.start()
        time.sleep(0.25)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        before = abi.lib.rotor_b200_launch_count()
        t0 = time.time()
        e0.record(st)
        for _ in range(K):
            run()
        e1.record(st)
        st.synchronize()
        t1 = time.time()
        clocks = sampler.stop(t0, t1)
        launches = abi.lib.rotor_b200_launch_count() - before
    abi.device_status()
    sec = e0.elapsed_time(e1) * 1e-3 / K
    d, ff, L = cfg["d_model"], cfg["d_ff"], cfg["n_layers"]
    hd = d // cfg["n_heads"]
    macs = (cfg["n_heads"] * hd + 2 * cfg["n_kv_heads"] * hd) * d + d * cfg["n_heads"] * hd + 3 * ff * d
    int8_ops = 2.0 * B * S * macs * L
    attn_flops = 4.0 * B * cfg["n_heads"] * S * S * hd * L / 2   # causal: half of the score matrix
    ops1, gsec = gemm_throughput(torch, abi, m=B * S)
    return {"metric": "2B-shape prompt prefill tokens/s", "value": B * S / sec, "unit": UNIT, "n_gpus": 1, "steps": K,
            "warmup": W, "ms_per_step": sec * 1e3, "higher_is_better": True, "data": "synthetic",
            "config": {"workload": f"{L}-layer 2B-shape model, batch {B} x {S} positions, causal, last-position pick"},
            "bitlinear_int8_ops": int8_ops, "attention_flops": attn_flops,
            "if_all_time_were_bitlinear_TOPS": int8_ops / sec / 1e12,
            "gate_up_gemm": {"shape": [13824, 2560, B * S], "ms": gsec * 1e3, "int8_tops": ops1 / gsec / 1e12,
                             "frac_of_nominal_4500": ops1 / gsec / 4.5e15,
                             "tensor_pipe_active_pct_ncu": profile_figure("gemm_tcgen05_kernel_13824x2560_m4096.md",
                                                                          "tensor_pipe_active_pct")},
            "gpu_launches": int(launches), "clocks": clocks}


def measure_xl(torch, abi, rank, world, group, batches, K, W, barrier, local, layers=0, graph=1):
    """The 80-layer d 8192 / FFN 28672 shape decoding after a 1024-token prompt: unsharded on one GPU, or
    sharded tensor-parallel over the `world` ranks of `group` (strong scaling: every rank works on every
    token).  One record per batch size."""
    import numpy as np
    import torch.distributed as dist
    from rotor_b200 import semantics
    from rotor_b200.synth import XL_TP, random_model_on_device
    from rotor_b200.tensor_parallel import ShardedBitNetModel
    cfg = dict(XL_TP)
    if layers:
        cfg["n_layers"] = layers
    sem = semantics.BASELINE
    max_seq = XL_PROMPT_LEN + 1 + W + K + 8
    b0 = batches[0]
    if world > 1:
        model = ShardedBitNetModel(cfg, group, semantics=sem, max_seq=max_seq, max_batch=b0, max_rows=b0 * XL_PROMPT_LEN)
        model.load_random(seed=4321)
    else:
        model = random_model_on_device(cfg, seed=4321, semantics=sem, max_seq=max_seq, max_batch=b0,
                                       max_rows=b0 * XL_PROMPT_LEN)
    peak, peak_kind = measured_peak_gbs()
    out = {"config": {"workload": f"random-init {cfg['n_layers']}-layer d {cfg['d_model']} ffn {cfg['d_ff']} "
                                  f"{cfg['n_heads']}q/{cfg['n_kv_heads']}kv model, vocab {cfg['vocab_size']}, greedy decode "
                                  f"after a {XL_PROMPT_LEN}-token prompt", "parallelism": f"tp{world}",
                      "cuda_graph": bool(graph)},
           "n_gpus": world, "scaling": "strong", "steps": K, "warmup": W, "unit": UNIT, "peak_kind": peak_kind,
           "exchanges_per_token": (5 * cfg["n_layers"] + 1) if world > 1 else 0,
           "transport": ("in-kernel peer-memory exchange (one 64-bit store per value and peer) for step payloads, "
                         "NCCL for prefill payloads and the pick" if world > 1 else "none"),
           "batch": {}}
    for B in batches:
        h = model._ensure_handle(B, XL_PROMPT_LEN, max_seq)
        handle = h if world > 1 else h.h
        prompt = np.random.default_rng(7).integers(0, cfg["vocab_size"], size=(B, XL_PROMPT_LEN)).astype(np.int64)
        sec, launches, clocks, checksum = time_decode(torch, abi, handle, B, prompt, W, K, graph, barrier, local)
        if world > 1:
            t = torch.tensor([sec], dtype=torch.float64, device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            sec = float(t[0])
        ctx = XL_PROMPT_LEN + 1 + W + K // 2
        weights = algorithmic_bytes_per_token(cfg, 0)                      # read once per step whatever the batch
        kv = (algorithmic_bytes_per_token(cfg, ctx) - weights) * B
        per_gpu = (weights + kv) / world
        out["batch"][str(B)] = {"tokens_per_s": B * K / sec, "ms_per_step": sec * 1e3 / K,
                                "algorithmic_bytes_per_step_per_gpu": per_gpu,
                                "achieved_gbs_per_gpu": per_gpu * K / sec / 1e9,
                                "frac_of_peak_per_gpu": per_gpu * K / sec / 1e9 / peak,
                                "gpu_launches": launches, "clocks": clocks, "token_checksum": checksum}
    del model
    torch.cuda.empty_cache()
    return out


def guarded(name, fn, line):
    """Runs one secondary section; a failure there is recorded instead of losing the headline."""
    try:
        line[name] = fn()
    except Exception as e:  # noqa: BLE001 - the record says what went wrong
        line[name] = {"error": f"{type(e).__name__}: {e}"[:300]}


def run_b200(args, rank, world):
    import numpy as np
    import torch
    import torch.distributed as dist
    from rotor_b200 import abi, semantics
    from rotor_b200.generation import TextGenerator
    from rotor_b200.synth import PassThroughTokenizer, random_model_on_device

    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    K, W = args.steps, max(args.warmup, 3)
    total_new = 1 + W + K                       # first token comes out of the prefill
    max_seq = PROMPT_LEN + total_new + 8
    model = random_model_on_device(CFG_2B, seed=1234 + rank, semantics=semantics.BASELINE, max_seq=max_seq,
                                   max_rows=PROMPT_LEN)
    rng = np.random.default_rng(99 + rank)
    prompt = rng.integers(0, CFG_2B["vocab_size"], size=PROMPT_LEN).astype(np.int64)

    # ---- device-resident timing (value)
    h = model._ensure_handle(1, PROMPT_LEN, max_seq)
    sec, launches, clocks, _ = time_decode(torch, abi, h.h, 1, prompt.reshape(1, -1), W, K, 1, barrier, local)

    if args.only == "decode":
        print(json.dumps({"only": "decode", "tokens_per_s": K / sec, "gpu_launches": int(launches)}), flush=True)
        return

    # ---- end to end through the public API (host prompt in, tokens to the host every step)
    tok = PassThroughTokenizer()
    text = " ".join(map(str, prompt))
    gen = TextGenerator(model, tok, max_length=PROMPT_LEN + 1 + W + K, use_cache=True, readback_chunk=1)
    stamps = []
    gen.generate(text, max_new_tokens=4, stop_on_eos=False)            # warm: graph already built
    barrier()
    t0 = time.perf_counter()
    gen.generate(text, max_new_tokens=1 + W + K, stop_on_eos=False, callback=lambda _t: stamps.append(time.perf_counter()))
    torch.cuda.synchronize()
    t_end = time.perf_counter()
    e2e_sec = stamps[-1] - stamps[W]           # the last K tokens of the call, as seen by the host callback
    e2e_total = t_end - t0

    secs = torch.tensor([sec, e2e_sec, e2e_total], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(secs, op=dist.ReduceOp.MAX)
    sec, e2e_sec, e2e_total = [float(v) for v in secs.cpu()]

    peak, peak_kind = measured_peak_gbs()
    line = None
    if rank == 0:
        alg, gsec = gemv_roofline(torch, abi)
        _, gsec_l2 = gemv_roofline(torch, abi, distinct=False)
        floor = launch_floor(torch, abi)
        alg_l, gsec_l = gemv_roofline(torch, abi, nmat=8, iters=10, out=28672, inn=8192)
        ctx_mid = PROMPT_LEN + 1 + W + K // 2
        step_bytes = algorithmic_bytes_per_token(CFG_2B, ctx_mid)
        ternary = CFG_2B["n_layers"] * ((2560 + 2 * 640) * 2560 + 2560 * 2560 + 3 * 6912 * 2560) // 4
        share = profile_figure("decode_step_2b_launch_list.md", "fused_gemv_share")
        line = {
            "metric": METRIC, "value": world * K / sec, "unit": UNIT, "n_gpus": world, "steps": K, "warmup": W,
            "ms_per_step": sec * 1e3 / K, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "int8 activations x ternary weights -> int32 (float32 glue, bf16 LM head)", "data": "synthetic",
            "semantics": SEM_GPU,
            "config": {"workload": WORKLOAD, "global_batch": world, "prompt_len": PROMPT_LEN},
            "parallelism": "single GPU" if world == 1 else f"{world} independent replicas (the 2B shape's 20 / 5 heads do not "
                                                          "shard 2/4/8-way); the sharded shape is under xl_tp",
            "l2": "inputs larger than L2 (1.18 GB of weights per step)",
            "e2e": {"value": world * K / e2e_sec, "unit": UNIT,
                    "h2d_bytes_per_step": PROMPT_LEN * 8 / (1 + W + K), "d2h_bytes_per_step": 8,
                    "call": "TextGenerator.generate (host string in, per-token ids out)",
                    "whole_call_tokens_per_s": world * (1 + W + K) / e2e_total},
            "gpu_launches": int(launches),
            "clocks": clocks,
            "roofline": {"bound": "hbm", "kernel": "fused_gemv_kernel as the stand-alone product (ternary GEMV 2560->6912, batch 1, tiles staged in shared memory)",
                         "achieved": alg / gsec / 1e9, "peak": peak, "unit": "GB/s", "frac": alg / gsec / 1e9 / peak,
                         "peak_kind": f"{peak_kind} HBM copy bandwidth",
                         # dram read + write per launch from the committed ncu capture (None if not recorded)
                         "traffic": profile_figure("fused_gemv_kernel_2560x6912_gemv.md", "traffic_bytes_per_launch"),
                         "bytes_per_launch": alg, "us_per_launch": gsec * 1e6,
                         "launch_floor_us": floor * 1e6,
                         "hbm_time_us": alg / (peak * 1e9) * 1e6,
                         "note": "64 distinct matrices per graph (283 MB > L2), one launch per matrix; launch_floor_us is a "
                                 "chain of empty kernels in the same harness: the part of us_per_launch no kernel can remove"},
            "roofline_l2_resident": {"kernel": "the same chain of 64 launches on ONE matrix (4.4 MB, L2-resident: not an HBM figure)",
                                     "achieved": alg / gsec_l2 / 1e9, "unit": "GB/s", "us_per_launch": gsec_l2 * 1e6},
            "roofline_large_matrix": {"kernel": "bitlinear_acc_kernel (ternary GEMV 8192->28672, batch 1; 8 distinct 58.7 MB matrices)",
                                      "achieved": alg_l / gsec_l / 1e9, "peak": peak, "unit": "GB/s",
                                      "frac": alg_l / gsec_l / 1e9 / peak, "bytes_per_launch": alg_l,
                                      "us_per_launch": gsec_l * 1e6},
            "step_roofline": {"algorithmic_bytes_per_token": step_bytes, "achieved_gbs": step_bytes * K / sec / 1e9,
                              "frac_of_peak": step_bytes * K / sec / 1e9 / peak},
        }
        if share:
            t_fused = share * sec / K
            line["roofline_step"] = {"bound": "hbm", "kernel": "fused_gemv_kernel (the four products of every block, "
                                                               "120 launches per token)",
                                     "bytes_per_token": ternary, "share_of_step_ncu": share,
                                     "achieved": ternary / t_fused / 1e9, "peak": peak, "unit": "GB/s",
                                     "frac": ternary / t_fused / 1e9 / peak}
    # ---- the other configurations (secondary records; the headline above is complete without them)
    full = args.only == "all" and not args.quick
    if world == 1 and full:
        guarded("parity", measure_parity, line)
        guarded("ffn_block", lambda: measure_ffn_block(torch, False), line)
        guarded("prefill_2b", lambda: measure_prefill(torch, abi, model, 8, 2048, 2, 1), line)
    del gen, model, h
    torch.cuda.empty_cache()
    if world == 1 and full:
        guarded("xl", lambda: measure_xl(torch, abi, 0, 1, None, [1, 64], 16, 3, barrier, local), line)
    if world > 1 and full:
        from rotor_b200.tensor_parallel import TPGroup
        group, rec = None, None
        try:
            group = TPGroup()
            rec = measure_xl(torch, abi, rank, world, group, [1, 8, 64], 16, 3, barrier, local)
        except Exception as e:  # noqa: BLE001
            rec = {"error": f"{type(e).__name__}: {e}"[:300]}
        finally:
            if group is not None:
                group.close()
        if rank == 0:
            line["xl_tp"] = rec
    if rank == 0:
        if world == 1 and not args.no_cpu_baseline:
            tps, threads, done = cpu_decode_sample(6, 1, budget_s=40.0)
            line["cpu_baseline"] = {"value": tps, "unit": UNIT, "cores": threads, "kind": "port", "semantics": SEM_CPU,
                                    "sample": f"{done} timed one-token steps (+1 warm-up), full 30-layer 2B-shape model, "
                                              f"NumPy oracle port of the reference path, KV cache pre-filled at {PROMPT_LEN}"}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_prefill(args, rank, world):
    """--workload prefill_2b: the prefill record alone."""
    import torch
    from rotor_b200 import abi, semantics
    from rotor_b200.synth import random_model_on_device
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    B, S = args.batch or 8, args.seq or 2048
    cfg = dict(CFG_2B)
    if args.layers:
        cfg["n_layers"] = args.layers
    model = random_model_on_device(cfg, seed=77, semantics=semantics.BASELINE, max_seq=S, max_batch=B, max_rows=B * S)
    print(json.dumps(measure_prefill(torch, abi, model, B, S, args.steps, max(args.warmup, 1), local)), flush=True)


def cpu_layer_samples():
    """The reference's CPU path (NumPy port in oracle/) on this box's host cores for the single layer of
    config 1 and the FFN block of config 2: median of 10 calls after 2 warm-up calls."""
    import numpy as np
    from oracle import bitlinear_np as O
    rng = np.random.default_rng(11)
    d, ff = 2560, 6912
    lw = {"gate": (O.synth_ternary(rng, ff, d), 0.016), "up": (O.synth_ternary(rng, ff, d), 0.016),
          "down": (O.synth_ternary(rng, d, ff), 0.016), "ffn_sub_norm": np.ones(ff, np.float32)}
    pre = np.ones(d, np.float32)

    def med(fn):
        ts = []
        for i in range(12):
            t0 = time.perf_counter()
            fn()
            if i >= 2:
                ts.append(time.perf_counter() - t0)
        return statistics.median(ts) * 1e6
    out = {}
    x1 = rng.standard_normal((1, d)).astype(np.float32)
    out["bitlinear_2560x6912_m1_us"] = med(lambda: O.bitlinear(x1, lw["gate"][0], lw["gate"][1], O.REFERENCE))
    for m in (1, 16):
        x = rng.standard_normal((m, d)).astype(np.float32)
        out[f"ffn_block_m{m}_us"] = med(lambda: O.ffn(O.rmsnorm(x, pre, 1e-5), lw, O.REFERENCE))
    try:
        from threadpoolctl import threadpool_info
        out["cores"] = max([p.get("num_threads", 1) for p in threadpool_info()] or [os.cpu_count() or 1])
    except Exception:
        out["cores"] = os.cpu_count() or 1
    out["kind"] = "port"
    return out


def run_ffn_block(args):
    """--workload ffn_block: the FFN-block record alone."""
    import torch
    torch.cuda.set_device(0)
    print(json.dumps(measure_ffn_block(torch, not args.no_cpu_baseline)), flush=True)


def run_xl_tp(args, rank, world):
    """--workload xl_tp: the 80-layer shape alone, sharded over `world` GPUs (1 = unsharded)."""
    import torch
    import torch.distributed as dist
    from rotor_b200 import abi
    from rotor_b200.tensor_parallel import TPGroup
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    group = None
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        group = TPGroup()

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
    batches = [args.batch] if args.batch else [1, 8, 64]
    rec = measure_xl(torch, abi, rank, world, group, batches, args.steps, max(args.warmup, 3), barrier, local,
                     layers=args.layers, graph=args.graph)
    if rank == 0:
        print(json.dumps(dict(rec, metric="XL-shape greedy decode tokens/s (tensor parallel)", data="synthetic",
                              higher_is_better=True)), flush=True)
    if group is not None:
        group.close()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--quick", action="store_true", help="headline sections only (no parity / FFN / prefill / XL records)")
    ap.add_argument("--only", default="all", choices=["all", "decode", "gemv", "gemm"],
                    help="profiling aid: run only the device-resident decode section, the GEMV section, or one "
                         "prefill GEMM (--m tokens)")
    ap.add_argument("--m", type=int, default=16384, help="--only gemm: activation columns (tokens)")
    ap.add_argument("--workload", default="decode_2b", choices=["decode_2b", "xl_tp", "prefill_2b", "ffn_block"],
                    help="decode_2b: the headline line; xl_tp: the tensor-parallel XL shape (separate line)")
    ap.add_argument("--batch", type=int, default=0, help="prefill_2b: sequences (0 = 8); xl_tp: sequences (0 = 1)")
    ap.add_argument("--seq", type=int, default=0, help="prefill_2b: positions per sequence (0 = 2048)")
    ap.add_argument("--layers", type=int, default=0, help="xl_tp: override the layer count (0 = 80)")
    ap.add_argument("--graph", type=int, default=1, help="xl_tp: replay the step as a CUDA graph (1) or launch it (0)")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    if args.only == "gemv":
        import torch
        from rotor_b200 import abi
        torch.cuda.set_device(0)
        alg, gsec = gemv_roofline(torch, abi)
        print(json.dumps({"only": "gemv", "bytes_per_launch": alg, "us_per_launch": gsec * 1e6,
                          "gbs": alg / gsec / 1e9}), flush=True)
        return
    if args.only == "gemm":
        import torch
        from rotor_b200 import abi
        torch.cuda.set_device(0)
        ops, sec = gemm_throughput(torch, abi, m=args.m)
        print(json.dumps({"only": "gemm", "shape": [13824, 2560, args.m], "ms_per_launch": sec * 1e3,
                          "int8_tops": ops / sec / 1e12}), flush=True)
        return
    if args.impl == "reference":
        run_reference(args, rank)
    elif args.workload == "xl_tp":
        run_xl_tp(args, rank, world)
    elif args.workload == "ffn_block":
        if rank == 0:
            run_ffn_block(args)
    elif args.workload == "prefill_2b":
        if rank == 0:
            run_prefill(args, rank, world)
    else:
        run_b200(args, rank, world)


if __name__ == "__main__":
    main()
