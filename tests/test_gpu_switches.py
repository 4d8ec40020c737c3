"""GPU: every environment switch the library reads selects a path that gives the same results.

The switches are read once per process, so each case runs in a child process with the switch
set.  The child drives the tiny head_dim-128 model through a prompt, a 150-position batch-2
prefill (row-wise stages, tiled GEMM, prefill attention, many-row LM head) and 32 greedy steps,
eager and as a replayed CUDA graph, and compares with the oracle: floating outputs to 1e-3 of
the output RMS, tokens equal."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

_ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

_CHILD = r'''
import sys, numpy as np
sys.path[:0] = [%r, %r, %r]
import golden_inputs as G
from oracle import bitlinear_np as O
from rotor_b200 import abi, semantics, synth

def rel_err(a, b):
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    return float(np.max(np.abs(a - b)) / np.sqrt(np.mean(b ** 2)))

om, prompt = G.tiny_model("hd128")
model = synth.model_from_oracle_params(om, semantics=semantics.REFERENCE, max_seq=256, max_batch=2)
want, _ = O.model_forward(om, prompt[None, :], O.REFERENCE)
got, _ = model.forward(prompt[None, :])
assert rel_err(got, want) < 1e-3, rel_err(got, want)

rng = np.random.default_rng(77)
ids = rng.integers(0, om["cfg"]["vocab_size"], size=(2, 150))
want, _ = O.model_forward(om, ids, O.REFERENCE)
got, _ = model.forward(ids)
assert rel_err(got, want) < 1e-3, rel_err(got, want)

tokens = O.generate_greedy(om, prompt, G.N_NEW, O.REFERENCE)[len(prompt):]
before = abi.lib.rotor_b200_launch_count()
assert model.generate_greedy(prompt, G.N_NEW, use_graph=False) == tokens
per_step = (abi.lib.rotor_b200_launch_count() - before) / G.N_NEW
assert model.generate_greedy(prompt, G.N_NEW, use_graph=True) == tokens
abi.device_status()
print("per_step", per_step)
print("ok")
''' % (_ROOT, os.path.join(_ROOT, "rotor-rag_b200"), os.path.join(_ROOT, "tests"))


def _run(env_extra):
    env = dict(os.environ, **env_extra)
    r = subprocess.run([sys.executable, "-c", _CHILD], env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and r.stdout.strip().endswith("ok"), (r.stdout[-500:], r.stderr[-2000:])
    return float(r.stdout.split("per_step")[1].split()[0])


@pytest.fixture(scope="module")
def default_launches():
    return _run({})


@pytest.mark.parametrize("switch", [
    {"ROTOR_B200_NO_FUSED_STEP": "1"},    # generation steps through the unfused kernels
    {"ROTOR_B200_PDL": "0"},              # no programmatic dependent launch between the step's kernels
    {"ROTOR_B200_NO_TCGEN05": "1"},       # mma.sync GEMM and attention instead of the tcgen05 kernels
    {"ROTOR_B200_NO_ROWSTAGE": "1"},      # the generation-step vector stage for prefill rows
    {"ROTOR_B200_NO_LMHEAD_MMA": "1"},    # the few-row LM head kernel for many rows
], ids=lambda s: next(iter(s)))
def test_switch_keeps_results(switch, default_launches):
    per_step = _run(switch)
    if "ROTOR_B200_NO_FUSED_STEP" in switch:
        assert per_step > default_launches      # the switch did select the other path
    else:
        assert per_step == default_launches
