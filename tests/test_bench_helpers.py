"""CPU: the figures bench.py reads from the committed ncu summaries are there and sane, and its
byte counts follow the formulas it documents."""
import importlib.util
import os

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _bench():
    spec = importlib.util.spec_from_file_location("bench_module", os.path.join(ROOT, "bench.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_profile_figures_present():
    b = _bench()
    share = b.profile_figure("decode_step_2b_launch_list.md", "fused_gemv_share")
    assert share is not None and 0.3 < share < 1.0
    traffic = b.profile_figure("fused_gemv_kernel_2560x6912_gemv.md", "traffic_bytes_per_launch")
    alg = 6912 * 2560 // 4 + 2560 + 4 * 6912 + 4          # config 1: packed weights + activations + sums + scale
    assert traffic is not None and alg <= traffic < 1.1 * alg
    tensor = b.profile_figure("gemm_tcgen05_kernel_13824x2560_m4096.md", "tensor_pipe_active_pct")
    assert tensor is not None and 0.0 < tensor <= 100.0
    assert b.profile_figure("no_such_file.md", "x") is None
    assert b.profile_figure("decode_step_2b_launch_list.md", "no_such_key") is None
