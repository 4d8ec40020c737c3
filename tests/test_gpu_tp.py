"""GPU, two ranks on two GPUs and four on four (skipped on a smaller box): the tensor-parallel model through
the C ABI against the single-device oracle.  Each rank checks its vocabulary slice of the
logits (tolerance: max-abs error below 1e-3 of the output RMS) and that greedy generation,
launch by launch and as a replayed CUDA graph, yields the oracle's tokens."""
import os
import socket

import numpy as np
import pytest

import golden_inputs as G
from oracle import bitlinear_np as O

pytestmark = pytest.mark.gpu
TOL = 1e-3


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, port, out_dir, name, WORLD, env=None):
    os.environ.update(env or {})
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    import torch
    import torch.distributed as dist
    from rotor_b200.semantics import BASELINE
    from rotor_b200.tensor_parallel import ShardedBitNetModel, TPGroup
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", rank=rank, world_size=WORLD)
    group = None
    try:
        group = TPGroup()
        om, prompt = G.tiny_model(name)
        model = ShardedBitNetModel(om["cfg"], group, semantics=BASELINE.with_(act_terms=1), max_seq=64)
        model.load_from_params(om)
        logits = model.forward(prompt[None, :])                      # [1, S, V/WORLD]
        last = model.forward(prompt[None, :], logits_positions="last")
        from rotor_b200 import abi
        before = abi.lib.rotor_b200_launch_count()
        eager = model.generate_greedy(prompt, G.N_NEW, use_graph=False)
        per_step = (abi.lib.rotor_b200_launch_count() - before) / G.N_NEW
        graph = model.generate_greedy(prompt, G.N_NEW, use_graph=True)
        torch.cuda.synchronize()
        np.savez(os.path.join(out_dir, f"rank{rank}.npz"), logits=logits, last=last, eager=np.array(eager),
                 graph=np.array(graph), per_step=per_step)
        del model
    finally:
        if group is not None:
            group.close()
        dist.destroy_process_group()


@pytest.mark.parametrize("name,WORLD,nccl_only", [("hd128", 2, False), ("wide_tp", 2, False), ("tp4", 4, False),
                                                  ("hd128", 2, True)])
def test_sharded_model_matches_oracle(tmp_path, name, WORLD, nccl_only):
    """nccl_only: ROTOR_B200_TP_NCCL=1 keeps every exchange on NCCL (no peer-memory exchange, hence no
    in-kernel exchanges and the unfused generation step); the results stay the same."""
    import torch
    if torch.cuda.device_count() < WORLD:
        pytest.skip(f"needs {WORLD} GPUs")
    import torch.multiprocessing as mp
    env = {"ROTOR_B200_TP_NCCL": "1"} if nccl_only else None
    mp.spawn(_worker, args=(_free_port(), str(tmp_path), name, WORLD, env), nprocs=WORLD, join=True)
    om, prompt = G.tiny_model(name)
    sem = O.with_semantics(O.BASELINE, act_terms=1)
    want, _ = O.model_forward(om, prompt[None, :], sem)
    ids = O.generate_greedy(om, prompt, G.N_NEW, sem)[len(prompt):]
    vl = om["cfg"]["vocab_size"] // WORLD
    rms = np.sqrt(np.mean(np.asarray(want, np.float64) ** 2))
    for r in range(WORLD):
        got = np.load(tmp_path / f"rank{r}.npz")
        ref = want[:, :, r * vl:(r + 1) * vl]
        assert np.max(np.abs(got["logits"] - ref)) / rms < TOL
        assert np.max(np.abs(got["last"][:, 0] - ref[:, -1])) / rms < TOL
        assert list(got["eager"]) == ids
        assert list(got["graph"]) == ids
        # generation steps take the seven-launch block with in-kernel exchanges (+ LM head, pick, advance, bump)
        if nccl_only:
            assert float(got["per_step"]) > 7 * om["cfg"]["n_layers"] + 8
        else:
            assert float(got["per_step"]) <= 7 * om["cfg"]["n_layers"] + 8
