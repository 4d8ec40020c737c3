"""CPU, two and four gloo ranks: the tensor-parallel split (row / column shards, shared row maximum,
integer all-reduce, sharded sub-norm, vocabulary-sharded pick) reproduces the single-device
oracle.  The collectives are torch.distributed over gloo on 127.0.0.1; the arithmetic is the
NumPy restatement in oracle/tp_np.py fed by rotor_b200.tensor_parallel.shard_layer, the same
shard function the GPU ranks load their weights with."""
import os
import socket

import numpy as np
import pytest

import golden_inputs as G
from oracle import bitlinear_np as O

WORLD = 2
N_NEW = 4


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, port, out_dir, name, WORLD):
    import torch
    import torch.distributed as dist
    from oracle import tp_np
    from rotor_b200.tensor_parallel import local_dims, shard_layer
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=WORLD)
    try:
        def allreduce(a, op):
            t = torch.from_numpy(np.ascontiguousarray(a).copy())
            dist.all_reduce(t, op=dist.ReduceOp.SUM if op == "sum" else dist.ReduceOp.MAX)
            return t.numpy()

        def allgather(pair):
            got = [None] * WORLD
            dist.all_gather_object(got, pair)
            return got

        om, prompt = G.tiny_model(name)
        cfg = om["cfg"]
        sem = O.with_semantics(O.BASELINE, act_terms=1)
        ld = local_dims(cfg, WORLD)
        shards = [shard_layer(lw, cfg, rank, WORLD) for lw in om["layers"]]
        ids, caches, slices, picks = prompt[None, :], None, [], []
        for _ in range(N_NEW):
            logits, caches = tp_np.model_forward_tp(om, shards, ld, rank, ids, sem, allreduce, caches)
            slices.append(logits[0, -1].astype(np.float32))
            tok = tp_np.pick_tp(logits[0, -1], rank, ld["vocab"], allgather)
            picks.append(tok)
            ids = np.array([[tok]], dtype=np.int64)
        np.savez(os.path.join(out_dir, f"rank{rank}.npz"), logits=np.stack(slices), picks=np.array(picks))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("name,world", [("hd128", 2), ("tp4", 4)])
def test_rank_split_matches_single_device_oracle(tmp_path, name, world):
    import torch.multiprocessing as mp
    mp.spawn(_worker, args=(_free_port(), str(tmp_path), name, world), nprocs=world, join=True)
    om, prompt = G.tiny_model(name)
    sem = O.with_semantics(O.BASELINE, act_terms=1)
    ids, want = O.generate_greedy(om, prompt, N_NEW, sem, return_logits=True)
    got = [np.load(tmp_path / f"rank{r}.npz") for r in range(world)]
    full = np.concatenate([g["logits"] for g in got], axis=1)  # vocabulary slices side by side
    for step in range(N_NEW):
        ref = np.asarray(want[step], np.float64)
        err = np.max(np.abs(full[step] - ref)) / np.sqrt(np.mean(ref ** 2))
        assert err < 1e-4, (step, err)  # integer parts are exact; only the sharded sub-norm sum reorders
    for g in got:
        assert list(g["picks"]) == ids[len(prompt):]


def test_shard_layer_partitions_every_matrix():
    from rotor_b200.tensor_parallel import local_dims, shard_layer
    om, _ = G.tiny_model("hd128")
    cfg, lw = om["cfg"], om["layers"][0]
    parts = [shard_layer(lw, cfg, r, WORLD) for r in range(WORLD)]
    for name in ("q", "k", "v", "gate", "up"):
        assert np.array_equal(np.concatenate([p[name][0] for p in parts], axis=0), lw[name][0])
    for name in ("o", "down"):
        assert np.array_equal(np.concatenate([p[name][0] for p in parts], axis=1), lw[name][0])
    assert np.array_equal(np.concatenate([p["ffn_sub_norm"] for p in parts]), lw["ffn_sub_norm"])
    with pytest.raises(ValueError):
        local_dims(cfg, 3)
