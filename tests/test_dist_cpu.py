"""Host-side logic of the expert-parallel path on CPU ranks (gloo, world_size 2 and 4): the contiguous
expert partition, identical routing on every rank, and the sum of the per-rank partials — the exchange
step the GPU path performs with NCCL — with the oracle standing in for the device kernels."""
import os
import socket

import numpy as np
import pytest

torch = pytest.importorskip("torch")
import torch.distributed as dist  # noqa: E402
import torch.multiprocessing as mp  # noqa: E402


def expert_range(rank, world, n_experts):
    """The reference's contiguous partition (getp-csrc/src/parallelism.cpp:1852-1855)."""
    per = n_experts // world
    return rank * per, (rank + 1) * per


def _worker(rank, world, port, out_path):
    import sys
    from pathlib import Path
    root = Path(__file__).resolve().parent.parent
    sys.path[:0] = [str(root), str(root / "tests")]
    import __graft_entry__ as entry
    entry.load_package()
    import oracle_lib
    from gptoss_b200 import synth

    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    H, I, E, k, T = 64, 48, 8, 2, 50
    ora = oracle_lib.oracle()
    w = synth.MoELayerWeights(H, I, E, 17, sigma=0.05)
    t = synth.activations(17, T, H)  # replicated activations: every rank holds all tokens
    scores = ora.router_scores(t, w.router_w, w.router_b)
    tw, ti, _, _ = ora.topk_softmax(scores, k)
    # every rank must derive the same routing
    ids = [torch.empty(T, k, dtype=torch.int32) for _ in range(world)]
    dist.all_gather(ids, torch.from_numpy(ti))
    assert all(torch.equal(ids[0], x) for x in ids)
    e0, e1 = expert_range(rank, world, E)
    part = ora.moe_block(t, tw, ti, w, mode=oracle_lib.MODE_GPU_BF16, e_begin=e0, e_end=e1)
    red = torch.from_numpy(part.copy())
    dist.all_reduce(red)  # the combine exchange
    full = ora.moe_block(t, tw, ti, w, mode=oracle_lib.MODE_GPU_BF16)
    err = float(np.linalg.norm(red.numpy() - full) / np.linalg.norm(full))
    # timing reduction used by the bench: max over ranks
    tm = torch.tensor([float(rank + 1)])
    dist.all_reduce(tm, op=dist.ReduceOp.MAX)
    if rank == 0:
        np.save(out_path, np.array([err, float(tm.item())]))
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_expert_parallel_partials_reduce_to_the_full_block(world, tmp_path):
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    out = tmp_path / "res.npy"
    mp.spawn(_worker, args=(world, port, str(out)), nprocs=world, join=True)
    err, tmax = np.load(out)
    assert err < 1e-6
    assert tmax == world


def test_partition_covers_all_experts_once():
    for world in (1, 2, 4, 8):
        for E in (32, 128):
            r = [expert_range(i, world, E) for i in range(world)]
            assert r[0][0] == 0 and r[-1][1] == E
            assert all(r[i][1] == r[i + 1][0] for i in range(world - 1))
