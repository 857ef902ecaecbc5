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


def _owner_worker(rank, world, port, out_path):
    """The owner-addressed exchange of the GPU path, with gloo collectives standing in for the peer stores: every rank
    computes the pair rows of its own experts, each row goes to the rank that owns the row's token, the owner sums
    the k slots of its tokens in slot order, and (replicated form) the sums are gathered back to every rank."""
    import sys
    from pathlib import Path
    root = Path(__file__).resolve().parent.parent
    sys.path[:0] = [str(root), str(root / "tests")]
    import __graft_entry__ as entry
    entry.load_package()
    import oracle_lib
    from gptoss_b200 import moe, synth

    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    H, I, E, k, T = 64, 48, 8, 2, 50 if world < 8 else 5  # world 8, T 5: the last ranks own no token
    ora = oracle_lib.oracle()
    w = synth.MoELayerWeights(H, I, E, 23, sigma=0.05)
    t = synth.activations(23, T, H)
    scores = ora.router_scores(t, w.router_w, w.router_b)
    tw, ti, _, _ = ora.topk_softmax(scores, k)
    e0, e1 = expert_range(rank, world, E)
    _, _, yp = ora.moe_block(t, tw, ti, w, mode=oracle_lib.MODE_GPU_BF16, e_begin=e0, e_end=e1, taps=True)
    mine = ((ti >= e0) & (ti < e1)).reshape(-1)  # pairs whose expert lives on this rank: the rows this rank writes
    yp = np.where(mine[:, None], yp, 0.0).astype(np.float32)
    # push to owners: rank r receives, from every rank, the rows of the tokens of r's slice
    bounds = [moe.slice_bounds(r, world, T) for r in range(world)]
    assert sum(n for _, n in bounds) == T and all(bounds[r][0] + bounds[r][1] == bounds[r + 1][0] or bounds[r + 1][1] == 0
                                                  for r in range(world - 1))
    per = max(n for _, n in bounds)  # slice size: ceil(T / world) rounded up to the routing block of 8 tokens
    send = [torch.zeros(per * k, H) for _ in range(world)]
    masks = [torch.zeros(per * k, dtype=torch.bool) for _ in range(world)]
    for r, (first, n) in enumerate(bounds):
        send[r][:n * k] = torch.from_numpy(yp[first * k:(first + n) * k])
        masks[r][:n * k] = torch.from_numpy(mine[first * k:(first + n) * k])
    # gloo has no all-to-all: every rank gathers what every rank sends and keeps the part addressed to it
    all_rows = [torch.zeros(world, per * k, H) for _ in range(world)]
    all_masks = [torch.zeros(world, per * k, dtype=torch.uint8) for _ in range(world)]
    dist.all_gather(all_rows, torch.stack(send))
    dist.all_gather(all_masks, torch.stack(masks).to(torch.uint8))
    recv = [all_rows[src][rank] for src in range(world)]
    recv_m = [all_masks[src][rank].bool() for src in range(world)]
    first, n = bounds[rank]
    rows = torch.zeros(per * k, H)
    writers = torch.zeros(per * k, dtype=torch.int32)
    for r in range(world):  # every row has exactly one writer
        rows[recv_m[r]] = recv[r][recv_m[r]]
        writers += recv_m[r].int()
    assert bool((writers[:n * k] == 1).all())
    # the oracle's taps hold the unweighted expert outputs: the owner applies the gate weights in slot order
    own = ora.combine_slots(rows[:n * k].numpy(), tw[first:first + n]) if n else np.zeros((0, H), np.float32)
    pad = torch.zeros(per, H)
    pad[:n] = torch.from_numpy(own)
    gathered = [torch.zeros(per, H) for _ in range(world)]
    dist.all_gather(gathered, pad)  # the delivery step of the replicated form
    got = torch.cat([g[:bounds[r][1]] for r, g in enumerate(gathered)]).numpy()
    _, _, yp_full = ora.moe_block(t, tw, ti, w, mode=oracle_lib.MODE_GPU_BF16, taps=True)
    want = ora.combine_slots(yp_full, tw)
    if rank == 0:
        np.save(out_path, np.array([float(np.array_equal(got, want)), float(np.abs(want).max() > 0)]))
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4, 8])
def test_owner_addressed_exchange_equals_the_single_rank_combine_bitwise(world, tmp_path):
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    out = tmp_path / "res.npy"
    mp.spawn(_owner_worker, args=(world, port, str(out)), nprocs=world, join=True)
    same, nonzero = np.load(out)
    assert same == 1.0 and nonzero == 1.0


def test_token_slices_are_contiguous_and_cover_the_batch():
    from gptoss_b200 import moe
    for world in (1, 2, 3, 4, 8, 16):
        for T in (0, 1, 5, 7, 16, 1000, 1024):
            b = [moe.slice_bounds(r, world, T) for r in range(world)]
            assert sum(n for _, n in b) == T
            nxt = 0
            for first, n in b:
                assert first == (nxt if n else T)
                nxt += n


def test_partition_covers_all_experts_once():
    for world in (1, 2, 4, 8):
        for E in (32, 128):
            r = [expert_range(i, world, E) for i in range(world)]
            assert r[0][0] == 0 and r[-1][1] == E
            assert all(r[i][1] == r[i + 1][0] for i in range(world - 1))
