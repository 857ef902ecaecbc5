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


def _dispatch_worker(rank, world, port, out_path):
    """The dispatch form of the GPU path on CPU ranks: every rank holds only ITS slice of the tokens.  It routes its
    own rows, the routing rows are shared (all ranks then hold the same expert assignment and run the same counting
    sort), each token row travels only to the ranks whose experts it selected, every rank runs its experts on the rows
    it received, the gate-weighted expert rows go back to the token's owner, and the owner sums its tokens' k slots in
    slot order.  gloo all-gathers stand in for the peer stores; a rank reads from a gathered buffer only what the GPU
    path would have stored into its memory."""
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
    H, I, E, k, T = 64, 48, 8, 2, 50 if world < 8 else 21  # world 8, T 21: the last ranks own no token
    ora = oracle_lib.oracle()
    w = synth.MoELayerWeights(H, I, E, 29, sigma=0.05)
    t_all = synth.activations(29, T, H)  # the whole batch exists only to cut this rank's slice from it and for the check
    bounds = [moe.slice_bounds(r, world, T) for r in range(world)]
    per = max(n for _, n in bounds)
    first, n = bounds[rank]
    t_own = t_all[first:first + n]
    # 1. route the own rows, share the routing rows
    tw_own = np.zeros((per, k), np.float32)
    ti_own = np.full((per, k), -1, np.int32)
    if n:
        tw_own[:n], ti_own[:n], _, _ = ora.topk_softmax(ora.router_scores(t_own, w.router_w, w.router_b), k)
    tws = [torch.zeros(per, k) for _ in range(world)]
    tis = [torch.zeros(per, k, dtype=torch.int32) for _ in range(world)]
    dist.all_gather(tws, torch.from_numpy(tw_own))
    dist.all_gather(tis, torch.from_numpy(ti_own))
    tw = np.concatenate([tws[r][:bounds[r][1]].numpy() for r in range(world)])
    ti = np.concatenate([tis[r][:bounds[r][1]].numpy() for r in range(world)])
    # 2. dispatch: a token row goes to rank r only if one of its slots selects an expert of r
    e0, e1 = expert_range(rank, world, E)
    rows = [torch.zeros(per, H) for _ in range(world)]
    pad = torch.zeros(per, H)
    pad[:n] = torch.from_numpy(t_own)
    dist.all_gather(rows, pad)
    t_recv = np.zeros((T, H), np.float32)
    wanted = ((ti >= e0) & (ti < e1)).any(axis=1)  # tokens with a slot on this rank
    for r, (f, m) in enumerate(bounds):
        sel = wanted[f:f + m]
        t_recv[f:f + m][sel] = rows[r][:m].numpy()[sel]  # nothing else of the gathered rows is read
    # 3. this rank's experts on the rows it received (rows of other tokens stay zero and must not matter)
    _, _, yp = ora.moe_block(t_recv, tw, ti, w, mode=oracle_lib.MODE_GPU_BF16, e_begin=e0, e_end=e1, taps=True)
    mine = ((ti >= e0) & (ti < e1)).reshape(-1)
    yp = np.where(mine[:, None], yp, 0.0).astype(np.float32)
    # 4. push the expert rows to the tokens' owners, 5. owner sum in slot order
    send = torch.zeros(world, per * k, H)
    for r, (f, m) in enumerate(bounds):
        send[r, :m * k] = torch.from_numpy(yp[f * k:(f + m) * k])
    gathered = [torch.zeros(world, per * k, H) for _ in range(world)]
    dist.all_gather(gathered, send)
    own_rows = torch.zeros(per * k, H)
    for src in range(world):  # exactly one rank wrote a non-zero row per pair: adding zeros keeps the bits
        s0, s1 = expert_range(src, world, E)
        m_src = torch.from_numpy(((ti[first:first + n] >= s0) & (ti[first:first + n] < s1)).reshape(-1))
        own_rows[:n * k][m_src] = gathered[src][rank][:n * k][m_src]
    got_own = ora.combine_slots(own_rows[:n * k].numpy(), tw[first:first + n]) if n else np.zeros((0, H), np.float32)
    # check against the single-rank block on the whole batch
    tw_f, ti_f, _, _ = ora.topk_softmax(ora.router_scores(t_all, w.router_w, w.router_b), k)
    _, _, yp_full = ora.moe_block(t_all, tw_f, ti_f, w, mode=oracle_lib.MODE_GPU_BF16, taps=True)
    want = ora.combine_slots(yp_full, tw_f)
    ok = torch.tensor([float(np.array_equal(ti, ti_f) and np.array_equal(tw, tw_f) and
                             np.array_equal(got_own, want[first:first + n]))])
    dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    if rank == 0:
        np.save(out_path, np.array([float(ok.item()), float(np.abs(want).max() > 0)]))
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4, 8])
def test_dispatch_form_on_token_slices_equals_the_single_rank_block_bitwise(world, tmp_path):
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    out = tmp_path / "res.npy"
    mp.spawn(_dispatch_worker, args=(world, port, str(out)), nprocs=world, join=True)
    same, nonzero = np.load(out)
    assert same == 1.0 and nonzero == 1.0
