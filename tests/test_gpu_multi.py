"""Fused cross-GPU combine on real peers: one process per GPU, CUDA IPC handles exchanged over gloo.
Needs at least two GPUs (skipped otherwise).  Every rank's residual stream must equal the single-GPU block
bit for bit, for several steps in a row."""
import os
import socket

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")


def _worker(rank, world, port, out_dir):
    import sys
    from pathlib import Path
    root = Path(__file__).resolve().parent.parent
    sys.path[:0] = [str(root), str(root / "tests")]
    import __graft_entry__ as entry
    entry.load_package()
    import torch.distributed as dist
    from gptoss_b200 import moe, synth

    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    os.environ["GPTOSS_SHARED_ROUTING"] = "1"  # also with two ranks: every rank routes its own token slice only
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.cuda.set_device(rank)
    H, I, E, k, T = 512, 384, 16, 4, 1000
    blk = moe.MoEBlock(hidden=H, intermediate=I, n_experts=E, top_k=k, max_tokens=T, device=rank, rank=rank,
                       world=world)
    blk.fill_layer_synthetic(0, 9, 0.05)
    blk.attach_peers()
    single = None
    if rank == 0:
        single = moe.MoEBlock(hidden=H, intermediate=I, n_experts=E, top_k=k, max_tokens=T, device=0)
        single.fill_layer_synthetic(0, 9, 0.05)
    dist.barrier()  # nobody starts waiting on a peer's flags while rank 0 is still setting up
    ok = True
    for step in range(4):
        t = synth.activations(300 + step, T, H)
        t_dev = torch.from_numpy(synth.f32_to_bf16_bits(t).view(np.int16).reshape(T, H)).cuda().view(torch.bfloat16)
        x = torch.ones((T, H), dtype=torch.float32, device="cuda")
        blk.forward(0, t_dev, x)
        blk.status()
        got = x.cpu()
        if rank == 0:
            want = torch.ones((T, H), dtype=torch.float32, device="cuda")
            single.forward(0, t_dev, want)
            want = want.cpu()
        else:
            want = torch.empty_like(got)
        dist.broadcast(want, src=0)
        ok = ok and bool(torch.equal(got, want))
    # the token-sliced form through host buffers: every rank moves only its rows over PCIe
    first, n = blk.slice(T)
    for step in range(3):
        t = synth.activations(400 + step, T, H)
        x0 = synth.normal(500 + step, synth.tensor_id(synth.TID_RESIDUAL), (T, H), 1.0)
        t_bits = torch.from_numpy(synth.f32_to_bf16_bits(t).view(np.int16).reshape(T, H))
        t_slice = t_bits[first:first + n].contiguous().pin_memory()
        x_slice = torch.from_numpy(x0[first:first + n].copy()).pin_memory()
        blk.forward_host_sliced(0, T, t_slice, x_slice)
        if rank == 0:
            want = torch.from_numpy(x0.copy()).cuda()
            single.forward(0, t_bits.cuda().view(torch.bfloat16), want)
            want = want.cpu()
        else:
            want = torch.empty((T, H), dtype=torch.float32)
        dist.broadcast(want, src=0)
        ok = ok and bool(torch.equal(x_slice, want[first:first + n]))
    # the dispatch form on device buffers: rows only to the ranks whose experts they selected
    for step in range(3):
        t = synth.activations(600 + step, T, H)
        x0 = synth.normal(700 + step, synth.tensor_id(synth.TID_RESIDUAL), (T, H), 1.0)
        t_dev = torch.from_numpy(synth.f32_to_bf16_bits(t).view(np.int16).reshape(T, H)).cuda().view(torch.bfloat16)
        t_slice = t_dev[first:first + n].contiguous()
        x_slice = torch.from_numpy(x0[first:first + n].copy()).cuda()
        blk.forward_dispatch(0, T, t_slice, x_slice)
        blk.status()
        if rank == 0:
            want = torch.from_numpy(x0.copy()).cuda()
            single.forward(0, t_dev, want)
            want = want.cpu()
        else:
            want = torch.empty((T, H), dtype=torch.float32)
        dist.broadcast(want, src=0)
        ok = ok and bool(torch.equal(x_slice.cpu(), want[first:first + n]))
    dist.barrier()
    blk.close()
    if single:
        single.close()
    (Path(out_dir) / f"rank{rank}.txt").write_text("ok" if ok else "mismatch")
    dist.destroy_process_group()


def _model_worker(rank, world, port, out_dir):
    import sys
    from pathlib import Path
    root = Path(__file__).resolve().parent.parent
    sys.path[:0] = [str(root), str(root / "tests")]
    import __graft_entry__ as entry
    entry.load_package()
    import torch.distributed as dist
    from gptoss_b200 import binfmt, model, synth

    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.cuda.set_device(rank)
    cfg = binfmt.config_7m()
    batch, n_pos = 11, 24
    ids = synth.uniform_ids(5, 6, batch * n_pos, cfg.vocab_size).reshape(n_pos, batch).astype(np.int32)
    m = model.Model(cfg, device=rank, max_batch=batch, max_seq=32, rank=rank, world=world)
    m.fill_synthetic(77)
    handles = [None] * world
    dist.all_gather_object(handles, m.comm_export())
    m.comm_attach(handles)
    first, n = m.slice(batch)
    single = None
    if rank == 0:
        single = model.Model(cfg, device=0, max_batch=batch, max_seq=32)
        single.fill_synthetic(77)
    dist.barrier()
    ok = True
    for pos in range(n_pos):
        got = m.step(ids[pos, first:first + n], pos, batch=batch)
        want = torch.from_numpy(single.step(ids[pos], pos)) if rank == 0 else torch.empty(batch, dtype=torch.int32)
        dist.broadcast(want, src=0)
        ok = ok and bool(np.array_equal(got, want.numpy()[first:first + n]))
    dist.barrier()
    m.close()
    if single:
        single.close()
    (Path(out_dir) / f"rank{rank}.txt").write_text("ok" if ok else "mismatch")
    dist.destroy_process_group()


def test_group_decode_across_processes_matches_single_gpu(tmp_path):
    """Whole-model decode by a group of real GPUs (one process each, sequences in slices, experts sharded): every
    rank's greedy tokens equal the single-GPU model's for its sequences, 24 positions in a row."""
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs at least two GPUs")
    world = 2 if n < 4 else 4
    import torch.multiprocessing as mp
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_model_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        assert (tmp_path / f"rank{r}.txt").read_text() == "ok"


def test_fused_combine_across_processes_matches_single_gpu(tmp_path):
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs at least two GPUs")
    world = 2 if n < 4 else 4
    import torch.multiprocessing as mp
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        assert (tmp_path / f"rank{r}.txt").read_text() == "ok"
