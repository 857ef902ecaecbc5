"""A group of GPUs decoding one batch together (sequences dealt out in slices, experts sharded by rank), with the
ranks emulated on one device: one model object per rank, attached to one another in-process, every phase of a step
run for every rank before the next phase (gptoss_model_step_begin / layer_attention / layer_moe_dispatch /
layer_moe_push / layer_moe_combine / step_end), so that each device-side wait finds its flags already raised.

The group must reproduce the single-GPU model bit for bit: attention and the dense GEMMs work per sequence, the
routing of a token has the same bits whichever rank computes it, every rank derives the same grouping, and the expert
outputs are summed in slot order by the token's owner."""
import ctypes as C

import numpy as np
import pytest

from gptoss_b200 import binfmt, capi, synth

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")

SEED = 31


@pytest.fixture(scope="module")
def checkpoint(tmp_path_factory):
    p = tmp_path_factory.mktemp("ckpt") / "gpt-oss-7m-synth.bin"
    binfmt.write_synthetic(str(p), binfmt.config_7m(), SEED)
    return p


@pytest.mark.parametrize("world,batch", [(2, 21), (4, 27), (8, 5)])
def test_group_matches_single_gpu_bitwise(checkpoint, world, batch):
    from gptoss_b200 import model
    cfg = binfmt.config_7m()
    n_pos = 40
    ids = synth.uniform_ids(SEED, 3, batch * n_pos, cfg.vocab_size).reshape(n_pos, batch).astype(np.int32)
    single = model.Model(cfg, max_batch=batch, max_seq=64)
    single.load_bin(checkpoint)
    group = [model.Model(cfg, max_batch=batch, max_seq=64, rank=r, world=world) for r in range(world)]
    for m in group:
        m.load_bin(checkpoint)
    model.Model.attach_local(group)
    slices = [m.slice(batch) for m in group]
    assert sum(n for _, n in slices) == batch and slices[0][0] == 0
    if world == 8:
        assert slices[-1][1] == 0  # fewer sequences than one slice (8): the other ranks hold none and still take part
    else:
        assert all(n > 0 for _, n in slices) and len({n for _, n in slices}) > 1  # uneven, non-empty slices
    for pos in range(n_pos):
        want = single.step(ids[pos], pos)
        got = model.Model.step_group(group, ids[pos], pos)
        assert np.array_equal(got, want), (pos, got, want)
        if pos % 13 == 0:
            for m, (first, n) in zip(group, slices):
                for i in range(n):
                    assert np.array_equal(m.logits(i), single.logits(first + i)), (pos, first + i)
    for m in group:
        m.close()
    single.close()


def test_group_step_without_peers_is_refused(checkpoint):
    from gptoss_b200 import model, moe
    cfg = binfmt.config_7m()
    m = model.Model(cfg, max_batch=4, max_seq=16, rank=0, world=2)
    m.load_bin(checkpoint)
    with pytest.raises(moe.GptossError) as e:
        m.step(np.zeros(2, np.int32), 0, batch=4)
    assert e.value.code == capi.ERR_STATE
    m.close()


def test_wait_for_a_rank_that_never_arrives_times_out(checkpoint):
    """Rank 1 never runs its attention phase: rank 0's wait for its routing rows runs out after the
    configured limit, the step reports a time-out and the context stays usable (no trap, no hang)."""
    from gptoss_b200 import model, moe
    cfg = binfmt.config_7m()
    group = [model.Model(cfg, max_batch=4, max_seq=16, rank=r, world=2) for r in range(2)]
    for m in group:
        m.load_bin(checkpoint)
        m.set_peer_timeout_ms(50)
    model.Model.attach_local(group)
    with pytest.raises(moe.GptossError) as e:
        group[0].step(np.zeros(2, np.int32), 0, batch=4)
    assert e.value.code == capi.ERR_TIMEOUT
    assert "site 0x23" in str(e.value) or "site 0x26" in str(e.value)  # a wait on a peer flag, not one inside a GEMM
    for m in group:
        m.close()
    # a fresh group on the same device works
    fresh = [model.Model(cfg, max_batch=4, max_seq=16, rank=r, world=2) for r in range(2)]
    for m in fresh:
        m.load_bin(checkpoint)
    model.Model.attach_local(fresh)
    out = model.Model.step_group(fresh, np.arange(4, dtype=np.int32), 0)
    assert out.shape == (4,)
    for m in fresh:
        m.close()
