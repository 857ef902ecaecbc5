"""The fused cross-GPU combine (peer stores from the down-GEMM epilogue, owner-side slot-ordered sum,
delivery to every rank) exercised on ONE GPU: the ranks are contexts of one process attached to one another,
and their stages are issued in an order in which no kernel ever has to wait for a later one (all pushes, then
all owner combines, then all adds).  The result must equal the single-context block bit for bit.  A second
test lets a wait on a peer run out (a rank that never pushes) and checks that it ends as a status code."""
import numpy as np
import pytest

from gptoss_b200 import synth

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")


def to_dev_bf16(x):
    T, H = x.shape
    return torch.from_numpy(synth.f32_to_bf16_bits(x).view(np.int16).reshape(T, H)).cuda().view(torch.bfloat16)


@pytest.mark.parametrize("world,T", [(2, 300), (4, 203), (8, 64)])
def test_emulated_ranks_match_single_context_bitwise(world, T):
    from gptoss_b200 import moe
    H, I, E, k = 256, 192, 16, 4
    w = synth.MoELayerWeights(H, I, E, 61, sigma=0.05)
    single = moe.MoEBlock(hidden=H, intermediate=I, n_experts=E, top_k=k, max_tokens=T)
    single.upload_layer(0, w)
    ranks = [moe.MoEBlock(hidden=H, intermediate=I, n_experts=E, top_k=k, max_tokens=T, rank=r, world=world)
             for r in range(world)]
    for b in ranks:
        b.upload_layer(0, w)
    moe.MoEBlock.attach_local(ranks)
    for step in range(3):  # flags carry the step number: several steps without any reset
        t = synth.activations(100 + step, T, H)
        x0 = synth.normal(200 + step, synth.tensor_id(synth.TID_RESIDUAL), (T, H), 1.0)
        t_dev = to_dev_bf16(t)
        want = torch.from_numpy(x0.copy()).cuda()
        single.forward(0, t_dev, want)
        xs = [torch.from_numpy(x0.copy()).cuda() for _ in range(world)]
        for b in ranks:
            b.route(0, t_dev)
            b.mlp1_swiglu(0)
            b.push_to_owners(0)
        for b in ranks:
            b.owner_combine()
        for b, x in zip(ranks, xs):
            b.add_delta(x)
        for b in ranks:
            b.status()
        for x in xs:
            assert torch.equal(x, want)
    for b in ranks + [single]:
        b.close()


@pytest.mark.parametrize("world,T", [(2, 300), (4, 203), (8, 64)])
def test_shared_routing_matches_single_context_bitwise(world, T, monkeypatch):
    """Replicated activations, routing shared: every rank routes only its token slice (router GEMM with the split-K
    factor of the whole batch, top-k, block histograms) and stores the rows to all ranks; after that every rank must
    hold the routing of the single-context block bit for bit, and the block output must be identical."""
    from gptoss_b200 import moe
    monkeypatch.setenv("GPTOSS_SHARED_ROUTING", "1")  # read when a context is created
    H, I, E, k = 256, 192, 16, 4
    w = synth.MoELayerWeights(H, I, E, 81, sigma=0.05)
    single = moe.MoEBlock(hidden=H, intermediate=I, n_experts=E, top_k=k, max_tokens=T)
    single.upload_layer(0, w)
    ranks = [moe.MoEBlock(hidden=H, intermediate=I, n_experts=E, top_k=k, max_tokens=T, rank=r, world=world)
             for r in range(world)]
    for b in ranks:
        b.upload_layer(0, w)
    moe.MoEBlock.attach_local(ranks)
    for step in range(2):
        t = synth.activations(600 + step, T, H)
        x0 = synth.normal(700 + step, synth.tensor_id(synth.TID_RESIDUAL), (T, H), 1.0)
        t_dev = to_dev_bf16(t)
        want = torch.from_numpy(x0.copy()).cuda()
        single.forward(0, t_dev, want)
        xs = [torch.from_numpy(x0.copy()).cuda() for _ in range(world)]
        for b in ranks:
            b.route_local(0, t_dev)
        for b in ranks:
            b.route_finish(0, t_dev)
            b.mlp1_swiglu(0)
            b.push_to_owners(0)
        for b in ranks:
            b.owner_combine()
        for b, x in zip(ranks, xs):
            b.add_delta(x)
        for b in ranks:
            b.status()
            for name in ("topk_i", "topk_w", "offsets", "sorted"):
                assert np.array_equal(b.tap(name, T), single.tap(name, T)), name
        for x in xs:
            assert torch.equal(x, want)
    for b in ranks + [single]:
        b.close()


def test_wait_on_a_silent_peer_times_out_as_status():
    from gptoss_b200 import capi, moe
    H, I, E, k, T = 128, 128, 8, 2, 32
    ranks = [moe.MoEBlock(hidden=H, intermediate=I, n_experts=E, top_k=k, max_tokens=T, rank=r, world=2)
             for r in range(2)]
    for b in ranks:
        b.fill_layer_synthetic(0, 5, 0.05)
    moe.MoEBlock.attach_local(ranks)
    ranks[0].set_peer_timeout_ms(150)
    t_dev = to_dev_bf16(synth.activations(5, T, H))
    x = torch.zeros((T, H), dtype=torch.float32, device="cuda")
    ranks[0].forward(0, t_dev, x)          # rank 1 never pushes: the owner's wait must give up
    with pytest.raises(moe.GptossError) as e:
        ranks[0].status()
    assert e.value.code == capi.ERR_TIMEOUT
    assert "site 0x2100" in str(e.value)   # the owner's wait for the "pushed" flags, not a wait inside a GEMM
    ranks[0].status()                      # the error word is cleared, the context stays usable
    part = torch.empty_like(x)
    ranks[0].forward_partial(0, t_dev, part)
    ranks[0].status()
    assert torch.isfinite(part).all()
    with pytest.raises(moe.GptossError) as e:   # but the group is out of step: exchanges are refused from now on
        ranks[0].forward(0, t_dev, x)
    assert e.value.code == capi.ERR_STATE
    for b in ranks:
        b.close()


def test_bf16_delivery_keeps_ranks_identical_and_close_to_fp32():
    from gptoss_b200 import capi, moe
    H, I, E, k, T, world = 256, 192, 16, 4, 300, 4
    w = synth.MoELayerWeights(H, I, E, 71, sigma=0.05)
    single = moe.MoEBlock(hidden=H, intermediate=I, n_experts=E, top_k=k, max_tokens=T)
    single.upload_layer(0, w)
    ranks = [moe.MoEBlock(hidden=H, intermediate=I, n_experts=E, top_k=k, max_tokens=T, rank=r, world=world,
                          wire=capi.WIRE_BF16) for r in range(world)]
    for b in ranks:
        b.upload_layer(0, w)
    moe.MoEBlock.attach_local(ranks)
    t_dev = to_dev_bf16(synth.activations(72, T, H))
    want = torch.zeros((T, H), dtype=torch.float32, device="cuda")
    single.forward(0, t_dev, want)
    xs = [torch.zeros((T, H), dtype=torch.float32, device="cuda") for _ in range(world)]
    for b in ranks:
        b.route(0, t_dev)
        b.mlp1_swiglu(0)
        b.push_to_owners(0)
    for b in ranks:
        b.owner_combine()
    for b, x in zip(ranks, xs):
        b.add_delta(x)
        b.status()
    for x in xs[1:]:
        assert torch.equal(x, xs[0])                      # replicated residual streams stay identical
    # exactly the fp32 result rounded to bf16 (x started at zero)
    assert torch.equal(xs[0], want.to(torch.bfloat16).to(torch.float32))
    for b in ranks + [single]:
        b.close()


@pytest.mark.parametrize("world,T", [(2, 300), (4, 203), (8, 5)])
def test_token_sliced_form_matches_single_context_bitwise(world, T):
    """Every rank holds only its rows of the residual stream: the rows are gathered to all ranks (with and without
    the fused residual + RMSNorm), every rank routes the gathered batch and pushes its experts' rows to the owners,
    the owners keep the slot-ordered sums.  Stage by stage over emulated ranks; uneven and empty slices."""
    from gptoss_b200 import moe
    H, I, E, k = 256, 192, 16, 4
    w = synth.MoELayerWeights(H, I, E, 71, sigma=0.05)
    single = moe.MoEBlock(hidden=H, intermediate=I, n_experts=E, top_k=k, max_tokens=T)
    single.upload_layer(0, w)
    ranks = [moe.MoEBlock(hidden=H, intermediate=I, n_experts=E, top_k=k, max_tokens=T, rank=r, world=world)
             for r in range(world)]
    for b in ranks:
        b.upload_layer(0, w)
    moe.MoEBlock.attach_local(ranks)
    bounds = [b.slice(T) for b in ranks]
    assert sum(n for _, n in bounds) == T
    for step in range(3):
        t = synth.activations(300 + step, T, H)
        x0 = synth.normal(400 + step, synth.tensor_id(synth.TID_RESIDUAL), (T, H), 1.0)
        t_dev = to_dev_bf16(t)
        want = torch.from_numpy(x0.copy()).cuda()
        single.forward(0, t_dev, want)
        xs = [torch.from_numpy(x0[f:f + n].copy()).cuda() for f, n in bounds]
        for b, (f, n) in zip(ranks, bounds):
            b.gather_rows(T, t_dev[f:f + n].contiguous() if n else None)
            b.sliced_route(0, T)
        for b in ranks:
            b.sliced_push(0, T)
        for b, x in zip(ranks, xs):
            b.sliced_combine(x)
        for b in ranks:
            b.status()
        got = torch.cat(xs)
        assert torch.equal(got, want)
    # fused residual + RMSNorm in front: compare with the same rows normalised by torch-free arithmetic on one context
    norm_w = torch.ones(H, dtype=torch.float32, device="cuda")
    x0 = synth.normal(500, synth.tensor_id(synth.TID_RESIDUAL), (T, H), 1.0)
    add = synth.normal(501, synth.tensor_id(synth.TID_RESIDUAL), (T, H), 0.5)
    xs = [torch.from_numpy(x0[f:f + n].copy()).cuda() for f, n in bounds]
    adds = [torch.from_numpy(add[f:f + n].copy()).cuda() for f, n in bounds]
    for b, x, a_ in zip(ranks, xs, adds):
        b.gather_slice(T, x, norm_w, add=a_)
        b.sliced_route(0, T)
    for b in ranks:
        b.sliced_push(0, T)
    for b, x in zip(ranks, xs):
        b.sliced_combine(x)
    for b in ranks:
        b.status()
    # reference: same arithmetic on the host (fp32 sum of squares is order-dependent: compare with a tolerance on t,
    # then bit for bit given the device's own gathered rows)
    xr = (x0 + add).astype(np.float32)
    gathered = ranks[0].tap("gathered", T)  # bf16 bits [T,H] as stored by all ranks
    t_ref = xr / np.sqrt((xr.astype(np.float64) ** 2).mean(axis=1, keepdims=True) + 1e-5).astype(np.float32)
    np.testing.assert_allclose(synth.bf16_bits_to_f32(gathered), t_ref, rtol=1e-2, atol=1e-3)
    for r in range(1, world):
        assert np.array_equal(ranks[r].tap("gathered", T), gathered)
    want = torch.from_numpy(xr.copy()).cuda()
    single.forward(0, torch.from_numpy(gathered.view(np.int16)).cuda().view(torch.bfloat16), want)
    assert torch.equal(torch.cat(xs), want)
    for b in ranks + [single]:
        b.close()


@pytest.mark.parametrize("world,T,E", [(2, 300, 16), (4, 203, 16), (8, 64, 16), (8, 5, 16), (8, 300, 128)])
def test_dispatch_form_matches_single_context_bitwise(world, T, E):
    """Dispatch form: every rank routes its own rows, shares the routing, and sends each row only to the ranks whose
    experts it selected (into its place in the receiver's grouped input); expert rows are pushed back to the token's
    owner.  fp32 wire: identical to one context bit for bit, routing and grouping included.  Stage by stage over
    emulated ranks; uneven and empty slices."""
    from gptoss_b200 import moe
    H, I, k = 256, 192, 4     # E = 128 on 8 ranks: 16 experts per rank, the 120b sharding
    w = synth.MoELayerWeights(H, I, E, 91, sigma=0.05)
    single = moe.MoEBlock(hidden=H, intermediate=I, n_experts=E, top_k=k, max_tokens=T)
    single.upload_layer(0, w)
    ranks = [moe.MoEBlock(hidden=H, intermediate=I, n_experts=E, top_k=k, max_tokens=T, rank=r, world=world)
             for r in range(world)]
    for b in ranks:
        b.upload_layer(0, w)
    moe.MoEBlock.attach_local(ranks)
    bounds = [b.slice(T) for b in ranks]
    for step in range(3):
        t = synth.activations(800 + step, T, H)
        x0 = synth.normal(900 + step, synth.tensor_id(synth.TID_RESIDUAL), (T, H), 1.0)
        t_dev = to_dev_bf16(t)
        want = torch.from_numpy(x0.copy()).cuda()
        single.forward(0, t_dev, want)
        ts = [t_dev[f:f + n].contiguous() if n else None for f, n in bounds]
        xs = [torch.from_numpy(x0[f:f + n].copy()).cuda() for f, n in bounds]
        for b, tsl in zip(ranks, ts):
            b.dispatch_route(0, T, tsl)
        for b, tsl in zip(ranks, ts):
            b.dispatch_rows(0, T, tsl)
        for b in ranks:
            b.dispatch_push(0)
        for b, x in zip(ranks, xs):
            b.sliced_combine(x)
        for b in ranks:
            b.status()
            for name in ("topk_i", "topk_w", "offsets"):
                assert np.array_equal(b.tap(name, T), single.tap(name, T)), name
        # every rank received exactly the rows of its experts, and their pair ids, in the grouped order
        off, xp, srt = single.tap("offsets", T), single.tap("x_packed", T), single.tap("sorted", T)
        n_local = E // world
        for r, b in enumerate(ranks):
            lo, hi = off[r * n_local], off[(r + 1) * n_local]
            assert np.array_equal(b.tap("x_packed", T)[lo:hi], xp[lo:hi])
            assert np.array_equal(b.tap("sorted", T)[lo:hi], srt[lo:hi])
        assert torch.equal(torch.cat(xs), want)
    for b in ranks + [single]:
        b.close()


def test_dispatch_form_bf16_wire_rounds_each_pushed_row_once():
    """bf16 wire: the gate-weighted expert rows travel as bf16 and the owner sums them in fp32 in slot order, i.e. the
    result is exactly x0 + ((r0 + r1) + r2) + r3 with r_j the bf16 rounding of the fp32 row of slot j."""
    from gptoss_b200 import capi, moe
    H, I, E, k, T, world = 256, 192, 16, 4, 300, 4
    w = synth.MoELayerWeights(H, I, E, 93, sigma=0.05)
    single = moe.MoEBlock(hidden=H, intermediate=I, n_experts=E, top_k=k, max_tokens=T)
    single.upload_layer(0, w)
    ranks = [moe.MoEBlock(hidden=H, intermediate=I, n_experts=E, top_k=k, max_tokens=T, rank=r, world=world,
                          wire=capi.WIRE_BF16) for r in range(world)]
    for b in ranks:
        b.upload_layer(0, w)
    moe.MoEBlock.attach_local(ranks)
    bounds = [b.slice(T) for b in ranks]
    t_dev = to_dev_bf16(synth.activations(94, T, H))
    x0 = synth.normal(95, synth.tensor_id(synth.TID_RESIDUAL), (T, H), 1.0)
    ref = torch.from_numpy(x0.copy()).cuda()
    single.forward(0, t_dev, ref)
    y = torch.from_numpy(single.tap("y_pairs", T)).reshape(T, k, H)
    r = y.to(torch.bfloat16).to(torch.float32)
    want = torch.from_numpy(x0.copy()) + (((r[:, 0] + r[:, 1]) + r[:, 2]) + r[:, 3])
    ts = [t_dev[f:f + n].contiguous() if n else None for f, n in bounds]
    xs = [torch.from_numpy(x0[f:f + n].copy()).cuda() for f, n in bounds]
    for b, tsl in zip(ranks, ts):
        b.dispatch_route(0, T, tsl)
    for b, tsl in zip(ranks, ts):
        b.dispatch_rows(0, T, tsl)
    for b in ranks:
        b.dispatch_push(0)
    for b, x in zip(ranks, xs):
        b.sliced_combine(x)
        b.status()
    got = torch.cat(xs).cpu()
    assert torch.equal(got, want)
    delta, delta_ref = got - torch.from_numpy(x0), ref.cpu() - torch.from_numpy(x0)
    assert float((delta - delta_ref).norm() / delta_ref.norm()) < 4e-3  # one bf16 rounding per row: 2^-9 relative
    for b in ranks + [single]:
        b.close()
