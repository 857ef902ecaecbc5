"""GPU parity of the routing kernels against the oracle: bit-exact expert assignment, offsets and
counting-sort permutation (called through the C ABI)."""
import numpy as np
import pytest

import oracle_lib
from gptoss_b200 import synth

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")


def _block(**kw):
    from gptoss_b200 import moe
    return moe.MoEBlock(**kw)


@pytest.mark.parametrize("E,k,T", [(32, 4, 1024), (128, 4, 333), (8, 2, 5), (40, 8, 64), (256, 4, 17), (32, 4, 1)])
def test_topk_softmax_bit_exact_on_given_scores(oracle, E, k, T):
    rng = np.random.default_rng(E * 1000 + T)
    scores = rng.standard_normal((T, E)).astype(np.float32)
    blk = _block(hidden=64, intermediate=64, n_experts=E, top_k=k, max_tokens=max(T, 8))
    w, i = blk.topk_softmax(torch.from_numpy(scores).cuda())
    ow, oi, _, ties = oracle.topk_softmax(scores, k, oracle_lib.RULE_SELECTION)
    assert ties == 0
    assert np.array_equal(i.cpu().numpy(), oi)
    np.testing.assert_allclose(w.cpu().numpy(), ow, rtol=2e-6, atol=0)
    blk.close()


def test_topk_tie_rule_matches_selection_sort_with_swap(oracle):
    # heavy ties: scores quantised to a handful of values, -inf and +inf included
    rng = np.random.default_rng(5)
    E, k, T = 64, 4, 512
    scores = rng.integers(0, 4, size=(T, E)).astype(np.float32)
    scores[::7, 3] = -np.inf
    scores[::11, 5] = np.inf
    scores[1] = 2.0  # a row of all-equal values
    blk = _block(hidden=64, intermediate=64, n_experts=E, top_k=k, max_tokens=T)
    w, i = blk.topk_softmax(torch.from_numpy(scores).cuda())
    ow, oi, _, ties = oracle.topk_softmax(scores, k, oracle_lib.RULE_SELECTION)
    assert ties > 0
    assert np.array_equal(i.cpu().numpy(), oi)
    finite = np.isfinite(ow).all(axis=1)
    np.testing.assert_allclose(w.cpu().numpy()[finite], ow[finite], rtol=2e-6, atol=0)
    blk.close()


@pytest.mark.parametrize("E,k,T", [(32, 4, 1024), (128, 4, 2048), (32, 4, 8192), (8, 2, 3), (32, 4, 1), (40, 8, 77)])
def test_build_offsets_bit_exact(oracle, E, k, T):
    rng = np.random.default_rng(T + E)
    p = 1.0 / np.arange(1, E + 1) ** 1.2  # skewed, like the Zipf-biased router
    ids = rng.choice(E, size=(T, k), p=p / p.sum()).astype(np.int32)
    blk = _block(hidden=64, intermediate=64, n_experts=E, top_k=k, max_tokens=max(T, 8))
    off, srt = blk.moe_build_offsets(torch.from_numpy(ids).cuda())
    ooff, osrt, placed = oracle.counting_sort(ids, E)
    assert placed == T * k
    assert np.array_equal(off.cpu().numpy(), ooff)
    assert np.array_equal(srt.cpu().numpy(), osrt)
    blk.close()


def test_build_offsets_skips_ids_outside_range_and_handles_empty_experts(oracle):
    E, k, T = 16, 4, 100
    rng = np.random.default_rng(3)
    ids = rng.integers(-2, E + 3, size=(T, k)).astype(np.int32)
    ids[ids == 5] = 6  # expert 5 receives nothing
    blk = _block(hidden=64, intermediate=64, n_experts=E, top_k=k, max_tokens=T)
    off, srt = blk.moe_build_offsets(torch.from_numpy(ids).cuda())
    ooff, osrt, placed = oracle.counting_sort(ids, E)
    assert placed < T * k and ooff[5] == ooff[6]
    assert np.array_equal(off.cpu().numpy(), ooff)
    assert np.array_equal(srt.cpu().numpy()[:placed], osrt[:placed])
    assert (srt.cpu().numpy()[placed:] == -1).all()  # untouched tail
    blk.close()


def test_empty_batch_is_a_no_op():
    blk = _block(hidden=64, intermediate=64, n_experts=8, top_k=2, max_tokens=8)
    ids = torch.empty((0, 2), dtype=torch.int32, device="cuda")
    off, srt = blk.moe_build_offsets(ids)
    assert off.cpu().numpy().tolist() == [0] * 9 and srt.numel() == 0
    w, i = blk.topk_softmax(torch.empty((0, 8), dtype=torch.float32, device="cuda"))
    assert w.numel() == 0
    blk.close()


@pytest.mark.parametrize("H,E,T,zipf", [(2880, 32, 1024, None), (2880, 32, 2048, 1.2), (256, 128, 300, None)])
def test_route_stage_matches_oracle(oracle, H, E, T, zipf):
    """router GEMM -> top-k -> offsets -> permutation -> gather, end to end.  Scores agree to fp32
    accumulation noise; the assignment must be identical for every token whose top-(k+1) margin
    exceeds that noise, and the permutation must be the oracle's permutation of the GPU's own ids."""
    k, I, seed = 4, 64, 11
    w = synth.MoELayerWeights(H, I, E, seed, zipf_s=zipf)
    t = synth.activations(seed, T, H)
    blk = _block(hidden=H, intermediate=I, n_experts=E, top_k=k, max_tokens=T)
    blk.upload_layer(0, w)
    t_dev = torch.from_numpy(synth.f32_to_bf16_bits(t).view(np.int16).reshape(T, H)).cuda().view(torch.bfloat16)
    blk.route(0, t_dev)
    blk.status()
    scores = blk.tap("scores", T)
    oscores = oracle.router_scores(t, w.router_w, w.router_b)
    np.testing.assert_allclose(scores, oscores, rtol=0, atol=2e-4)
    _, oi, _, _ = oracle.topk_softmax(oscores, k, oracle_lib.RULE_SELECTION)
    margin = oracle.topk_margin(oscores, k)
    ti = blk.tap("topk_i", T)
    safe = margin > 5e-4
    assert safe.mean() > 0.9
    assert np.array_equal(ti[safe], oi[safe])
    # given the GPU's scores, everything downstream is bit-exact
    gw, gi, _, _ = oracle.topk_softmax(scores, k, oracle_lib.RULE_SELECTION)
    assert np.array_equal(ti, gi)
    np.testing.assert_allclose(blk.tap("topk_w", T), gw, rtol=2e-6, atol=0)
    ooff, osrt, _ = oracle.counting_sort(ti, E)
    assert np.array_equal(blk.tap("offsets", T), ooff)
    srt = blk.tap("sorted", T)
    assert np.array_equal(srt, osrt)
    xp = blk.tap("x_packed", T)
    tb = synth.f32_to_bf16_bits(t).reshape(T, H)
    assert np.array_equal(xp, tb[srt // k])
    blk.close()


def test_argmax_first_maximum_and_degenerate_rows():
    """sample_argmax (run.cpp:739-750): first maximum; rows without a comparable maximum give index 0."""
    import ctypes as C
    from gptoss_b200 import capi
    lib = capi.load()
    V = 201088
    rng = np.random.default_rng(7)
    rows = rng.standard_normal((6, V)).astype(np.float32)
    rows[1, [5, 70000, 200000]] = 9.0          # three equal maxima: the first wins
    rows[2, :] = -np.inf                       # nothing comparable
    rows[3, :] = np.nan
    rows[4, 0] = np.nan                        # NaN in front: the reference's running maximum never moves
    rows[5, V - 1] = 50.0                      # maximum in the last (scalar-tail) position
    want = np.array([int(rows[0].argmax()), 5, 0, 0, 0, V - 1], np.int32)
    dev = torch.from_numpy(rows).cuda()
    out = torch.full((6,), -1, dtype=torch.int32, device="cuda")
    rc = lib.gptoss_argmax_rows(C.c_void_p(dev.data_ptr()), 6, V, C.c_void_p(out.data_ptr()), None)
    assert rc == capi.OK
    torch.cuda.synchronize()
    assert np.array_equal(out.cpu().numpy(), want)
