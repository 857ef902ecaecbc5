"""Pins the C oracle (oracle/moe_oracle.c) to outputs of the reference's own forward()
(tests/golden/moe_7m_golden.npz, produced by tests/golden/make_golden.py)."""
from pathlib import Path
from types import SimpleNamespace

import numpy as np
import pytest

import oracle_lib
from gptoss_b200 import binfmt, synth

GOLDEN = Path(__file__).parent / "golden" / "moe_7m_golden.npz"


@pytest.fixture(scope="module")
def golden():
    return np.load(GOLDEN)


@pytest.fixture(scope="module")
def weights(golden):
    """MoE tensors of the captured layer, regenerated from the seed (checkpoint streams 64+pos)."""
    cfg = binfmt.config_7m()
    seed, layer = int(golden["seed"]), int(golden["layer"])
    shapes = dict(binfmt.tensor_shapes(cfg))
    pos = {n: i for i, n in enumerate(binfmt.TENSOR_ORDER)}
    w = SimpleNamespace()
    for name in ("router_w", "router_b", "mlp1_w", "mlp1_b", "mlp2_w", "mlp2_b"):
        per_layer = int(np.prod(shapes[name][1:]))
        bits = synth.normal_bf16_bits(seed, 64 + pos[name], per_layer, 0.02, start=layer * per_layer)
        setattr(w, name, synth.bf16_bits_to_f32(bits).reshape(shapes[name][1:]))
    return w


def test_router_scores_bit_exact(oracle, golden, weights):
    s = oracle.router_scores(np.ascontiguousarray(golden["t"]), weights.router_w, weights.router_b)
    assert np.array_equal(s, golden["router_score"])


def test_topk_and_gate_weights_bit_exact(oracle, golden):
    sc = np.ascontiguousarray(golden["router_score"])
    w, i, _, ties = oracle.topk_softmax(sc, 4, oracle_lib.RULE_QSORT)
    assert ties == 0
    assert np.array_equal(i, golden["topk_i"])
    assert np.array_equal(w, golden["topk_v"])
    # the GPU rule (selection sort) agrees on the assignment when there are no ties; its softmax
    # formula differs from the CPU one by at most an ulp or two
    w2, i2, _, _ = oracle.topk_softmax(sc, 4, oracle_lib.RULE_SELECTION)
    assert np.array_equal(i2, golden["topk_i"])
    np.testing.assert_allclose(w2, golden["topk_v"], rtol=3e-7, atol=0)


def test_moe_block_bit_exact(oracle, golden, weights):
    t = np.ascontiguousarray(golden["t"])
    out = oracle.moe_block(t, np.ascontiguousarray(golden["topk_v"]),
                           np.ascontiguousarray(golden["topk_i"]), weights, limit=7.0,
                           mode=oracle_lib.MODE_CPU)
    assert np.array_equal(out, golden["e_agg"])


def test_expert_parallel_partials_sum_to_block(oracle, golden, weights):
    t = np.ascontiguousarray(golden["t"][:16])
    tv = np.ascontiguousarray(golden["topk_v"][:16])
    ti = np.ascontiguousarray(golden["topk_i"][:16])
    full = oracle.moe_block(t, tv, ti, weights, mode=oracle_lib.MODE_CPU)
    parts = sum(oracle.moe_block(t, tv, ti, weights, mode=oracle_lib.MODE_CPU, e_begin=e, e_end=e + 8)
                for e in range(0, 32, 8))
    np.testing.assert_allclose(parts, full, rtol=1e-5, atol=1e-9)


def test_slot_order_combine_close_to_expert_order(oracle, golden, weights):
    t = np.ascontiguousarray(golden["t"][:32])
    tv = np.ascontiguousarray(golden["topk_v"][:32])
    ti = np.ascontiguousarray(golden["topk_i"][:32])
    out, _, yp = oracle.moe_block(t, tv, ti, weights, mode=oracle_lib.MODE_CPU, taps=True)
    slot = oracle.combine_slots(yp, tv)
    np.testing.assert_allclose(slot, out, rtol=1e-5, atol=1e-9)


def test_reference_moe_rows_matches_forward_state(reference, golden, weights):
    t = np.ascontiguousarray(golden["t"])
    agg, tv, ti = reference.moe_rows(t, weights, 4)
    assert np.array_equal(ti, golden["topk_i"])
    assert np.array_equal(tv, golden["topk_v"])
    assert np.array_equal(agg, golden["e_agg"])


def test_checkpoint_roundtrip_and_hash(golden, tmp_path):
    import hashlib
    cfg = binfmt.config_7m()
    p = tmp_path / "m.bin"
    binfmt.write_synthetic(str(p), cfg, int(golden["seed"]))
    assert hashlib.sha256(p.read_bytes()).digest() == golden["checkpoint_sha256"].tobytes()
    c2, tensors = binfmt.read(str(p))
    assert c2 == cfg
    assert tensors["mlp1_w"].shape == (2, 32, 128, 32)
    assert np.all(tensors["mlp_norm"] == 1.0)
    assert p.stat().st_size == 53151948  # 60-byte header + fp32 tensors of the 7m dims
