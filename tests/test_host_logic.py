"""Host-side pieces that need no GPU: the seeded generator, bf16 helpers, routing oracle edge cases."""
import numpy as np

import oracle_lib
from gptoss_b200 import synth


def test_generator_is_reproducible_and_chunk_invariant():
    a = synth.normal_bf16_bits(7, synth.tensor_id(synth.TID_MLP1_W, 3), 10000, 0.02)
    b = np.concatenate([synth.normal_bf16_bits(7, synth.tensor_id(synth.TID_MLP1_W, 3), 5000, 0.02),
                        synth.normal_bf16_bits(7, synth.tensor_id(synth.TID_MLP1_W, 3), 5000, 0.02, start=5000)])
    assert np.array_equal(a, b)
    c = synth.normal_bf16_bits(7, synth.tensor_id(synth.TID_MLP1_W, 3), 10000, 0.02, chunk=777)
    assert np.array_equal(a, c)
    assert not np.array_equal(a, synth.normal_bf16_bits(8, synth.tensor_id(synth.TID_MLP1_W, 3), 10000, 0.02))


def test_generator_known_answers():
    # fixed vectors: any change to the generator invalidates every committed fixture
    bits = synth.normal_bf16_bits(20240607, 64 + 12, 6, 0.02)
    assert bits.tolist() == [0x3C8A, 0xBBF5, 0x3CBA, 0x3A83, 0xBC87, 0xBD22]
    assert synth.normal_bf16_bits(1, 1, 4, 1.0, start=1000).tolist() == [0x3F9D, 0x3F09, 0xBFA9, 0xBFDA]
    x = synth.normal(1, 4, (1 << 16,), 0.02)
    assert abs(float(x.std()) - 0.02) < 3e-4 and abs(float(x.mean())) < 3e-4
    assert np.array_equal(x, synth.round_bf16(x))  # bf16-representable


def test_bf16_rounding_is_nearest_even():
    x = np.array([1.0, 1.00390625, 1.01171875, -2.5, 3.0e38], np.float32)
    # 1 + 2^-8 is a tie between 1.0 and 1 + 2^-7 -> even mantissa (1.0); 1 + 3*2^-8 ties up to 1 + 2^-6
    r = synth.round_bf16(x)
    assert r[0] == 1.0 and r[1] == 1.0 and r[2] == np.float32(1.015625) and r[3] == -2.5


def test_zipf_bias_orders_experts():
    b = synth.zipf_router_bias(3, 0, 32, 1.2)
    assert b[0] > b[8] > b[31]
    assert np.array_equal(b, synth.round_bf16(b))


def test_topk_tie_rule_of_the_gpu_kernel(oracle):
    # selection sort with swap: after round 0 swaps position 0 with the winner, the displaced value sits
    # at the winner's old position, so among equal values the order is not simply "lowest id first"
    s = np.array([[1.0, 5.0, 5.0, 1.0, 5.0, 0.0, 1.0, 1.0]], np.float32)
    w, i, raw, ties = oracle.topk_softmax(s, 4, oracle_lib.RULE_SELECTION)
    assert i.tolist() == [[1, 2, 4, 3]]  # 0 was moved to slot 1, then to slot 2, then to slot 4
    assert ties == 1
    np.testing.assert_allclose(w.sum(), 1.0, rtol=1e-6)


def test_counting_sort_is_stable_and_skips_invalid_ids(oracle):
    ids = np.array([[3, 1, 0, 2], [1, 3, 7, -1], [0, 0, 2, 9]], np.int32)  # 7, -1, 9 are outside [0,4)
    off, srt, placed = oracle.counting_sort(ids, 4)
    assert off.tolist() == [0, 3, 5, 7, 9] and placed == 9
    assert srt[:9].tolist() == [2, 8, 9, 1, 4, 3, 10, 0, 5]
    assert (srt[9:] == -1).all()


def test_margin_flags_near_ties(oracle):
    s = np.array([[4.0, 3.0, 2.0, 1.0, 0.9999999, -1.0], [6.0, 5.0, 4.0, 3.0, 1.0, 0.0]], np.float32)
    m = oracle.topk_margin(s, 4)
    assert m[0] < 1e-6 and abs(m[1] - 1.0) < 1e-6


def test_c_generator_matches_numpy_generator(oracle):
    a = oracle.synth_normal(99, synth.tensor_id(synth.TID_MLP2_W, 2), (1000,), 0.02, start=12345)
    b = synth.bf16_bits_to_f32(synth.normal_bf16_bits(99, synth.tensor_id(synth.TID_MLP2_W, 2), 1000, 0.02, start=12345))
    assert np.array_equal(a, b)
    w = oracle.layer_weights(32, 64, 8, 5)
    ref = synth.MoELayerWeights(32, 64, 8, 5)
    for n in ("router_w", "router_b", "mlp1_w", "mlp1_b", "mlp2_w", "mlp2_b"):
        assert np.array_equal(getattr(w, n), getattr(ref, n)), n


def test_synthetic_tokenizer_file_encodes_text_to_its_bytes_with_the_reference_encoder(reference, tmp_path):
    from gptoss_b200 import binfmt
    p = tmp_path / "tokenizer.bin"
    binfmt.write_synthetic_tokenizer(str(p), 201088)
    for text in ["hello world", "The quick brown fox", "x 12345 y", "B200"]:
        assert reference.encode(p, 201088, text) == list(text.encode())
