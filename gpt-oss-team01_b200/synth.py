"""Seeded synthetic tensors, bit-identical on every platform and on the GPU.

Real GPT-OSS checkpoints are not available, so every weight and activation is drawn from a
counter-based generator keyed by ``(seed, tensor_id, element_index)``.  Only integer arithmetic and
ONE correctly rounded fp32 multiply are used, so the numpy implementation here and the CUDA
implementation in ``csrc/synth.cu`` produce the same bits, and every value is rounded to bf16 so
that an fp32 CPU model and a bf16 GPU model see identical numbers.

Element ``i`` of tensor ``tensor_id``:

    key = splitmix64(seed * 0x100000001B3 + tensor_id)
    a, b = splitmix64(key + 2 i), splitmix64(key + 2 i + 1)
    S   = sum of the eight 16-bit fields of a and b            (Irwin-Hall, n = 8)
    z   = fp32(S - 262140) * fp32(fp32(sigma) / 53509.9199...) (approximately N(0, sigma))
    val = bf16_round_nearest_even(z)

The tails stop at +-4.9 sigma; for the N(0, 0.02) weights and N(0, 1) activations used by the
benchmark configurations that is indistinguishable from a normal for the purposes of routing
statistics and GEMM numerics.
"""
from __future__ import annotations

import math

import numpy as np

_M64 = np.uint64(0xFFFFFFFFFFFFFFFF)
IH_MEAN = 4 * 65535  # mean of the sum of eight uniform 16-bit integers
IH_STD = math.sqrt(8 * (65536.0**2 - 1.0) / 12.0)

# tensor ids (shared with csrc/synth.cu callers; one id per logical tensor, layer folded in)
TID_ACTIVATION = 1
TID_ROUTER_W = 2
TID_ROUTER_B = 3
TID_MLP1_W = 4
TID_MLP1_B = 5
TID_MLP2_W = 6
TID_MLP2_B = 7
TID_RESIDUAL = 8
TID_GENERIC = 9


def tensor_id(kind: int, layer: int = 0) -> int:
    return kind + 16 * layer


def _splitmix64(z: np.ndarray) -> np.ndarray:
    with np.errstate(over="ignore"):
        z = z + np.uint64(0x9E3779B97F4A7C15)
        z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
        z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
        return z ^ (z >> np.uint64(31))


def stream_key(seed: int, tid: int) -> np.uint64:
    v = (int(seed) * 0x100000001B3 + int(tid)) & 0xFFFFFFFFFFFFFFFF
    return _splitmix64(np.array([v], dtype=np.uint64))[0]


def scale_f32(sigma: float) -> np.float32:
    """The fp32 constant both implementations multiply by (sigma is first rounded to fp32, because
    it crosses the C ABI as a float)."""
    return np.float32(float(np.float32(sigma)) / IH_STD)


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    r = (u + np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1))) >> np.uint32(16)
    return r.astype(np.uint16)


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << np.uint32(16)).view(np.float32)


def round_bf16(x: np.ndarray) -> np.ndarray:
    return bf16_bits_to_f32(f32_to_bf16_bits(x))


def _irwin_hall(key: np.uint64, start: int, n: int) -> np.ndarray:
    idx = np.arange(start, start + n, dtype=np.uint64)
    with np.errstate(over="ignore"):
        a = _splitmix64(key + np.uint64(2) * idx)
        b = _splitmix64(key + np.uint64(2) * idx + np.uint64(1))
    s = np.zeros(n, dtype=np.int64)
    for w in (a, b):
        for sh in (0, 16, 32, 48):
            s += ((w >> np.uint64(sh)) & np.uint64(0xFFFF)).astype(np.int64)
    return s


def normal_bf16_bits(seed: int, tid: int, n: int, sigma: float, start: int = 0,
                     chunk: int = 1 << 22) -> np.ndarray:
    """bf16 bit patterns (uint16) of elements [start, start+n) of the stream."""
    key = stream_key(seed, tid)
    sc = scale_f32(sigma)
    out = np.empty(n, dtype=np.uint16)
    for c0 in range(0, n, chunk):
        c1 = min(n, c0 + chunk)
        s = _irwin_hall(key, start + c0, c1 - c0)
        z = (s - IH_MEAN).astype(np.float32) * sc
        out[c0:c1] = f32_to_bf16_bits(z)
    return out


def normal(seed: int, tid: int, shape, sigma: float) -> np.ndarray:
    """fp32 array of bf16-representable values."""
    n = int(np.prod(shape)) if len(tuple(shape)) else 1
    return bf16_bits_to_f32(normal_bf16_bits(seed, tid, n, sigma)).reshape(shape)


def uniform_ids(seed: int, tid: int, n: int, vocab: int) -> np.ndarray:
    key = stream_key(seed, tid)
    idx = np.arange(n, dtype=np.uint64)
    with np.errstate(over="ignore"):
        h = _splitmix64(key + idx)
    return (h % np.uint64(vocab)).astype(np.int32)


def zipf_router_bias(seed: int, layer: int, n_experts: int, s: float = 1.2) -> np.ndarray:
    """Router bias of the skewed-routing configuration: N(0,0.02) - s*ln(e+1), rounded to bf16
    (hottest expert = id 0)."""
    b = normal(seed, tensor_id(TID_ROUTER_B, layer), (n_experts,), 0.02)
    skew = (-s * np.log(np.arange(1, n_experts + 1, dtype=np.float64))).astype(np.float32)
    return round_bf16(b + skew)


class MoELayerWeights:
    """One layer's MoE tensors in the flat-checkpoint layouts (fp32, bf16-representable)."""

    def __init__(self, hidden: int, intermediate: int, n_experts: int, seed: int, layer: int = 0,
                 sigma: float = 0.02, zipf_s: float | None = None):
        H, I, E = hidden, intermediate, n_experts
        self.hidden, self.intermediate, self.n_experts = H, I, E
        self.router_w = normal(seed, tensor_id(TID_ROUTER_W, layer), (E, H), sigma)
        if zipf_s is None:
            self.router_b = normal(seed, tensor_id(TID_ROUTER_B, layer), (E,), sigma)
        else:
            self.router_b = zipf_router_bias(seed, layer, E, zipf_s)
        self.mlp1_w = normal(seed, tensor_id(TID_MLP1_W, layer), (E, 2 * I, H), sigma)
        self.mlp1_b = normal(seed, tensor_id(TID_MLP1_B, layer), (E, 2 * I), sigma)
        self.mlp2_w = normal(seed, tensor_id(TID_MLP2_W, layer), (E, H, I), sigma)
        self.mlp2_b = normal(seed, tensor_id(TID_MLP2_B, layer), (E, H), sigma)


def activations(seed: int, T: int, hidden: int, sigma: float = 1.0, layer: int = 0) -> np.ndarray:
    return normal(seed, tensor_id(TID_ACTIVATION, layer), (T, hidden), sigma)
