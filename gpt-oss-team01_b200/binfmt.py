"""The reference's flat checkpoint format (``model.bin``): reader, writer, seeded generator.

Layout (reference export_model_bin/gpt-oss-20b/export_model_bin.py:34-62, struct at run.cpp:25-45,
pointer walk at run.cpp:194-233): fifteen little-endian 4-byte header fields, then fp32 tensors, each
category stacked over layers, in the order of ``TENSOR_ORDER`` below.
"""
from __future__ import annotations

import dataclasses
import struct

import numpy as np

from . import synth

HEADER_FMT = "<11i2fif"  # 11 ints, 2 floats, 1 int, 1 float
HEADER_BYTES = 60


@dataclasses.dataclass
class Config:
    vocab_size: int
    hidden_dim: int
    n_experts: int
    experts_per_token: int
    intermediate_dim: int
    n_layers: int
    head_dim: int
    n_attn_heads: int
    n_kv_heads: int
    seq_len: int
    initial_context_length: int
    rope_theta: float
    rope_scaling_factor: float
    sliding_window: int
    swiglu_limit: float

    def pack(self) -> bytes:
        return struct.pack(HEADER_FMT, *dataclasses.astuple(self))

    @staticmethod
    def unpack(raw: bytes) -> "Config":
        return Config(*struct.unpack(HEADER_FMT, raw[:HEADER_BYTES]))


# dims of export_model_bin/gpt-oss-7m/config.json:2-16 (seq_len shortened by callers as needed)
def config_7m(seq_len: int = 2048) -> Config:
    return Config(201088, 32, 32, 4, 64, 2, 32, 2, 1, seq_len, 4096, 150000.0, 32.0, 128, 7.0)


# export_model_bin/gpt-oss-20b/config.json:2-16
def config_20b(seq_len: int = 1024) -> Config:
    return Config(201088, 2880, 32, 4, 2880, 24, 64, 64, 8, seq_len, 4096, 150000.0, 32.0, 128, 7.0)


# export_model_bin/gpt-oss-120b/config.json:2-16
def config_120b(seq_len: int = 1024) -> Config:
    return Config(201088, 2880, 128, 4, 2880, 36, 64, 64, 8, seq_len, 4096, 150000.0, 32.0, 128, 7.0)


def tensor_shapes(c: Config):
    """(name, shape) in file order."""
    L, H, E, I = c.n_layers, c.hidden_dim, c.n_experts, c.intermediate_dim
    qkv = c.head_dim * (c.n_attn_heads + 2 * c.n_kv_heads)
    return [
        ("embedding", (c.vocab_size, H)),
        ("unembedding", (c.vocab_size, H)),
        ("attn_norm", (L, H)),
        ("mlp_norm", (L, H)),
        ("final_norm", (H,)),
        ("qkv_w", (L, qkv, H)),
        ("qkv_b", (L, qkv)),
        ("attn_out_w", (L, H, c.head_dim * c.n_attn_heads)),
        ("attn_out_b", (L, H)),
        ("sinks", (L, c.n_attn_heads)),
        ("router_w", (L, E, H)),
        ("router_b", (L, E)),
        ("mlp1_w", (L, E, 2 * I, H)),
        ("mlp1_b", (L, E, 2 * I)),
        ("mlp2_w", (L, E, H, I)),
        ("mlp2_b", (L, E, H)),
    ]


TENSOR_ORDER = [n for n, _ in tensor_shapes(config_7m())]
_NORMS = ("attn_norm", "mlp_norm", "final_norm")


def write_synthetic(path: str, c: Config, seed: int, sigma: float = 0.02) -> None:
    """Random-init checkpoint: every tensor N(0, sigma) rounded to bf16 from the seeded generator,
    except the three RMSNorm scales, which are 1.0 (an all-N(0,0.02) scale would shrink the
    activations by 50x at every norm).  Stream ids: 64 + position in file order."""
    with open(path, "wb") as f:
        f.write(c.pack())
        for pos, (name, shape) in enumerate(tensor_shapes(c)):
            n = int(np.prod(shape))
            if name in _NORMS:
                np.ones(n, dtype=np.float32).tofile(f)
                continue
            for c0 in range(0, n, 1 << 24):
                c1 = min(n, c0 + (1 << 24))
                bits = synth.normal_bf16_bits(seed, 64 + pos, c1 - c0, sigma, start=c0)
                synth.bf16_bits_to_f32(bits).tofile(f)


def read(path: str):
    """Returns (Config, dict name -> fp32 memmap view) without loading the file."""
    with open(path, "rb") as f:
        c = Config.unpack(f.read(HEADER_BYTES))
    mm = np.memmap(path, dtype=np.float32, mode="r", offset=HEADER_BYTES)
    out, off = {}, 0
    for name, shape in tensor_shapes(c):
        n = int(np.prod(shape))
        out[name] = mm[off:off + n].reshape(shape)
        off += n
    if off != mm.size:
        raise ValueError(f"{path}: expected {off} floats after the header, file holds {mm.size}")
    return c, out


def write_synthetic_tokenizer(path: str, vocab_size: int) -> None:
    """A stand-in ``tokenizer.bin`` in the reference's binary format (export_tokenizer_bin.py:128-138, reader
    tokenizer.cpp:49-102): ``int32 max_token_length`` then, per token, ``float32 score, int32 len, bytes``.
    The real vocabulary cannot be obtained offline, so tokens 0..255 are the single raw bytes (the reference
    looks pieces up by their raw bytes, tokenizer.cpp:129-134,170-176; every text then encodes to its UTF-8
    bytes, id = byte value) and the rest are unmergeable fillers (score -1e30, tokenizer.cpp:160-161)."""
    with open(path, "wb") as f:
        f.write(struct.pack("<i", 24))
        for i in range(vocab_size):
            s = bytes([i]) if i < 256 else f"<|synthetic_{i}|>".encode()
            f.write(struct.pack("<fi", 0.0 if i < 256 else -1e30, len(s)))
            f.write(s)
