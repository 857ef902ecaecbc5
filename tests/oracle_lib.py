"""ctypes access to the CPU oracles under oracle/ (test infrastructure; never used by the product).

``oracle()`` loads (building on first use) the C restatement; ``reference()`` loads the shared
object compiled from the reference's own run.cpp, or returns None where neither the prebuilt object
nor the reference sources are present.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent.parent
ORACLE_DIR = ROOT / "oracle"
# the reference checkout: GPTOSS_REFERENCE_DIR, else a directory called `reference` beside this repository (may be absent)
REF_SRC = Path(os.environ.get("GPTOSS_REFERENCE_DIR") or ROOT.parent / "reference")

MODE_CPU, MODE_GPU_BF16 = 0, 1
RULE_SELECTION, RULE_QSORT = 0, 1

_f32p = np.ctypeslib.ndpointer(dtype=np.float32, flags="C_CONTIGUOUS")
_i32p = np.ctypeslib.ndpointer(dtype=np.int32, flags="C_CONTIGUOUS")


class Dims(C.Structure):
    _fields_ = [("hidden", C.c_int), ("intermediate", C.c_int), ("n_experts", C.c_int),
                ("top_k", C.c_int), ("swiglu_limit", C.c_float)]


def _make(target: str) -> None:
    subprocess.run(["make", "-C", str(ORACLE_DIR), target, f"REF={REF_SRC}"], check=True,
                   stdout=subprocess.PIPE, stderr=subprocess.STDOUT)


def _opt(a, dtype):
    if a is None:
        return None
    assert a.dtype == dtype and a.flags.c_contiguous
    return a.ctypes.data_as(C.c_void_p)


class Oracle:
    def __init__(self, lib):
        self.lib = lib
        lib.oracle_router_scores.argtypes = [_f32p, _f32p, _f32p, C.c_int, C.c_int, C.c_int, _f32p]
        lib.oracle_topk_softmax.argtypes = [_f32p, C.c_int, C.c_int, C.c_int, C.c_int, _f32p, _i32p,
                                            C.c_void_p]
        lib.oracle_topk_softmax.restype = C.c_int
        lib.oracle_topk_margin.argtypes = [_f32p, C.c_int, C.c_int, C.c_int, _f32p]
        lib.oracle_counting_sort.argtypes = [_i32p, C.c_int, C.c_int, _i32p, _i32p]
        lib.oracle_counting_sort.restype = C.c_int
        lib.oracle_moe_block.argtypes = [C.POINTER(Dims), C.c_int, _f32p, C.c_int, _f32p, _i32p, _f32p,
                                         _f32p, _f32p, _f32p, C.c_int, C.c_int, _f32p, C.c_void_p,
                                         C.c_void_p]
        lib.oracle_combine_slots.argtypes = [_f32p, _f32p, C.c_int, C.c_int, C.c_int, _f32p]
        lib.oracle_num_threads.restype = C.c_int
        lib.oracle_synth_normal_f32.argtypes = [C.c_uint64, C.c_uint64, C.c_uint64, C.c_uint64, C.c_float,
                                                _f32p]

    def router_scores(self, t, wr, br):
        T, H = t.shape
        E = wr.shape[0]
        s = np.empty((T, E), np.float32)
        self.lib.oracle_router_scores(t, wr, br, T, H, E, s)
        return s

    def topk_softmax(self, scores, k, rule=RULE_SELECTION):
        T, E = scores.shape
        w = np.empty((T, k), np.float32)
        i = np.empty((T, k), np.int32)
        raw = np.empty((T, k), np.float32)
        ties = self.lib.oracle_topk_softmax(scores, T, E, k, rule, w, i, raw.ctypes.data_as(C.c_void_p))
        return w, i, raw, ties

    def topk_margin(self, scores, k):
        T, E = scores.shape
        m = np.empty(T, np.float32)
        self.lib.oracle_topk_margin(scores, T, E, k, m)
        return m

    def counting_sort(self, topk_i, E):
        flat = np.ascontiguousarray(topk_i.reshape(-1), dtype=np.int32)
        off = np.empty(E + 1, np.int32)
        srt = np.full(flat.size, -1, np.int32)
        placed = self.lib.oracle_counting_sort(flat, flat.size, E, off, srt)
        return off, srt, placed

    def moe_block(self, t, topk_w, topk_i, w, limit=7.0, mode=MODE_GPU_BF16, e_begin=0, e_end=None,
                  taps=False):
        """w: object with router_w/mlp1_w/mlp1_b/mlp2_w/mlp2_b in checkpoint layouts."""
        T, H = t.shape
        E, I2, _ = w.mlp1_w.shape
        I, k = I2 // 2, topk_i.shape[1]
        d = Dims(H, I, E, k, limit)
        out = np.empty((T, H), np.float32)
        hp = np.zeros((T * k, I), np.float32) if taps else None
        yp = np.zeros((T * k, H), np.float32) if taps else None
        self.lib.oracle_moe_block(C.byref(d), mode, np.ascontiguousarray(t), T,
                                  np.ascontiguousarray(topk_w), np.ascontiguousarray(topk_i),
                                  w.mlp1_w.reshape(-1), w.mlp1_b.reshape(-1), w.mlp2_w.reshape(-1),
                                  w.mlp2_b.reshape(-1), e_begin, E if e_end is None else e_end, out,
                                  _opt(hp, np.float32), _opt(yp, np.float32))
        return (out, hp, yp) if taps else out

    def combine_slots(self, y_pairs, topk_w):
        T, k = topk_w.shape
        H = y_pairs.shape[1]
        out = np.empty((T, H), np.float32)
        self.lib.oracle_combine_slots(np.ascontiguousarray(y_pairs), np.ascontiguousarray(topk_w), T, k,
                                      H, out)
        return out

    def num_threads(self):
        return self.lib.oracle_num_threads()

    def synth_normal(self, seed, tensor_id, shape, sigma, start=0):
        out = np.empty(shape, np.float32)
        self.lib.oracle_synth_normal_f32(seed, tensor_id, start, out.size, sigma, out.reshape(-1))
        return out

    def layer_weights(self, H, I, E, seed, layer=0, sigma=0.02):
        """Same tensors as synth.MoELayerWeights, generated by the multithreaded C generator."""
        from types import SimpleNamespace
        tid = lambda kind: kind + 16 * layer  # noqa: E731
        return SimpleNamespace(
            router_w=self.synth_normal(seed, tid(2), (E, H), sigma),
            router_b=self.synth_normal(seed, tid(3), (E,), sigma),
            mlp1_w=self.synth_normal(seed, tid(4), (E, 2 * I, H), sigma),
            mlp1_b=self.synth_normal(seed, tid(5), (E, 2 * I), sigma),
            mlp2_w=self.synth_normal(seed, tid(6), (E, H, I), sigma),
            mlp2_b=self.synth_normal(seed, tid(7), (E, H), sigma))


class Reference:
    """The reference's own CPU code (run.cpp) behind C entry points (oracle/ref_driver.cpp)."""

    def __init__(self, lib):
        self.lib = lib
        lib.ref_open.restype = C.c_void_p
        lib.ref_open.argtypes = [C.c_char_p]
        lib.ref_close.argtypes = [C.c_void_p]
        lib.ref_forward.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_void_p]
        lib.ref_forward.restype = C.c_int
        lib.ref_last_moe_state.argtypes = [C.c_void_p] + [C.c_void_p] * 5
        if hasattr(lib, "ref_forward_prefix"):
            lib.ref_forward_prefix.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int]
        lib.ref_moe_rows.argtypes = [_f32p, C.c_int, C.c_int, _f32p, _f32p, _f32p, _f32p, _f32p, _f32p,
                                     C.c_int, C.c_int, C.c_int, C.c_int, C.c_float, _f32p, C.c_void_p,
                                     C.c_void_p]
        lib.ref_moe_rows.restype = C.c_int
        lib.ref_num_threads.restype = C.c_int
        lib.ref_encode.argtypes = [C.c_char_p, C.c_int, C.c_char_p, C.c_void_p, C.c_int]
        lib.ref_encode.restype = C.c_int

    def encode(self, tokenizer_path, vocab_size, text, max_tokens=4096):
        """read_tokenizer + encode of the reference (tokenizer.cpp:49,268), no BOS/EOS."""
        out = np.zeros(max_tokens, np.int32)
        n = self.lib.ref_encode(str(tokenizer_path).encode(), vocab_size, text.encode(), out.ctypes.data_as(C.c_void_p),
                                max_tokens)
        return out[:n].tolist()

    def open(self, path):
        return self.lib.ref_open(str(path).encode())

    def close(self, h):
        self.lib.ref_close(h)

    def forward(self, h, token, pos, logits=None):
        return self.lib.ref_forward(h, int(token), int(pos), _opt(logits, np.float32))

    def forward_prefix(self, h, token, pos, n_layers):
        """forward() through the first n_layers layers only; last_moe_state then describes layer n_layers - 1."""
        self.lib.ref_forward_prefix(h, int(token), int(pos), int(n_layers))

    def last_moe_state(self, h, H, E, k):
        t = np.empty(H, np.float32)
        v = np.empty(k, np.float32)
        i = np.empty(k, np.int32)
        agg = np.empty(H, np.float32)
        sc = np.empty(E, np.float32)
        self.lib.ref_last_moe_state(h, *[a.ctypes.data_as(C.c_void_p) for a in (t, v, i, agg, sc)])
        return t, v, i, agg, sc

    def moe_rows(self, t, w, k, limit=7.0, rows=None):
        T, H = t.shape
        E, I2, _ = w.mlp1_w.shape
        r0, r1 = (0, T) if rows is None else rows
        agg = np.zeros((T, H), np.float32)
        tv = np.zeros((T, k), np.float32)
        ti = np.zeros((T, k), np.int32)
        self.lib.ref_moe_rows(np.ascontiguousarray(t), r0, r1, w.router_w.reshape(-1),
                              np.ascontiguousarray(w.router_b), w.mlp1_w.reshape(-1),
                              w.mlp1_b.reshape(-1), w.mlp2_w.reshape(-1), w.mlp2_b.reshape(-1), H,
                              I2 // 2, E, k, limit, agg, tv.ctypes.data_as(C.c_void_p),
                              ti.ctypes.data_as(C.c_void_p))
        return agg, tv, ti

    def num_threads(self):
        return self.lib.ref_num_threads()


_cache = {}


def oracle() -> Oracle:
    if "o" not in _cache:
        so = ORACLE_DIR / "_build" / "libmoe_oracle.so"
        src_newer = (not so.exists()) or any(
            (ORACLE_DIR / f).stat().st_mtime > so.stat().st_mtime for f in ("moe_oracle.c", "moe_oracle.h"))
        if src_newer:
            _make("oracle")
        _cache["o"] = Oracle(C.CDLL(str(so)))
    return _cache["o"]


def reference():
    if "r" not in _cache:
        so = ORACLE_DIR / "_ref" / "libref_cpu.so"
        if not so.exists() and (REF_SRC / "run.cpp").exists():
            _make("ref")
        _cache["r"] = Reference(C.CDLL(str(so))) if so.exists() else None
    return _cache["r"]
