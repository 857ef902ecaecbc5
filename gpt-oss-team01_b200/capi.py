"""ctypes binding of the C ABI in ``include/gptoss_b200.h`` (the CUDA shared library).

There is no CPU fallback: if the library has not been built, ``load()`` raises.
"""
from __future__ import annotations

import ctypes as C
import subprocess
from pathlib import Path

import os

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
# GPTOSS_B200_LIB points the binding at another build of the same C ABI (e.g. a tuning variant)
LIB_PATH = Path(os.environ.get("GPTOSS_B200_LIB", CSRC / "libgptoss_b200.so"))
SOURCES = ["routing.cu", "router.cu", "grouped_gemm.cu", "grouped_gemm_pair.cu", "comm.cu", "convert.cu", "capi.cu", "model_kernels.cu",
           "model.cu"]
HEADERS = ["common.cuh", "kernels.cuh", "tcgen05.cuh", "gemm_tile.cuh", "../../include/gptoss_b200.h"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "-shared", "--threads", "4"]

OK, ERR_BAD_ARG, ERR_CUDA, ERR_TIMEOUT, ERR_UNSUPPORTED, ERR_STATE = range(6)
WIRE_F32, WIRE_BF16 = 0, 1
IPC_HANDLE_BYTES = 64
(TAP_SCORES, TAP_TOPK_W, TAP_TOPK_I, TAP_OFFSETS, TAP_SORTED, TAP_X_PACKED, TAP_GATE_UP,
 TAP_Y_PAIRS, TAP_GATHERED) = range(9)

# every symbol include/gptoss_b200.h declares
EXPORTS = [
    "gptoss_ctx_create", "gptoss_ctx_destroy", "gptoss_last_error", "gptoss_ctx_status",
    "gptoss_upload_layer", "gptoss_fill_layer_synthetic", "gptoss_set_router_bias",
    "gptoss_download_layer", "gptoss_moe_forward", "gptoss_moe_forward_host",
    "gptoss_moe_forward_partial", "gptoss_moe_route", "gptoss_moe_mlp1_swiglu", "gptoss_moe_mlp2",
    "gptoss_moe_combine", "gptoss_topk_softmax", "gptoss_moe_build_offsets", "gptoss_read_tap",
    "gptoss_synth_normal_bf16", "gptoss_version", "gptoss_moe_build_offsets_noalloc",
    "gptoss_noalloc_last_error", "gptoss_comm_export", "gptoss_comm_attach",
    "gptoss_comm_attach_local", "gptoss_comm_set_timeout_ms", "gptoss_moe_push_to_owners",
    "gptoss_moe_owner_combine", "gptoss_moe_add_delta", "gptoss_model_create", "gptoss_model_destroy",
    "gptoss_model_last_error", "gptoss_model_load_bin", "gptoss_model_load_mem", "gptoss_model_fill_synthetic", "gptoss_model_step",
    "gptoss_model_read_logits", "gptoss_moe_slice_bounds", "gptoss_moe_gather_slice", "gptoss_moe_sliced_push",
    "gptoss_moe_sliced_combine", "gptoss_moe_forward_sliced", "gptoss_model_create_ep", "gptoss_model_moe_ctx",
    "gptoss_model_slice", "gptoss_model_step_begin", "gptoss_model_layer_attention", "gptoss_model_layer_moe_push",
    "gptoss_model_layer_moe_combine", "gptoss_model_step_end", "gptoss_comm_rendezvous", "gptoss_moe_gather_rows", "gptoss_moe_forward_host_sliced",
    "gptoss_moe_route_local", "gptoss_moe_route_finish", "gptoss_moe_sliced_route",
    "gptoss_moe_dispatch_route", "gptoss_moe_dispatch_rows", "gptoss_moe_dispatch_push", "gptoss_moe_forward_dispatch",
    "gptoss_launch_count", "gptoss_argmax_rows", "gptoss_model_step_rows", "gptoss_model_step_seqs",
    "gptoss_moe_forward_host_submit", "gptoss_moe_forward_host_sliced_submit", "gptoss_moe_forward_host_wait",
    "gptoss_model_layer_moe_dispatch",
]


class ModelConfig(C.Structure):
    """The 15-field checkpoint header (run.cpp:25-45)."""
    _fields_ = [(n, C.c_int) for n in ("vocab_size", "hidden_dim", "n_experts", "experts_per_token",
                                       "intermediate_dim", "n_layers", "head_dim", "n_attn_heads", "n_kv_heads",
                                       "seq_len", "initial_context_length")] + \
               [("rope_theta", C.c_float), ("rope_scaling_factor", C.c_float), ("sliding_window", C.c_int),
                ("swiglu_limit", C.c_float)]


class MoEDims(C.Structure):
    _fields_ = [("hidden", C.c_int), ("intermediate", C.c_int), ("n_experts", C.c_int),
                ("top_k", C.c_int), ("n_layers", C.c_int), ("swiglu_limit", C.c_float)]


def needs_build() -> bool:
    if not LIB_PATH.exists():
        return True
    t = LIB_PATH.stat().st_mtime
    return any((CSRC / f).stat().st_mtime > t for f in SOURCES + HEADERS)


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compiles the library for sm_100a with nvcc (works without a GPU)."""
    if not force and not needs_build():
        return LIB_PATH
    cmd = ["nvcc", *NVCC_FLAGS, "-o", str(LIB_PATH), *SOURCES]
    if verbose:
        cmd[1:1] = ["-Xptxas", "-v"]
    r = subprocess.run(cmd, cwd=CSRC, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed:\n{r.stdout}")
    if verbose:
        print(r.stdout)
    return LIB_PATH


_lib = None


def load() -> C.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise RuntimeError(f"{LIB_PATH} is missing: run `python -c 'import __graft_entry__ as e; "
                           "e.build()'` first (there is no CPU fallback)")
    lib = C.CDLL(str(LIB_PATH))
    vp, i32, u64, f32 = C.c_void_p, C.c_int, C.c_uint64, C.c_float
    ctxp = vp
    sig = {
        "gptoss_ctx_create": ([C.POINTER(MoEDims), i32, i32, i32, i32, i32, C.POINTER(vp)], i32),
        "gptoss_ctx_destroy": ([ctxp], i32),
        "gptoss_last_error": ([ctxp], C.c_char_p),
        "gptoss_ctx_status": ([ctxp], i32),
        "gptoss_upload_layer": ([ctxp, i32, vp, vp, vp, vp, vp, vp], i32),
        "gptoss_fill_layer_synthetic": ([ctxp, i32, u64, f32], i32),
        "gptoss_set_router_bias": ([ctxp, i32, vp], i32),
        "gptoss_download_layer": ([ctxp, i32, vp, vp, vp, vp, vp, vp], i32),
        "gptoss_moe_forward": ([ctxp, i32, i32, vp, vp, vp], i32),
        "gptoss_moe_forward_host": ([ctxp, i32, i32, vp, vp], i32),
        "gptoss_moe_forward_partial": ([ctxp, i32, i32, vp, vp, vp], i32),
        "gptoss_moe_route": ([ctxp, i32, i32, vp, vp], i32),
        "gptoss_moe_mlp1_swiglu": ([ctxp, i32, vp], i32),
        "gptoss_moe_mlp2": ([ctxp, i32, vp], i32),
        "gptoss_moe_combine": ([ctxp, i32, vp, i32, vp], i32),
        "gptoss_topk_softmax": ([ctxp, i32, vp, vp, vp, vp], i32),
        "gptoss_moe_build_offsets": ([ctxp, i32, vp, vp, vp, vp], i32),
        "gptoss_read_tap": ([ctxp, i32, vp, u64], i32),
        "gptoss_synth_normal_bf16": ([vp, u64, u64, u64, u64, f32, vp], i32),
        "gptoss_version": ([], C.c_char_p),
        "gptoss_moe_build_offsets_noalloc": ([i32, i32, i32, vp, vp, vp, vp], i32),
        "gptoss_noalloc_last_error": ([], C.c_char_p),
        "gptoss_comm_export": ([ctxp, vp], i32),
        "gptoss_comm_attach": ([ctxp, vp], i32),
        "gptoss_comm_attach_local": ([ctxp, C.POINTER(vp)], i32),
        "gptoss_comm_set_timeout_ms": ([ctxp, i32], i32),
        "gptoss_moe_push_to_owners": ([ctxp, i32, vp], i32),
        "gptoss_moe_owner_combine": ([ctxp, vp], i32),
        "gptoss_moe_add_delta": ([ctxp, vp, vp], i32),
        "gptoss_model_create": ([C.POINTER(ModelConfig), i32, i32, i32, C.POINTER(vp)], i32),
        "gptoss_model_destroy": ([vp], i32),
        "gptoss_model_last_error": ([vp], C.c_char_p),
        "gptoss_model_load_bin": ([vp, C.c_char_p], i32),
        "gptoss_model_load_mem": ([vp, vp, u64], i32),
        "gptoss_model_fill_synthetic": ([vp, u64, f32], i32),
        "gptoss_model_step": ([vp, vp, i32, i32, vp], i32),
        "gptoss_model_read_logits": ([vp, i32, vp], i32),
        "gptoss_moe_slice_bounds": ([ctxp, i32, C.POINTER(i32), C.POINTER(i32)], i32),
        "gptoss_moe_gather_slice": ([ctxp, i32, vp, vp, vp, vp], i32),
        "gptoss_moe_sliced_push": ([ctxp, i32, i32, vp], i32),
        "gptoss_moe_sliced_combine": ([ctxp, vp, vp], i32),
        "gptoss_moe_forward_sliced": ([ctxp, i32, i32, vp, vp], i32),
        "gptoss_model_create_ep": ([C.POINTER(ModelConfig), i32, i32, i32, i32, i32, C.POINTER(vp)], i32),
        "gptoss_model_moe_ctx": ([vp], vp),
        "gptoss_model_slice": ([vp, i32, C.POINTER(i32), C.POINTER(i32)], i32),
        "gptoss_model_step_begin": ([vp, vp, i32, i32], i32),
        "gptoss_model_layer_attention": ([vp, i32], i32),
        "gptoss_model_layer_moe_push": ([vp, i32], i32),
        "gptoss_model_layer_moe_dispatch": ([vp, i32], i32),
        "gptoss_model_layer_moe_combine": ([vp, i32], i32),
        "gptoss_model_step_end": ([vp, vp], i32),
        "gptoss_comm_rendezvous": ([ctxp, vp], i32),
        "gptoss_moe_gather_rows": ([ctxp, i32, vp, vp], i32),
        "gptoss_moe_forward_host_sliced": ([ctxp, i32, i32, vp, vp], i32),
        "gptoss_moe_route_local": ([ctxp, i32, i32, vp, vp], i32),
        "gptoss_moe_route_finish": ([ctxp, i32, i32, vp, vp], i32),
        "gptoss_moe_sliced_route": ([ctxp, i32, i32, vp], i32),
        "gptoss_moe_dispatch_route": ([ctxp, i32, i32, vp, vp], i32),
        "gptoss_moe_dispatch_rows": ([ctxp, i32, i32, vp, vp], i32),
        "gptoss_moe_dispatch_push": ([ctxp, i32, vp], i32),
        "gptoss_moe_forward_dispatch": ([ctxp, i32, i32, vp, vp, vp], i32),
        "gptoss_launch_count": ([], u64),
        "gptoss_argmax_rows": ([vp, i32, i32, vp, vp], i32),
        "gptoss_model_step_rows": ([vp, vp, vp, i32, i32, vp], i32),
        "gptoss_model_step_seqs": ([vp, vp, vp, vp, i32, vp], i32),
        "gptoss_moe_forward_host_submit": ([ctxp, i32, i32, vp, vp], i32),
        "gptoss_moe_forward_host_sliced_submit": ([ctxp, i32, i32, vp, vp], i32),
        "gptoss_moe_forward_host_wait": ([ctxp], i32),
    }
    for name, (args, res) in sig.items():
        fn = getattr(lib, name)
        fn.argtypes, fn.restype = args, res
    _lib = lib
    return lib
