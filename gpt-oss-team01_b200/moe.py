"""Host-side operator interface of the MoE block, over the C ABI.

Mirrors the reference's per-layer launchers (getp-csrc/include/layer_hip_batch.hpp:103-240,
getp-csrc/include/kernel.hpp): same operator names and argument meaning, device buffers in,
device buffers out, an explicit stream last.  Errors raise ``GptossError`` (the reference aborts).
PyTorch is used only to hold device memory and streams.
"""
from __future__ import annotations

import ctypes as C
from types import SimpleNamespace

import numpy as np
import torch

from . import capi


class GptossError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"gptoss status {code}: {message}")
        self.code = code


def _ptr(t):
    if t is None:
        return None
    if isinstance(t, torch.Tensor):
        assert t.is_contiguous()
        return C.c_void_p(t.data_ptr())
    if isinstance(t, np.ndarray):
        assert t.flags.c_contiguous
        return C.c_void_p(t.ctypes.data)
    raise TypeError(type(t))


def slice_bounds(rank: int, world: int, n_tokens: int):
    """(first token, token count) of the slice rank ``rank`` owns in a batch of ``n_tokens``: contiguous slices of
    ceil(n_tokens / world) tokens rounded up to a multiple of 8, the last ones shorter or empty (same rule as
    gptoss_moe_slice_bounds)."""
    per = ((n_tokens + world - 1) // world + 7) // 8 * 8  # a multiple of the routing block of 8 tokens
    first = rank * per
    count = max(0, min(per, n_tokens - first))
    return (first if count else n_tokens), count


def _stream(stream):
    if stream is None:
        stream = torch.cuda.current_stream()
    return C.c_void_p(stream.cuda_stream)


class MoEBlock:
    """One GPU's context: weights of `n_layers` layers (this rank's experts) + all scratch."""

    def __init__(self, hidden, intermediate, n_experts, top_k, n_layers=1, swiglu_limit=7.0, device=0,
                 rank=0, world=1, max_tokens=1024, wire=capi.WIRE_F32):
        self.lib = capi.load()
        self.H, self.I, self.E, self.k, self.L = hidden, intermediate, n_experts, top_k, n_layers
        self.rank, self.world, self.max_tokens = rank, world, max_tokens
        self.n_local = n_experts // world if world > 0 and n_experts % max(world, 1) == 0 else 0
        self.device = torch.device("cuda", device)
        self._ctx = C.c_void_p()
        dims = capi.MoEDims(hidden, intermediate, n_experts, top_k, n_layers, swiglu_limit)
        rc = self.lib.gptoss_ctx_create(C.byref(dims), device, rank, world, max_tokens, wire,
                                        C.byref(self._ctx))
        if rc != capi.OK:
            self._ctx = C.c_void_p()
            raise GptossError(rc, "gptoss_ctx_create failed (bad dimensions, no sm_100 device, or out of memory)")

    # -- plumbing -------------------------------------------------------------------------------------
    def _check(self, rc):
        if rc != capi.OK:
            raise GptossError(rc, self.lib.gptoss_last_error(self._ctx).decode())

    def close(self):
        if self._ctx:
            self.lib.gptoss_ctx_destroy(self._ctx)
            self._ctx = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def status(self):
        """Synchronises and raises if a kernel reported a device-side time-out."""
        self._check(self.lib.gptoss_ctx_status(self._ctx))

    # -- weights ----------------------------------------------------------------------------------------
    def upload_layer(self, layer, w):
        """w: object with router_w [E,H], router_b [E], mlp1_w [E,2I,H], mlp1_b [E,2I], mlp2_w [E,H,I],
        mlp2_b [E,H] as fp32 numpy arrays in the checkpoint layouts."""
        arrs = [np.ascontiguousarray(getattr(w, n), dtype=np.float32)
                for n in ("router_w", "router_b", "mlp1_w", "mlp1_b", "mlp2_w", "mlp2_b")]
        self._check(self.lib.gptoss_upload_layer(self._ctx, layer, *[_ptr(a) for a in arrs]))

    def fill_layer_synthetic(self, layer, seed, sigma=0.02):
        self._check(self.lib.gptoss_fill_layer_synthetic(self._ctx, layer, seed, sigma))

    def set_router_bias(self, layer, bias):
        b = np.ascontiguousarray(bias, dtype=np.float32)
        assert b.shape == (self.E,)
        self._check(self.lib.gptoss_set_router_bias(self._ctx, layer, _ptr(b)))

    def download_layer(self, layer, big=True):
        H, I, E, EL = self.H, self.I, self.E, self.n_local
        w = SimpleNamespace(
            router_w=np.empty((E, H), np.float32), router_b=np.empty(E, np.float32),
            mlp1_w=np.empty((EL, 2 * I, H), np.float32) if big else None,
            mlp1_b=np.empty((EL, 2 * I), np.float32),
            mlp2_w=np.empty((EL, H, I), np.float32) if big else None,
            mlp2_b=np.empty((EL, H), np.float32))
        self._check(self.lib.gptoss_download_layer(
            self._ctx, layer, _ptr(w.router_w), _ptr(w.router_b), _ptr(w.mlp1_w), _ptr(w.mlp1_b),
            _ptr(w.mlp2_w), _ptr(w.mlp2_b)))
        return w

    # -- peer memory (fused cross-GPU combine) ----------------------------------------------------------------
    def attach_peers(self, group=None):
        """Exchanges the IPC handles of the combine buffers over torch.distributed (one process per GPU)
        and attaches all ranks; afterwards forward() runs the fused peer-store combine."""
        import torch.distributed as dist
        mine = (C.c_uint8 * capi.IPC_HANDLE_BYTES)()
        self._check(self.lib.gptoss_comm_export(self._ctx, mine))
        gathered = [None] * self.world
        dist.all_gather_object(gathered, bytes(mine), group=group)
        blob = b"".join(gathered)
        assert len(blob) == self.world * capi.IPC_HANDLE_BYTES
        buf = (C.c_uint8 * len(blob)).from_buffer_copy(blob)
        self._check(self.lib.gptoss_comm_attach(self._ctx, buf))
        dist.barrier(group=group)

    @staticmethod
    def attach_local(blocks):
        """Attaches contexts that live in this process (ranks 0..world-1, in order) to one another."""
        arr = (C.c_void_p * len(blocks))(*[b._ctx for b in blocks])
        for b in blocks:
            b._check(b.lib.gptoss_comm_attach_local(b._ctx, arr))

    def rendezvous(self, stream=None):
        """Device-side meeting point of the ranks on the stream (no data)."""
        self._check(self.lib.gptoss_comm_rendezvous(self._ctx, _stream(stream)))

    def set_peer_timeout_ms(self, ms):
        self._check(self.lib.gptoss_comm_set_timeout_ms(self._ctx, ms))

    def push_to_owners(self, layer, stream=None):
        """down GEMM with peer stores into the owners' buffers + "pushed" flag"""
        self._check(self.lib.gptoss_moe_push_to_owners(self._ctx, layer, _stream(stream)))

    def owner_combine(self, stream=None):
        self._check(self.lib.gptoss_moe_owner_combine(self._ctx, _stream(stream)))

    def add_delta(self, x, stream=None):
        self._check(self.lib.gptoss_moe_add_delta(self._ctx, _ptr(x), _stream(stream)))

    # -- the per-layer operator -----------------------------------------------------------------------------
    def forward(self, layer, t, x, stream=None):
        """x[T,H] (fp32 cuda) += MoE(t[T,H] (bf16 cuda)), asynchronous on the stream."""
        T = t.shape[0]
        assert t.dtype == torch.bfloat16 and x.dtype == torch.float32
        assert t.shape == (T, self.H) and x.shape == (T, self.H)
        self._check(self.lib.gptoss_moe_forward(self._ctx, layer, T, _ptr(t), _ptr(x), _stream(stream)))

    def forward_partial(self, layer, t, partial, stream=None):
        T = t.shape[0]
        assert t.dtype == torch.bfloat16 and partial.dtype == torch.float32
        self._check(self.lib.gptoss_moe_forward_partial(self._ctx, layer, T, _ptr(t), _ptr(partial),
                                                        _stream(stream)))

    def forward_host(self, layer, t_bits, x):
        """Host buffers: t_bits uint16 [T,H] (bf16 bit patterns), x fp32 [T,H] in/out (numpy arrays or
        pinned CPU torch tensors).  Synchronous."""
        T = t_bits.shape[0]
        self._check(self.lib.gptoss_moe_forward_host(self._ctx, layer, T, _ptr(t_bits), _ptr(x)))

    def forward_host_submit(self, layer, t_bits, x):
        """First half of forward_host: queues the uploads, the kernels and the download; at most two calls in flight.
        The buffers must stay alive (pinned, for the overlap) until the matching forward_host_wait()."""
        self._check(self.lib.gptoss_moe_forward_host_submit(self._ctx, layer, t_bits.shape[0], _ptr(t_bits), _ptr(x)))

    def forward_host_wait(self):
        """Blocks until the oldest submitted host-buffer call has finished; its x then holds the result."""
        self._check(self.lib.gptoss_moe_forward_host_wait(self._ctx))

    # -- token-sliced form: every rank holds only its rows of the residual stream ---------------------------------
    def slice(self, n_tokens):
        """(first token, token count) of this rank's slice of a batch of n_tokens."""
        return slice_bounds(self.rank, self.world, n_tokens)

    def gather_slice(self, n_tokens, x_slice, norm_w, add=None, stream=None):
        """x_slice (+)= add; bf16(RMSNorm(x_slice) * norm_w) stored into every rank's gathered activations."""
        self._check(self.lib.gptoss_moe_gather_slice(self._ctx, n_tokens, _ptr(x_slice), _ptr(add) if add is not None else None,
                                                     _ptr(norm_w), _stream(stream)))

    def gather_rows(self, n_tokens, t_slice, stream=None):
        """this rank's (already normalised) bf16 rows copied into every rank's gathered activations."""
        self._check(self.lib.gptoss_moe_gather_rows(self._ctx, n_tokens, _ptr(t_slice) if t_slice is not None else None,
                                                    _stream(stream)))

    def sliced_route(self, layer, n_tokens, stream=None):
        """routes this rank's own rows of its gathered buffer, rows stored to every rank (no waiting)"""
        self._check(self.lib.gptoss_moe_sliced_route(self._ctx, layer, n_tokens, _stream(stream)))

    def route_local(self, layer, t, stream=None):
        """replicated activations t [T,H]: this rank routes its token slice and stores the rows to every rank"""
        self._check(self.lib.gptoss_moe_route_local(self._ctx, layer, t.shape[0], _ptr(t), _stream(stream)))

    def route_finish(self, layer, t, stream=None):
        """waits for every rank's routing rows, then counting sort + gather of the rows of this rank's experts"""
        self._check(self.lib.gptoss_moe_route_finish(self._ctx, layer, t.shape[0], _ptr(t), _stream(stream)))

    def sliced_push(self, layer, n_tokens, stream=None):
        self._check(self.lib.gptoss_moe_sliced_push(self._ctx, layer, n_tokens, _stream(stream)))

    def sliced_combine(self, x_slice, stream=None):
        self._check(self.lib.gptoss_moe_sliced_combine(self._ctx, _ptr(x_slice), _stream(stream)))

    def forward_sliced(self, layer, n_tokens, x_slice, stream=None):
        self._check(self.lib.gptoss_moe_forward_sliced(self._ctx, layer, n_tokens, _ptr(x_slice), _stream(stream)))

    # -- dispatch form: token rows go only to the ranks whose experts they selected -----------------------------
    def dispatch_route(self, layer, n_tokens, t_slice, stream=None):
        """routes this rank's rows t_slice [slice count, H] (bf16 cuda) and stores the routing rows to every rank"""
        self._check(self.lib.gptoss_moe_dispatch_route(self._ctx, layer, n_tokens, _ptr(t_slice) if t_slice is not None else None,
                                                       _stream(stream)))

    def dispatch_rows(self, layer, n_tokens, t_slice, stream=None):
        """waits for every rank's routing rows; grouping of the batch; this rank's rows to the experts' owners"""
        self._check(self.lib.gptoss_moe_dispatch_rows(self._ctx, layer, n_tokens, _ptr(t_slice) if t_slice is not None else None,
                                                      _stream(stream)))

    def dispatch_push(self, layer, stream=None):
        """waits for every rank's rows; gate/up GEMM + SwiGLU; down GEMM pushing to the tokens' owners"""
        self._check(self.lib.gptoss_moe_dispatch_push(self._ctx, layer, _stream(stream)))

    def forward_dispatch(self, layer, n_tokens, t_slice, x_slice, stream=None):
        """x_slice (+)= MoE(t_slice) for this rank's rows of a batch of n_tokens; every rank calls it"""
        self._check(self.lib.gptoss_moe_forward_dispatch(self._ctx, layer, n_tokens, _ptr(t_slice) if t_slice is not None else None,
                                                         _ptr(x_slice) if x_slice is not None else None, _stream(stream)))

    def forward_host_sliced(self, layer, n_tokens, t_bits_slice, x_slice):
        """Host buffers holding THIS RANK'S rows of a batch of n_tokens: t_bits_slice uint16 [n,H], x_slice fp32 [n,H]
        in/out.  Synchronous; every rank calls it."""
        self._check(self.lib.gptoss_moe_forward_host_sliced(self._ctx, layer, n_tokens, _ptr(t_bits_slice), _ptr(x_slice)))

    def forward_host_sliced_submit(self, layer, n_tokens, t_bits_slice, x_slice):
        """First half of forward_host_sliced (forward_host_wait is the other); every rank submits the same calls."""
        self._check(self.lib.gptoss_moe_forward_host_sliced_submit(self._ctx, layer, n_tokens, _ptr(t_bits_slice), _ptr(x_slice)))

    # -- stages (reference launcher names in the docstrings) --------------------------------------------------
    def route(self, layer, t, stream=None):
        """router_gemm_v2 + topk_softmax_batched + moe_build_offsets_hip + moe_pack_inputs_hip"""
        self._check(self.lib.gptoss_moe_route(self._ctx, layer, t.shape[0], _ptr(t), _stream(stream)))

    def mlp1_swiglu(self, layer, stream=None):
        """moe_mlp1_swiglu_fused_hip"""
        self._check(self.lib.gptoss_moe_mlp1_swiglu(self._ctx, layer, _stream(stream)))

    def mlp2(self, layer, stream=None):
        """moe_mlp2_forward_hip (+ the gate-weight multiply of moe_agg_kernel_120b)"""
        self._check(self.lib.gptoss_moe_mlp2(self._ctx, layer, _stream(stream)))

    def combine(self, x, residual=True, stream=None):
        """moe_scatter_aggregate_ep_hip + add_vector_batched"""
        self._check(self.lib.gptoss_moe_combine(self._ctx, x.shape[0], _ptr(x), int(residual),
                                                _stream(stream)))

    def topk_softmax(self, scores, stream=None):
        """topk_softmax_batched on a caller-supplied fp32 [T,E] cuda tensor -> (weights, ids)."""
        T = scores.shape[0]
        assert scores.dtype == torch.float32 and scores.shape == (T, self.E)
        w = torch.empty((T, self.k), dtype=torch.float32, device=scores.device)
        i = torch.empty((T, self.k), dtype=torch.int32, device=scores.device)
        self._check(self.lib.gptoss_topk_softmax(self._ctx, T, _ptr(scores), _ptr(w), _ptr(i),
                                                 _stream(stream)))
        return w, i

    def moe_build_offsets(self, topk_i, stream=None):
        """moe_build_offsets on a caller-supplied int32 [T,k] cuda tensor -> (offsets [E+1], sorted [T*k])."""
        T = topk_i.shape[0]
        assert topk_i.dtype == torch.int32 and topk_i.shape == (T, self.k)
        off = torch.empty(self.E + 1, dtype=torch.int32, device=topk_i.device)
        srt = torch.full((T * self.k,), -1, dtype=torch.int32, device=topk_i.device)
        self._check(self.lib.gptoss_moe_build_offsets(self._ctx, T, _ptr(topk_i), _ptr(off), _ptr(srt),
                                                      _stream(stream)))
        return off, srt

    # -- taps ---------------------------------------------------------------------------------------------
    _TAPS = {
        "scores": (capi.TAP_SCORES, np.float32), "topk_w": (capi.TAP_TOPK_W, np.float32),
        "topk_i": (capi.TAP_TOPK_I, np.int32), "offsets": (capi.TAP_OFFSETS, np.int32),
        "sorted": (capi.TAP_SORTED, np.int32), "x_packed": (capi.TAP_X_PACKED, np.uint16),
        "gate_up": (capi.TAP_GATE_UP, np.uint16), "y_pairs": (capi.TAP_Y_PAIRS, np.float32),
        "gathered": (capi.TAP_GATHERED, np.uint16),
    }

    def tap(self, name, T):
        tap, dt = self._TAPS[name]
        H, I, E, k = self.H, self.I, self.E, self.k
        shape = {"scores": (T, E), "topk_w": (T, k), "topk_i": (T, k), "offsets": (E + 1,),
                 "sorted": (T * k,), "x_packed": (T * k, H), "gate_up": (T * k, I),
                 "y_pairs": (T * k, H), "gathered": (T, H)}[name]
        out = np.empty(shape, dt)
        self._check(self.lib.gptoss_read_tap(self._ctx, tap, _ptr(out), out.nbytes))
        return out


def launch_count() -> int:
    """kernels launched by the library in this process so far"""
    return int(capi.load().gptoss_launch_count())


def synth_normal_bf16(n, seed, tensor_id, sigma, start=0, device="cuda"):
    """bf16 cuda tensor of the seeded generator (same bits as ``synth.normal_bf16_bits``)."""
    out = torch.empty(n, dtype=torch.bfloat16, device=device)
    rc = capi.load().gptoss_synth_normal_bf16(_ptr(out), n, seed, tensor_id, start, sigma, _stream(None))
    if rc != capi.OK:
        raise GptossError(rc, "gptoss_synth_normal_bf16 failed")
    return out
