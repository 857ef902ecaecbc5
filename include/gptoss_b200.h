/*
 * gptoss_b200 — C ABI of the B200-native GPT-OSS MoE FFN block.
 *
 * This is the boundary a C++ host (the replacement for the reference's getp-csrc/getp_run.cpp and
 * src/model.cpp) binds to.  Plain pointers and sizes only; every call returns an int status
 * (GPTOSS_OK == 0), nothing aborts and no exception crosses the boundary — unlike the reference's
 * launchers, which return void and abort through CHECK_HIP (getp-csrc/include/tensor.hpp:20-27).
 *
 * One context per GPU (one host thread or one process per GPU, the reference's threading model,
 * getp-csrc/submit/getp_run_submit.cpp:106-178).  The context owns all scratch, pre-allocated for
 * `max_tokens` like the reference's run state (getp-csrc/submit/alloc_submit.cpp:882-1014); the caller
 * owns the activations `t` and the residual stream `x`.
 *
 * Each entry point names the reference interface it replaces (paths relative to the reference
 * project root).
 */
#ifndef GPTOSS_B200_H
#define GPTOSS_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes ---------------------------------------------------------------------------- */
#define GPTOSS_OK 0
#define GPTOSS_ERR_BAD_ARG 1     /* null pointer, size out of range, unsupported dimension          */
#define GPTOSS_ERR_CUDA 2        /* a CUDA runtime/driver call failed; see gptoss_last_error()       */
#define GPTOSS_ERR_TIMEOUT 3     /* a bounded device-side wait (mbarrier / peer flag) gave up        */
#define GPTOSS_ERR_UNSUPPORTED 4 /* device is not compute capability 10.x                            */
#define GPTOSS_ERR_STATE 5       /* call out of order (e.g. forward before the layer has weights)    */

/* wire format of the cross-GPU combine: the gate-weighted rows always travel to the owner in fp32 and are
 * summed there in fp32; this selects the format in which the owner delivers the summed rows to every rank.
 * F32: the result equals the single-GPU block bit for bit.  BF16: half the delivered bytes; every rank
 * (the owner included) adds the same bf16-rounded sums, so the replicated residual streams stay identical.
 * (The reference sends e5m2 and also ACCUMULATES in it at every hop, parallelism.cpp:53-68.) */
#define GPTOSS_WIRE_F32 0
#define GPTOSS_WIRE_BF16 1

/* Dimensions of the MoE block; the subset of the checkpoint header (run.cpp:25-45) the block uses. */
typedef struct {
  int hidden;         /* hidden_dim        H                      */
  int intermediate;   /* intermediate_dim  I                      */
  int n_experts;      /* n_experts         E   (<= 256)           */
  int top_k;          /* experts_per_token k   (<= 8)             */
  int n_layers;       /* number of layer slots to hold weights for */
  float swiglu_limit; /* swiglu_limit (7.0)                       */
} gptoss_moe_dims;

typedef struct gptoss_ctx gptoss_ctx;

/* ---- life cycle --------------------------------------------------------------------------------
 * Replaces the MoE part of our_init / our_free (getp-csrc/src/alloc.cpp:1035,1192) and of
 * our_init_run_state_* (getp-csrc/submit/alloc_submit.cpp:882-1014).
 * rank/world: this GPU owns experts [rank*E/world, (rank+1)*E/world), the reference's contiguous
 * expert partition (getp-csrc/src/parallelism.cpp:1852-1855).  world == 1: no sharding. */
int gptoss_ctx_create(const gptoss_moe_dims *dims, int device, int rank, int world, int max_tokens,
                      int wire_dtype, gptoss_ctx **out);
int gptoss_ctx_destroy(gptoss_ctx *ctx);
/* Message of the last failing call on this context (never NULL; "" if none). */
const char *gptoss_last_error(const gptoss_ctx *ctx);
/* Synchronises the context's device and reports a sticky device-side error word:
 * GPTOSS_OK, or GPTOSS_ERR_TIMEOUT if any kernel gave up on a bounded wait since the last call. */
int gptoss_ctx_status(gptoss_ctx *ctx);

/* ---- weights -----------------------------------------------------------------------------------
 * Takes one layer's tensors in the flat checkpoint layouts AS THEY ARE (host fp32; run.cpp:66-76,
 * 194-233): router_w [E,H], router_b [E], mlp1_w [E,2I,H] (gate rows even, up rows odd),
 * mlp1_b [E,2I], mlp2_w [E,H,I], mlp2_b [E,H]; converts to bf16 and keeps this rank's experts.
 * Replaces the host transposes + copies of getp-csrc/src/alloc.cpp:77-181 and the expert slicing of
 * getp-csrc/submit/alloc_submit.cpp:555-598,744-832. */
int gptoss_upload_layer(gptoss_ctx *ctx, int layer, const float *router_w, const float *router_b,
                        const float *mlp1_w, const float *mlp1_b, const float *mlp2_w,
                        const float *mlp2_b);
/* Fills one layer with the seeded synthetic tensors (N(0,sigma) rounded to bf16) directly on the
 * device; bit-identical to uploading the host generator's tensors.  No reference counterpart
 * (real checkpoints are loaded through gptoss_upload_layer). */
int gptoss_fill_layer_synthetic(gptoss_ctx *ctx, int layer, uint64_t seed, float sigma);
/* Replaces the router bias of a layer (host fp32 [E]); used for the skewed-routing workload. */
int gptoss_set_router_bias(gptoss_ctx *ctx, int layer, const float *router_b);
/* Reads this rank's experts of one layer back in the checkpoint layouts (host fp32; any pointer may
 * be NULL): router_w [E,H], router_b [E], mlp1_w [E_local,2I,H], mlp1_b [E_local,2I],
 * mlp2_w [E_local,H,I], mlp2_b [E_local,H].  Test/debug aid (the reference has Tensor::from_device,
 * getp-csrc/src/tensor.cpp:207-210). */
int gptoss_download_layer(gptoss_ctx *ctx, int layer, float *router_w, float *router_b, float *mlp1_w,
                          float *mlp1_b, float *mlp2_w, float *mlp2_b);

/* ---- the per-layer operator ----------------------------------------------------------------------
 * x[T,H] (fp32, device, in/out) += MoE(t[T,H]) (bf16, device).  Replaces the sequence
 * getp-csrc/src/model.cpp:300-445 (120B) / :73-132 (20B): router_gemm_v2, topk_softmax_batched,
 * moe_init_buffers_hip, moe_build_offsets_hip, moe_pack_inputs_hip, moe_build_local_ep_data,
 * moe_get_max_rows_per_expert_hip, moe_mlp1_swiglu_fused_hip, moe_mlp2_forward_hip,
 * moe_scatter_aggregate_ep_hip, tensor_quantize_fp8 + ring_reduce_agg_quantize_fp8 +
 * tensor_dequantize_fp8, add_vector_batched.  Asynchronous on `stream` (a cudaStream_t, may be
 * NULL for the default stream); no host round trip inside.  With world > 1 and peers attached the
 * cross-GPU combine runs inside; with world > 1 and no peers use gptoss_moe_forward_partial. */
int gptoss_moe_forward(gptoss_ctx *ctx, int layer, int T, const void *t_dev_bf16, float *x_dev,
                       void *stream);
/* Same with HOST buffers (t: bf16 bits [T,H]; x: fp32 [T,H] in/out): copies in, runs, copies out,
 * synchronises, and returns the device status.  Pinned host memory makes the copies asynchronous. */
int gptoss_moe_forward_host(gptoss_ctx *ctx, int layer, int T, const uint16_t *t_host, float *x_host);
/* The same call in two halves, for a host that feeds batch after batch: submit returns once the uploads, the kernels and
 * the download of the result are queued; wait blocks until the OLDEST submitted call has finished (its x_host then
 * holds the result) and returns its device status.  Two calls may be in flight: while the result of one crosses PCIe
 * towards the host, the next one's activations cross it the other way and its kernels run, so a stream of batches
 * is bound by the slowest of the three (upload, kernels, download) instead of their sum.  A third submit without a
 * wait is refused (GPTOSS_ERR_STATE); the host buffers must stay valid (and pinned, for the overlap) until the wait.
 * Between a submit and its wait the context serves host-buffer calls only.  (The reference keeps its activations on
 * the device, getp-csrc/src/model.cpp:153-489; these entry points exist for hosts that do not.) */
int gptoss_moe_forward_host_submit(gptoss_ctx *ctx, int layer, int T, const uint16_t *t_host, float *x_host);
int gptoss_moe_forward_host_wait(gptoss_ctx *ctx);
/* Expert-parallel partial: partial[T,H] (fp32, device, overwritten) = sum over THIS rank's experts
 * of gate_weight * expert(t) — the tensor the reference all-reduces (rs_now->e_agg,
 * getp-csrc/src/model.cpp:411-423).  The caller reduces it across ranks and adds it to x. */
int gptoss_moe_forward_partial(gptoss_ctx *ctx, int layer, int T, const void *t_dev_bf16,
                               float *partial_dev, void *stream);

/* ---- peer memory for the fused cross-GPU combine -----------------------------------------------------
 * Replaces the all-pairs hipDeviceEnablePeerAccess of warm_up (getp-csrc/getp_run.cpp:41-48) and the event /
 * pthread-barrier hand-shake of ring_reduce_agg_quantize_fp8 (getp-csrc/src/parallelism.cpp:1605-1670).
 * One process (or thread) per GPU: every rank exports a 64-byte handle of its combine buffers, the host
 * exchanges the handles by any means (the tests use torch.distributed), and every rank attaches all of
 * them (rank order).  Afterwards gptoss_moe_forward on world > 1 pushes the gate-weighted expert rows
 * from the down-GEMM epilogue straight into the buffer of the GPU that owns the token (peer stores over
 * NVLink), the owner sums its slice in slot order and stores it to every rank, and every rank adds it to
 * its residual stream.  All ranks must call gptoss_moe_forward the same number of times with the same T.
 * Device-side waits on peers are bounded (2 s) and end as GPTOSS_ERR_TIMEOUT in gptoss_ctx_status.  After such a
 * time-out the context still serves calls that involve no peer (gptoss_moe_forward_partial, the stages, the taps), but
 * the ranks' step counters no longer match: every later call that exchanges with peers returns GPTOSS_ERR_STATE until
 * the contexts of all ranks have been destroyed and created again. */
#define GPTOSS_IPC_HANDLE_BYTES 64
int gptoss_comm_export(gptoss_ctx *ctx, void *handle_out);
int gptoss_comm_attach(gptoss_ctx *ctx, const void *handles /* world x GPTOSS_IPC_HANDLE_BYTES */);
/* Same for contexts that live in ONE process (one host thread per GPU, the reference's model,
 * getp-csrc/submit/getp_run_submit.cpp:176-178): `all` holds the contexts of ranks 0..world-1. */
int gptoss_comm_attach_local(gptoss_ctx *ctx, gptoss_ctx *const *all);
/* Limit of every device-side wait on a peer (default 2000 ms). */
int gptoss_comm_set_timeout_ms(gptoss_ctx *ctx, int ms);
/* The three stages of the fused combine, in the order gptoss_moe_forward runs them after
 * gptoss_moe_route and gptoss_moe_mlp1_swiglu (replace moe_mlp2_forward_hip + moe_scatter_aggregate_ep_hip
 * + ring_reduce_agg_quantize_fp8 + add_vector_batched, getp-csrc/src/model.cpp:384-444):
 *   push_to_owners : down GEMM whose epilogue stores each gate-weighted row into the owner's buffer,
 *                    then raises this rank's "pushed" flag on every rank;
 *   owner_combine  : waits for the "pushed" flags of all ranks, sums the k slots of this rank's token
 *                    slice in slot order, stores the sums to every rank, raises "delivered" everywhere;
 *   add_delta      : waits for the "delivered" flags of all ranks, x += delivered sums. */
/* Shared routing (what gptoss_moe_forward runs in front of those stages once peers are attached): the activations are
 * replicated, so instead of every rank routing every token (the reference: router_gemm_v2 + topk_softmax_batched on
 * the whole batch on all ranks, getp-csrc/src/model.cpp:300-340)
 *   route_local  : this rank routes only ITS token slice (router GEMM, top-k, softmax, block histograms) and stores the
 *                  rows into the routing buffers of every rank, then raises its "routed" flag everywhere;
 *   route_finish : waits for the "routed" flags of all ranks, then counting sort of the whole batch and gather of the
 *                  token rows of this rank's experts (moe_build_offsets_hip + moe_pack_inputs_hip).
 * t_dev_bf16: the replicated activations [T,H] (NULL in the token-sliced form: the context's gathered buffer).  The
 * split-K factor of the router GEMM is derived from T, not from the slice, so a token's scores have the same bits
 * whoever routes it.  Slices are contiguous and a multiple of 8 tokens (gptoss_moe_slice_bounds).  Sharing is OFF unless
 * the environment holds GPTOSS_SHARED_ROUTING=1 when the context is created (then route_local does nothing and
 * route_finish routes the whole batch on this rank): measured, the extra meeting point costs what the smaller router
 * GEMM and top-k save, because the stage is dominated by the scatter/gather that every rank needs anyway. */
int gptoss_moe_route_local(gptoss_ctx *ctx, int layer, int T, const void *t_dev_bf16, void *stream);
int gptoss_moe_route_finish(gptoss_ctx *ctx, int layer, int T, const void *t_dev_bf16, void *stream);
int gptoss_moe_push_to_owners(gptoss_ctx *ctx, int layer, void *stream);
int gptoss_moe_owner_combine(gptoss_ctx *ctx, void *stream);
int gptoss_moe_add_delta(gptoss_ctx *ctx, float *x_dev, void *stream);

/* ---- token-sliced form of the expert-parallel block ------------------------------------------------
 * For callers that keep only a slice of the residual stream on each GPU (data-parallel attention in front
 * of the expert-parallel block): rank r owns tokens [r*S, (r+1)*S) with S = ceil(T/world) rounded up to a multiple of 8.  It replaces, together,
 * ring_all_reduce_tb2_quantize_fp8 + residual_rmsnorm (the all-reduce that re-creates the replicated
 * activations, getp-csrc/src/parallelism.cpp:1195, layer_hip_batch.cpp:95) and the second half of
 * ring_reduce_agg_quantize_fp8 (the all-gather of the reduced sums, parallelism.cpp:1605-1670): the owner
 * keeps the sums, nothing is delivered back.  Results are bit-identical to the replicated form and to one GPU.
 *   slice_bounds   : first token and token count of this rank's slice for a batch of T tokens;
 *   gather_slice   : x_slice += add (if add != NULL); bf16(RMSNorm(x_slice) * norm_w) stored into the gathered
 *                    activation buffer [T,H] of EVERY rank; raises this rank's "gathered" flag everywhere;
 *   sliced_route   : routes this rank's own rows (already in its gathered buffer) and stores the routing rows to
 *                    every rank (route_local); does not wait for anybody;
 *   sliced_push    : waits for the "gathered" and "routed" flags of all ranks, groups the T tokens by expert, gate/up
 *                    GEMM + SwiGLU, down GEMM pushing to the owners, raises "pushed";
 *   sliced_combine : waits for "pushed" of all ranks; x_slice += slot-ordered sum of this rank's tokens;
 *   forward_sliced : sliced_route + sliced_push + sliced_combine.
 * x_slice_dev, add_dev: fp32 [slice count, H] on the device; norm_w_dev: fp32 [H].  Every rank must make the
 * same sequence of these calls; they must not be interleaved with the replicated form within one step. */
int gptoss_moe_slice_bounds(const gptoss_ctx *ctx, int T, int *first, int *count);
/* Device-side rendezvous of the ranks on `stream`, no data: kernels queued after it start only once every rank
 * has reached its own call (bounded wait; a rank that never arrives shows as GPTOSS_ERR_TIMEOUT in gptoss_ctx_status).
 * Every rank must call it the same number of times; it shares its counter with gather_slice.  Measurement aid: a
 * step of per-rank work followed by a rendezvous costs what the expert-parallel step costs without its data exchange. */
int gptoss_comm_rendezvous(gptoss_ctx *ctx, void *stream);
int gptoss_moe_gather_slice(gptoss_ctx *ctx, int T, float *x_slice_dev, const float *add_dev, const float *norm_w_dev,
                            void *stream);
/* gather_rows: like gather_slice for rows that are already normalised: copies this rank's bf16 rows
 * [slice count, H] (device, 16-byte aligned) into the gathered activations of every rank and raises "gathered". */
int gptoss_moe_gather_rows(gptoss_ctx *ctx, int T, const void *t_slice_dev_bf16, void *stream);
int gptoss_moe_sliced_route(gptoss_ctx *ctx, int layer, int T, void *stream);
int gptoss_moe_sliced_push(gptoss_ctx *ctx, int layer, int T, void *stream);
int gptoss_moe_sliced_combine(gptoss_ctx *ctx, float *x_slice_dev, void *stream);
int gptoss_moe_forward_sliced(gptoss_ctx *ctx, int layer, int T, float *x_slice_dev, void *stream);
/* Dispatch form of the token-sliced block: instead of gathering every rank's activations on every rank, each rank
 * routes ITS tokens and sends each token row only to the ranks whose experts the token selected (top-4 of 32 experts
 * on 8 GPUs: 3.0 remote rows per token on average instead of 7), straight into the row's position in the receiver's
 * grouped input.  Together with the push of the expert outputs to the token's owner this is the dispatch / combine
 * pair of an expert-parallel layer, both halves by peer stores from the kernels that produce the rows; it replaces
 * moe_build_local_ep_data + ring_reduce_agg_quantize_fp8 (getp-csrc/src/parallelism.cpp:1848-1873,1605-1670).
 *   dispatch_route : router GEMM + top-k + softmax + block histograms of this rank's rows t_slice [slice count, H]
 *                    (bf16, device, 16-byte aligned), results stored to every rank; raises "routed"; waits for nobody;
 *   dispatch_rows  : waits for "routed" of all ranks; prefix sums and pair-id placement of the whole batch (every rank
 *                    holds the complete, identical grouping); copies each row of t_slice to the grouped input of the
 *                    rank that owns the selected expert; raises "gathered";
 *   dispatch_push  : waits for "gathered" of all ranks; gate/up GEMM + SwiGLU; down GEMM pushing to the owners;
 *   then gptoss_moe_sliced_combine.  forward_dispatch runs all four.
 * With the context's wire format GPTOSS_WIRE_BF16 the pushed rows travel as bf16 (summed in fp32 by the owner); with
 * GPTOSS_WIRE_F32 the result is bit-identical to one GPU.  Same calling rules as the forms above. */
int gptoss_moe_dispatch_route(gptoss_ctx *ctx, int layer, int T, const void *t_slice_dev_bf16, void *stream);
int gptoss_moe_dispatch_rows(gptoss_ctx *ctx, int layer, int T, const void *t_slice_dev_bf16, void *stream);
int gptoss_moe_dispatch_push(gptoss_ctx *ctx, int layer, void *stream);
int gptoss_moe_forward_dispatch(gptoss_ctx *ctx, int layer, int T, const void *t_slice_dev_bf16, float *x_slice_dev,
                                void *stream);
/* The token-sliced block (dispatch form) through HOST buffers (pinned memory recommended): t_host_slice bf16 [slice count, H] and
 * x_host_slice fp32 [slice count, H] hold THIS RANK'S rows of a batch of T tokens; on return x_host_slice holds
 * x + MoE(t) for them.  Per step each GPU moves only its slice over PCIe (the batch crosses the host link once in
 * total, not once per GPU); the other ranks' activations arrive over NVLink.  Synchronous; every rank must call it. */
int gptoss_moe_forward_host_sliced(gptoss_ctx *ctx, int layer, int T, const uint16_t *t_host_slice, float *x_host_slice);
/* Its submit half (gptoss_moe_forward_host_wait is the other): every rank submits the same calls in the same order. */
int gptoss_moe_forward_host_sliced_submit(gptoss_ctx *ctx, int layer, int T, const uint16_t *t_host_slice, float *x_host_slice);

/* ---- stages of the operator (same order as inside gptoss_moe_forward) ------------------------------
 * They work on the context's scratch so that a test can stop after any stage and read the taps. */
/* router_gemm_v2 + topk_softmax_batched + moe_build_offsets_hip + moe_pack_inputs_hip
 * (getp-csrc/src/layer_hip_batch.cpp:1046,1157; getp-csrc/src/kernel.cpp:851,867) */
int gptoss_moe_route(gptoss_ctx *ctx, int layer, int T, const void *t_dev_bf16, void *stream);
/* moe_mlp1_swiglu_fused_hip (getp-csrc/src/kernel.cpp:1033; kernel matrix_core.cpp:1448) */
int gptoss_moe_mlp1_swiglu(gptoss_ctx *ctx, int layer, void *stream);
/* moe_mlp2_forward_hip (getp-csrc/src/kernel.cpp:1061,1094) with the gate weight applied in the
 * epilogue (moe_agg_kernel_120b's multiply, getp-csrc/src/kernel.cpp:764-767) */
int gptoss_moe_mlp2(gptoss_ctx *ctx, int layer, void *stream);
/* moe_scatter_aggregate_ep_hip + add_vector_batched (getp-csrc/src/layer_hip_batch.cpp:1344,856):
 * residual != 0: x += sum of slots;  residual == 0: x = sum of this rank's slots. */
int gptoss_moe_combine(gptoss_ctx *ctx, int T, float *x_dev, int residual, void *stream);

/* ---- stand-alone routing operators on caller-supplied device buffers ------------------------------ */
/* topk_softmax_batched (getp-csrc/src/layer_hip_batch.cpp:1157, kernel :1087): scores [T,E] fp32 ->
 * topk_w [T,k] fp32 (softmax over the selected raw scores), topk_i [T,k] int32, descending, with
 * the reference kernel's tie rule (selection sort with swap, strict '>'). */
int gptoss_topk_softmax(gptoss_ctx *ctx, int T, const float *scores_dev, float *topk_w_dev,
                        int *topk_i_dev, void *stream);
/* moe_build_offsets (getp-csrc/src/kernel.cpp:851, kernel :504): topk_i [T*k] -> offsets [E+1],
 * sorted_pair_ids [T*k] (pair id = token*k + slot), stable within an expert; ids outside [0,E) are
 * skipped and the tail of sorted_pair_ids beyond offsets[E] is left untouched. */
/* It uses the context's routing scratch (block histograms and bases): do not let it run concurrently with a
 * gptoss_moe_forward / gptoss_moe_route of the same context on another stream. */
int gptoss_moe_build_offsets(gptoss_ctx *ctx, int T, const int *topk_i_dev, int *offsets_dev,
                             int *sorted_pair_ids_dev, void *stream);

/* sample_argmax (run.cpp:739-750; GPU: layer_hip_batch.cpp:1542-1583) on device rows: next[b] = index of the FIRST
 * maximum of logits[b, 0..V) (fp32).  A row with no comparable maximum (all -inf / NaN, or NaN in front) gives 0, as
 * the reference's scan does; the result is always inside [0, V). */
int gptoss_argmax_rows(const float *logits_dev, int B, int V, int *next_dev, void *stream);

/* Grouping for callers that must not allocate: same result as gptoss_moe_build_offsets, but it needs no
 * context and calls no cudaMalloc/cudaFree or any other allocating routine.  It has no counterpart in
 * the reference.  It is meant for hosts that hand all device memory to their own pool at start-up (as
 * the reference engine does in our_init), so that a later cudaMalloc would fail or stall, and for code
 * on a serving path where an implicit device synchronisation inside an allocator is not acceptable.
 * The scratch (block histograms and bases) lives in a fixed 1 MiB device array inside the library, held
 * on every GPU that loads it until the process exits.  Limit: ceil(T/8) * n_experts <= 131072 (e.g.
 * T = 8192 with 128 experts); larger batches are rejected with GPTOSS_ERR_BAD_ARG and a message from
 * gptoss_noalloc_last_error().  Works on the CURRENT device.  The first call on each device resolves
 * the array's device address; make that first call outside any stream capture.  All calls share the
 * array, which keeps the previous call's contents (each call overwrites what it reads, nothing needs
 * clearing): two calls whose kernels may overlap on the GPU (different streams) race — serialise them. */
int gptoss_moe_build_offsets_noalloc(int T, int n_experts, int top_k, const int *topk_i_dev,
                                     int *offsets_dev, int *sorted_pair_ids_dev, void *stream);
/* Message of the last failing gptoss_moe_build_offsets_noalloc call on this host thread ("" if none). */
const char *gptoss_noalloc_last_error(void);

/* ---- taps (debug/parity; the reference's DEBUG printDebug, getp-csrc/src/model.cpp:205-450) -------- */
#define GPTOSS_TAP_SCORES 0    /* fp32 [T,E]   router scores incl. bias                            */
#define GPTOSS_TAP_TOPK_W 1    /* fp32 [T,k]   gate weights                                        */
#define GPTOSS_TAP_TOPK_I 2    /* int32 [T,k]  expert ids                                          */
#define GPTOSS_TAP_OFFSETS 3   /* int32 [E+1]  expert_offsets                                      */
#define GPTOSS_TAP_SORTED 4    /* int32 [T*k]  sorted_pair_ids (dispatch form: rows of this rank's experts only) */
#define GPTOSS_TAP_X_PACKED 5  /* bf16 [T*k,H] gathered inputs (rows of this rank's experts only)  */
#define GPTOSS_TAP_GATE_UP 6   /* bf16 [T*k,I] SwiGLU output, rows in sorted order                 */
#define GPTOSS_TAP_Y_PAIRS 7   /* fp32 [T*k,H] gate_weight * expert output, rows by PAIR id        */
#define GPTOSS_TAP_GATHERED 8  /* bf16 [T,H]   token-sliced form: the activations gathered from all ranks */
/* Copies `bytes` from the start of the tap to host memory after synchronising the device. */
int gptoss_read_tap(gptoss_ctx *ctx, int tap, void *host_dst, uint64_t bytes);

/* ---- synthetic data ------------------------------------------------------------------------------
 * dst_dev_bf16[i] = bf16(N(0,sigma)) for stream (seed, tensor_id), elements [start, start+n);
 * the generator is specified in the Python module `synth` and reproduced bit for bit. */
int gptoss_synth_normal_bf16(void *dst_dev_bf16, uint64_t n, uint64_t seed, uint64_t tensor_id,
                             uint64_t start, float sigma, void *stream);

/* ---- whole-model decode step (the callers either side of the MoE block) --------------------------------
 * The checkpoint header (15 four-byte fields, run.cpp:25-45), field for field. */
typedef struct {
  int vocab_size, hidden_dim, n_experts, experts_per_token, intermediate_dim, n_layers, head_dim, n_attn_heads,
      n_kv_heads, seq_len, initial_context_length;
  float rope_theta, rope_scaling_factor;
  int sliding_window;
  float swiglu_limit;
} gptoss_model_config;

typedef struct gptoss_model gptoss_model;

/* One GPU holding the whole model (weights bf16, KV cache bf16 [layer][sequence][kv head][position][head_dim],
 * scratch for max_batch sequences of at most max_seq positions).  Replaces build_transformer + our_init for the
 * single-GPU (20B-style, data-parallel replica) engine: run.cpp:283, getp-csrc/src/alloc.cpp:1035.
 * Limits: head_dim 32 or 64; 1, 2, 4 or 8 query heads per kv head. */
int gptoss_model_create(const gptoss_model_config *cfg, int device, int max_batch, int max_seq, gptoss_model **out);
/* Rank `rank` of a group of `world` GPUs that decode one batch together (the 120B-style engine,
 * forward_gpu_120b_batched, getp-csrc/src/model.cpp:153-489; one model object per GPU, one calling thread or
 * process each).  max_batch is the batch of the whole group.  The sequences are dealt out in contiguous slices
 * (gptoss_model_slice): attention, dense GEMMs, KV cache and residual stream of a sequence live on its rank only, so
 * the attention side needs no all-reduce (the reference's ring_all_reduce_tb2_quantize_fp8, parallelism.cpp:1195,
 * has no counterpart); the experts are sharded by rank (n_experts % world == 0) and each layer exchanges routing
 * rows, token rows and expert outputs over peer memory (dispatch form of the MoE block above).
 * Every rank loads the same checkpoint (or the same synthetic seed) and keeps its share.  Before the first step
 * the ranks' MoE contexts (gptoss_model_moe_ctx) must be attached to one another with gptoss_comm_export /
 * gptoss_comm_attach (processes) or gptoss_comm_attach_local (one process).  A decode must keep the same batch
 * size B on every step (a sequence stays on its rank).  Results are bit-identical to the single-GPU model. */
int gptoss_model_create_ep(const gptoss_model_config *cfg, int device, int rank, int world, int max_batch, int max_seq,
                           gptoss_model **out);
gptoss_ctx *gptoss_model_moe_ctx(gptoss_model *m);
/* First sequence and number of sequences of this rank for a batch of B (everything for a single-GPU model). */
int gptoss_model_slice(const gptoss_model *m, int B, int *first, int *count);
int gptoss_model_destroy(gptoss_model *m);
const char *gptoss_model_last_error(const gptoss_model *m);
/* load_checkpoint (run.cpp:235-281): reads a flat model.bin (header + fp32 tensors in the order of
 * run.cpp:194-233); the header must match the configuration the model was created with. */
int gptoss_model_load_bin(gptoss_model *m, const char *path);
/* Same from a checkpoint image already in host memory — the mapping the reference keeps in
 * Transformer::data (run.cpp:274,279: the header sits in front of the tensors). */
int gptoss_model_load_mem(gptoss_model *m, const void *image, uint64_t bytes);
/* Random-init weights generated on the device (N(0,sigma) rounded to bf16, RMSNorm scales 1.0), for
 * throughput runs of architectures whose fp32 checkpoint would not fit on the host. */
int gptoss_model_fill_synthetic(gptoss_model *m, uint64_t seed, float sigma);
/* One lock-step decode step for B sequences at position pos: host token ids in, greedy next token ids out
 * (forward_gpu_20b_batched, getp-csrc/src/model.cpp:6-151 / include/model.hpp:9; CPU: forward +
 * sample_argmax, run.cpp:501,739).  Prompt tokens are force-fed by the caller, one position per step, as
 * in getp-csrc/submit/getp_run_submit.cpp:60-87.  next_tokens_host may be NULL for a step whose outputs the
 * caller would discard anyway (every sequence still inside its prompt): the KV caches are updated, the
 * final norm, classifier and argmax are skipped.  Synchronous. */
int gptoss_model_step(gptoss_model *m, const int *tokens_host, int pos, int B, int *next_tokens_host);
/* The same step for a batch from which finished sequences have been dropped — the dead-sequence compaction the
 * reference's scheduler lacks (getp-csrc/submit/getp_run_submit.cpp:60-96 keeps stepping a finished sequence until
 * the whole batch has drained).  n live sequences; sequence i keeps the KV-cache row rows_host[i] (in
 * [0, max_batch), distinct) that it has used since position 0, so nothing is moved: every kernel of the step works on
 * n rows and only the cache accesses go through the map.  A sequence's tokens do not depend on which other
 * sequences share its batch, so the survivors continue bit for bit as if nothing had been dropped.  Single-GPU models
 * only (the ranks of a group keep their slices). */
int gptoss_model_step_rows(gptoss_model *m, const int *tokens_host, const int *rows_host, int pos, int n,
                           int *next_tokens_host);
/* The same step for sequences that did not start together — continuous batching, which the reference's scheduler
 * lacks too (getp-csrc/submit/getp_run_submit.cpp:33-96 starts the next batch only when the current one has
 * drained): a finished sequence hands its KV-cache row to a waiting request, which starts at position 0 while its batch
 * mates carry on.  Sequence i holds cache row rows_host[i] (in [0, max_batch), distinct) and is at position
 * pos_host[i] (in [0, max_seq)); only RoPE (run.cpp:545-563) and attention (run.cpp:565-607) depend on the position,
 * and they take it per sequence.  A sequence's tokens are bit for bit those of a lock-step batch at its position,
 * whoever shares the batch.  Single-GPU models only. */
int gptoss_model_step_seqs(gptoss_model *m, const int *tokens_host, const int *rows_host, const int *pos_host, int n,
                           int *next_tokens_host);
/* The phases of gptoss_model_step, which runs begin, then per layer attention / moe_dispatch / moe_push / moe_combine,
 * then end.  In a group, B is the batch of the group and tokens_host / next_tokens_host hold this rank's sequences only.
 * Separate entry points so that one host thread can drive the ranks of a group in turn (each phase for every rank
 * before the next phase: a rank's moe_dispatch waits on the device for every rank's attention phase, its moe_push for
 * every rank's moe_dispatch, its moe_combine for every rank's moe_push).  attention: RMSNorm, QKV GEMM, RoPE + KV
 * store, attention, o-proj GEMM, residual + RMSNorm (group: and the routing of this rank's rows, shared with all).
 * moe_dispatch: group only, grouping of the batch and this rank's rows to the experts' ranks (dispatch form of the MoE
 * block above).  moe_push: the MoE block (group: expert GEMMs on the received rows, outputs pushed to their owners).
 * moe_combine: group only, the owner's slot-ordered sum into its residual rows.  end: final norm, classifier with the
 * argmax fused, synchronises and reports device-side errors. */
int gptoss_model_step_begin(gptoss_model *m, const int *tokens_host, int pos, int B);
int gptoss_model_layer_attention(gptoss_model *m, int layer);
int gptoss_model_layer_moe_dispatch(gptoss_model *m, int layer);
int gptoss_model_layer_moe_push(gptoss_model *m, int layer);
int gptoss_model_layer_moe_combine(gptoss_model *m, int layer);
int gptoss_model_step_end(gptoss_model *m, int *next_tokens_host);
/* Logits (fp32 [vocab]) of one sequence of the last step that produced tokens; debug/parity tap (PRINT_LOGITS,
 * getp_run.cpp:236).  A step keeps no logits (the classifier's epilogue reduces them to the greedy token, as
 * layer_hip_batch.cpp:1465-1712 does for the reference): the row is computed when asked for.  `row` is the index of
 * the sequence in the arrays of that step. */
int gptoss_model_read_logits(gptoss_model *m, int row, float *host_out);

/* Library build info: "gptoss_b200 <version> sm_100a". */
const char *gptoss_version(void);
/* Number of kernels this library has launched in this process so far (all contexts); measurement aid. */
uint64_t gptoss_launch_count(void);

#ifdef __cplusplus
}
#endif
#endif
