// C++ host mirror of the reference's MoE launchers over the gptoss_b200 C ABI.
//
// Same operator names and argument meaning as the reference's host launchers
// (getp-csrc/include/layer_hip_batch.hpp:103-240, getp-csrc/include/kernel.hpp), so the call sites of
// getp-csrc/src/model.cpp:300-445 keep their shape: device buffers in, device buffers out, explicit stream
// last.  Differences: the scratch tensors (sorted_pair_ids, expert_offsets, x_packed, gate_up, tb3) live in
// the context instead of the run state, and errors throw gptoss::Error instead of aborting
// (CHECK_HIP, getp-csrc/include/tensor.hpp:20-27).
#pragma once

#include <stdexcept>
#include <string>

extern "C" {
#include "gptoss_b200.h"
}

namespace gptoss {

struct Error : std::runtime_error {
  int code;
  Error(int c, const std::string &m) : std::runtime_error(m), code(c) {}
};

class MoeLayerOps {
 public:
  // our_init / our_init_run_state_* (MoE part): one instance per GPU thread
  MoeLayerOps(const gptoss_moe_dims &dims, int device, int rank, int world, int max_tokens,
              int wire = GPTOSS_WIRE_F32) {
    int rc = gptoss_ctx_create(&dims, device, rank, world, max_tokens, wire, &ctx_);
    if (rc) throw Error(rc, "gptoss_ctx_create failed");
  }
  ~MoeLayerOps() {
    if (ctx_) gptoss_ctx_destroy(ctx_);
  }
  MoeLayerOps(const MoeLayerOps &) = delete;
  MoeLayerOps &operator=(const MoeLayerOps &) = delete;

  // weights of one layer in the checkpoint layouts (run.cpp:66-76)
  void load_layer(int layer, const float *w_router, const float *b_router, const float *w_mlp1,
                  const float *b_mlp1, const float *w_mlp2, const float *b_mlp2) {
    check(gptoss_upload_layer(ctx_, layer, w_router, b_router, w_mlp1, b_mlp1, w_mlp2, b_mlp2));
  }

  // router_gemm_v2 + topk_softmax_batched + moe_build_offsets_hip + moe_pack_inputs_hip
  void route(int layer, const void *t_bf16, int cur_batch_size, void *stream) {
    check(gptoss_moe_route(ctx_, layer, cur_batch_size, t_bf16, stream));
  }
  // moe_mlp1_swiglu_fused_hip
  void moe_mlp1_swiglu_fused(int layer, void *stream) { check(gptoss_moe_mlp1_swiglu(ctx_, layer, stream)); }
  // moe_mlp2_forward_hip
  void moe_mlp2_forward(int layer, void *stream) { check(gptoss_moe_mlp2(ctx_, layer, stream)); }
  // moe_scatter_aggregate_ep_hip (+ add_vector_batched when add_residual)
  void moe_scatter_aggregate(float *x_or_e_agg, int cur_batch_size, bool add_residual, void *stream) {
    check(gptoss_moe_combine(ctx_, cur_batch_size, x_or_e_agg, add_residual ? 1 : 0, stream));
  }
  // the whole block: x += MoE(t)   (getp-csrc/src/model.cpp:300-445)
  void forward(int layer, const void *t_bf16, float *x, int cur_batch_size, void *stream) {
    check(gptoss_moe_forward(ctx_, layer, cur_batch_size, t_bf16, x, stream));
  }
  // expert-parallel partial (rs_now->e_agg before the all-reduce, getp-csrc/src/model.cpp:411-421)
  void forward_partial(int layer, const void *t_bf16, float *e_agg, int cur_batch_size, void *stream) {
    check(gptoss_moe_forward_partial(ctx_, layer, cur_batch_size, t_bf16, e_agg, stream));
  }
  // stand-alone operators on caller buffers
  void topk_softmax_batched(const float *router_score, float *topk_v, int *topk_i, int cur_batch_size,
                            void *stream) {
    check(gptoss_topk_softmax(ctx_, cur_batch_size, router_score, topk_v, topk_i, stream));
  }
  void moe_build_offsets(const int *topk_i, int *sorted_pair_ids, int *expert_offsets, int cur_batch_size,
                         void *stream) {
    check(gptoss_moe_build_offsets(ctx_, cur_batch_size, topk_i, expert_offsets, sorted_pair_ids, stream));
  }
  // ---- peers (one MoeLayerOps per GPU thread of the same process, rank order) -----------------------------------
  // replaces the hipDeviceEnablePeerAccess setup of the reference's ring (getp-csrc/src/parallelism.cpp)
  static void attach_local(MoeLayerOps *const *ranks, int world) {
    gptoss_ctx *ctxs[16] = {};
    for (int r = 0; r < world && r < 16; ++r) ctxs[r] = ranks[r]->ctx_;
    for (int r = 0; r < world; ++r) ranks[r]->check(gptoss_comm_attach_local(ranks[r]->ctx_, ctxs));
  }
  // router_gemm_v2 + topk_softmax_batched shared between the GPUs: each routes its own token slice and stores the rows
  // to all (route_local), then moe_build_offsets_hip + moe_pack_inputs_hip on the whole batch (route_finish)
  void route_local(int layer, const void *t_bf16, int cur_batch_size, void *stream) {
    check(gptoss_moe_route_local(ctx_, layer, cur_batch_size, t_bf16, stream));
  }
  void route_finish(int layer, const void *t_bf16, int cur_batch_size, void *stream) {
    check(gptoss_moe_route_finish(ctx_, layer, cur_batch_size, t_bf16, stream));
  }
  // ring_reduce_agg_quantize_fp8 + add_vector_batched, fused with moe_mlp2_forward_hip + moe_scatter_aggregate_ep_hip:
  // the three stages behind forward() once peers are attached
  void moe_mlp2_push_to_owners(int layer, void *stream) { check(gptoss_moe_push_to_owners(ctx_, layer, stream)); }
  void owner_combine(void *stream) { check(gptoss_moe_owner_combine(ctx_, stream)); }
  void add_delivered(float *x, void *stream) { check(gptoss_moe_add_delta(ctx_, x, stream)); }
  // token-sliced form: residual_rmsnorm (layer_hip_batch.cpp:95) of this rank's rows + the all-gather that replaces
  // ring_all_reduce_tb2_quantize_fp8 (parallelism.cpp:1195); then the block on the gathered rows, sums kept by the owner
  void residual_rmsnorm_gather(float *x_slice, const float *add, const float *norm_w, int cur_batch_size, void *stream) {
    check(gptoss_moe_gather_slice(ctx_, cur_batch_size, x_slice, add, norm_w, stream));
  }
  void forward_sliced(int layer, float *x_slice, int cur_batch_size, void *stream) {
    check(gptoss_moe_forward_sliced(ctx_, layer, cur_batch_size, x_slice, stream));
  }
  // dispatch form of the token-sliced block: this rank routes ITS rows (router_gemm_v2 + topk_softmax_batched on the
  // slice), every rank groups the whole batch (moe_build_offsets_hip), each row goes only to the GPUs whose experts it
  // selected (what moe_pack_inputs_hip + moe_build_local_ep_data copy locally), then the expert GEMMs with the rows
  // pushed back to the token's GPU; moe_sliced_combine adds the slot-ordered sums to this rank's residual rows
  void dispatch_route(int layer, const void *t_slice_bf16, int cur_batch_size, void *stream) {
    check(gptoss_moe_dispatch_route(ctx_, layer, cur_batch_size, t_slice_bf16, stream));
  }
  void dispatch_rows(int layer, const void *t_slice_bf16, int cur_batch_size, void *stream) {
    check(gptoss_moe_dispatch_rows(ctx_, layer, cur_batch_size, t_slice_bf16, stream));
  }
  void dispatch_push(int layer, void *stream) { check(gptoss_moe_dispatch_push(ctx_, layer, stream)); }
  void moe_sliced_combine(float *x_slice, void *stream) { check(gptoss_moe_sliced_combine(ctx_, x_slice, stream)); }
  void forward_dispatch(int layer, const void *t_slice_bf16, float *x_slice, int cur_batch_size, void *stream) {
    check(gptoss_moe_forward_dispatch(ctx_, layer, cur_batch_size, t_slice_bf16, x_slice, stream));
  }
  void slice_bounds(int cur_batch_size, int *first, int *count) const {
    gptoss_moe_slice_bounds(ctx_, cur_batch_size, first, count);
  }
  // synchronises and reports a device-side time-out, if any
  void check_device() { check(gptoss_ctx_status(ctx_)); }
  gptoss_ctx *raw() { return ctx_; }

 private:
  void check(int rc) {
    if (rc) throw Error(rc, gptoss_last_error(ctx_));
  }
  gptoss_ctx *ctx_ = nullptr;
};

}  // namespace gptoss
