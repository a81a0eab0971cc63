// Operator-registry adapter: the reference's launch_cuda(node, mp, ctx, state)
// signature on one side, the trb200 C ABI on the other.
//
//   tr_b200_register_ops() overwrites the launch_cuda entries of
//     CBR_AMP_BWD, CBR_AMP_BWD_FIRST_LAYER      (reference: cbr_op.cpp:1359-1651, 1866-1908)
//     SOFTMAX_CE_AMP_FWD, SOFTMAX_CE_AMP_BWD    (reference: softmax_ce_op.cpp:409-455, 591-627)
//     CBR_AMP_FWD                               (reference: cbr_op.cpp:1013-1250)
//     FC_AMP_FWD, FC_AMP_BWD                    (reference: fc_op.cpp:259-480)
//   and, in g_range_op_table,
//     RANGE_SUM_ALLREDUCE, RANGE_MEAN_ALLREDUCE, RANGE_BN_STATS_ALLREDUCE   (allreduce_op.cpp:37-105)
//     RANGE_GRAD_SCALING                        (grad_scaling_op.cu:15-22)
//   It must run after register_default_ops(), which every compile re-runs
//   (src/task/task_base.cpp:219-220).
//
// Each launcher resolves ids to pointers (ctx.ptr_at), shapes (mp.get_dtensor),
// conv parameters (node.params.cbr()) and streams (ctx.stream), follows the
// reference's event protocol on MultiStreamCaptureState, and makes one C-ABI call.
// A non-zero return becomes TR_DEVICE_ERROR, the reference's error convention.
// Called twice per node like every reference op: once outside capture (warm-up:
// the only call that may grow the workspace) and once inside stream capture.
#ifdef TRB200_WITH_REFERENCE_HEADERS
#include "renaissance/backend/memory_arena.h"
#include "renaissance/core/global_registry.h"
#include "renaissance/backend/device_context.h"
#include "renaissance/backend/op_registry.h"
#include "renaissance/core/tr_exception.h"
#include "renaissance/graph/capture_multi_stream.h"
#include "renaissance/graph/computation_graph.h"
#include "renaissance/graph/memory_plan.h"
#else
#include "tr_shim.h"
#endif

#include "trb200.h"

#ifdef TR_USE_NCCL
#include <nccl.h>
#endif

#include <algorithm>

namespace tr {
namespace {

void check(int rc, const char* op) {
    if (rc != TRB200_OK) TR_DEVICE_ERROR(op << ": " << trb200_last_error() << " (trb200 status " << rc << ")");
}

trb200_conv_desc conv_desc(const DTensor& x, const DTensor& w, const ConvParams& cp) {
    trb200_conv_desc d{};
    d.dtype = TRB200_DTYPE_F16;                       // the reference's AMP tensors are DType::FP16
    d.n = x.n(); d.h = x.h(); d.w = x.w(); d.c = x.c();
    d.k = w.n(); d.r = w.h(); d.s = w.w();            // KRSC stored as (n,h,w,c) = (K,R,S,C)
    d.pad_h = cp.pad_h; d.pad_w = cp.pad_w;
    d.stride_h = cp.stride_h; d.stride_w = cp.stride_w;
    return d;
}

// CBR_AMP_BWD and CBR_AMP_BWD_FIRST_LAYER.
// input_ids:  [0]=dY [1]=W16 [2]=gamma [3]=saved_mean [4]=saved_inv_var [5]=mask [6]=X
// output_ids: [0]=dX (= X's buffer; the first layer's data buffer, not written) [1]=dW16
//             [2]=dgamma [3]=dbeta [4]=conv_output [5]=bn_output (scratch)
void launch_cbr_bwd_common(const GraphNode& node, const MemoryPlan& mp, const DeviceContext& ctx,
                           MultiStreamCaptureState& state, bool first_layer) {
    const ConvParams& cp = node.params.cbr().conv;
    cudaStream_t s_bn = static_cast<cudaStream_t>(ctx.stream(StreamKind::COMP_1));
    cudaStream_t s_wg = static_cast<cudaStream_t>(ctx.stream(StreamKind::COMP_3));
    cudaStream_t s_dg = static_cast<cudaStream_t>(ctx.stream(StreamKind::COMP_2));
    const int i_bn = state.get_or_register(s_bn);
    const int i_wg = state.get_or_register(s_wg);
    const int i_dg = first_layer ? -1 : state.get_or_register(s_dg);

    // wait for the producer of dY if it ran on another stream (cbr_op.cpp:1380-1383)
    const int out_idx = state.output_stream_idx;
    if (out_idx >= 0 && state.streams[out_idx].stream != s_bn)
        cudaStreamWaitEvent(s_bn, state.streams[out_idx].last_done_event, 0);

    const DTensor& dt_x = mp.get_dtensor(node.input_ids[6]);
    const DTensor& dt_w = mp.get_dtensor(node.input_ids[1]);
    trb200_cbr_bwd_args a{};
    a.conv = conv_desc(dt_x, dt_w, cp);
    a.dy = ctx.ptr_at(node.input_ids[0]);
    a.w = ctx.ptr_at(node.input_ids[1]);
    a.gamma = static_cast<const float*>(ctx.ptr_at(node.input_ids[2]));
    a.saved_mean = static_cast<const float*>(ctx.ptr_at(node.input_ids[3]));
    a.saved_inv_std = static_cast<const float*>(ctx.ptr_at(node.input_ids[4]));
    a.mask_bits = ctx.ptr_at(node.input_ids[5]);
    a.x = ctx.ptr_at(node.input_ids[6]);
    a.dx = first_layer ? nullptr : ctx.ptr_at(node.output_ids[0]);
    a.dw = ctx.ptr_at(node.output_ids[1]);
    a.dgamma = static_cast<float*>(ctx.ptr_at(node.output_ids[2]));
    a.dbeta = static_cast<float*>(ctx.ptr_at(node.output_ids[3]));
    a.conv_out = ctx.ptr_at(node.output_ids[4]);
    a.bn_scratch = ctx.ptr_at(node.output_ids[5]);

    // one workspace for the whole block, on COMP_1's slot; grown only in the warm-up call
    const size_t need = trb200_cbr_bwd_workspace_bytes(&a.conv, first_layer ? 1 : 0);
    ctx.ensure_workspace_grow(StreamKind::COMP_1, need);
    a.workspace = ctx.workspace(StreamKind::COMP_1);
    a.workspace_bytes = ctx.workspace_size(StreamKind::COMP_1);
    a.stream_bn = s_bn;
    a.stream_wgrad = s_wg;
    a.stream_dgrad = first_layer ? s_wg : s_dg;
    a.ev_bn = state.streams[i_bn].last_done_event;
    a.ev_wgrad = state.streams[i_wg].last_done_event;
    a.ev_dgrad = first_layer ? nullptr : state.streams[i_dg].last_done_event;
    check(trb200_cbr_bwd(&a), first_layer ? "CBR_AMP_BWD_FIRST_LAYER" : "CBR_AMP_BWD");

    state.streams[i_bn].has_pending_work = true;
    state.streams[i_wg].has_pending_work = true;
    if (!first_layer) state.streams[i_dg].has_pending_work = true;
    state.output_stream_idx = i_bn;      // joined back onto COMP_1 (cbr_op.cpp:1510-1521)
}

void launch_cbr_amp_bwd_b200(const GraphNode& node, const MemoryPlan& mp, const DeviceContext& ctx,
                             MultiStreamCaptureState& state) {
    launch_cbr_bwd_common(node, mp, ctx, state, false);
}

void launch_cbr_amp_bwd_first_layer_b200(const GraphNode& node, const MemoryPlan& mp, const DeviceContext& ctx,
                                         MultiStreamCaptureState& state) {
    launch_cbr_bwd_common(node, mp, ctx, state, true);
}

// SOFTMAX_CE_AMP_FWD
// input_ids:  [0]=logits fp16 [1]=scaling [2]=local_batch_size [3]=labels int32 [4]=label_smoothing
// output_ids: [0]=loss [1]=inv_scaling [2]=pred [3]=probs fp32 [4]=top1 [5]=top5 [6]=loss_partial [7],[8]
void launch_softmax_ce_amp_fwd_b200(const GraphNode& node, const MemoryPlan& mp, const DeviceContext& ctx,
                                    MultiStreamCaptureState& state) {
    cudaStream_t s = static_cast<cudaStream_t>(ctx.stream(StreamKind::COMP_1));
    const int si = state.get_or_register(s);
    state.output_stream_idx = si;
    state.streams[si].has_pending_work = true;
    const DTensor& logits = mp.get_dtensor(node.input_ids[0]);
    const DTensor& probs = mp.get_dtensor(node.output_ids[3]);
    check(trb200_softmax_ce_fwd(ctx.ptr_at(node.input_ids[0]), logits.n_stride_cuda(),
                                static_cast<const int32_t*>(ctx.ptr_at(node.input_ids[3])),
                                static_cast<const float*>(ctx.ptr_at(node.input_ids[4])),
                                static_cast<float*>(ctx.ptr_at(node.output_ids[3])), probs.n_stride_cuda(),
                                static_cast<float*>(ctx.ptr_at(node.output_ids[6])),
                                static_cast<float*>(ctx.ptr_at(node.output_ids[0])),
                                static_cast<float*>(ctx.ptr_at(node.output_ids[1])), logits.n(), logits.c(), s),
          "SOFTMAX_CE_AMP_FWD");
    cudaEventRecord(state.streams[si].last_done_event, s);
}

// SOFTMAX_CE_AMP_BWD
// input_ids:  [0]=d_logits placeholder [1]=probs [2]=inv_scaling [3]=scaling [4]=labels [5]=label_smoothing
// output_ids: [0]=d_logits fp16
void launch_softmax_ce_amp_bwd_b200(const GraphNode& node, const MemoryPlan& mp, const DeviceContext& ctx,
                                    MultiStreamCaptureState& state) {
    cudaStream_t s = static_cast<cudaStream_t>(ctx.stream(StreamKind::COMP_1));
    const int si = state.get_or_register(s);
    state.output_stream_idx = si;
    state.streams[si].has_pending_work = true;
    const DTensor& probs = mp.get_dtensor(node.input_ids[1]);
    const DTensor& dl = mp.get_dtensor(node.output_ids[0]);
    check(trb200_softmax_ce_bwd(static_cast<const float*>(ctx.ptr_at(node.input_ids[1])), probs.n_stride_cuda(),
                                static_cast<const int32_t*>(ctx.ptr_at(node.input_ids[4])),
                                static_cast<const float*>(ctx.ptr_at(node.input_ids[3])),
                                static_cast<const float*>(ctx.ptr_at(node.input_ids[2])),
                                static_cast<const float*>(ctx.ptr_at(node.input_ids[5])),
                                ctx.ptr_at(node.output_ids[0]), dl.n_stride_cuda(), probs.n(), probs.c(), s),
          "SOFTMAX_CE_AMP_BWD");
    cudaEventRecord(state.streams[si].last_done_event, s);
}

// SOFTMAX_CE_AMP_FWD with the backward folded in.  The graph builder is patched so that the forward node also lists
// the d_logits tensor (ce_output) as output [9] and the backward node lists the logits as input [6]
// (build_softmaxce_backward, layer_descriptor_registry.cpp:794-804): one pass then reads each logit once and writes
// d_logits, and the backward node has nothing left to do.  Unpatched graphs keep the two launchers above.
void launch_softmax_ce_amp_fwd_fused_b200(const GraphNode& node, const MemoryPlan& mp, const DeviceContext& ctx,
                                          MultiStreamCaptureState& state) {
    if (node.output_ids.size() < 10) {                  // not patched: the forward node alone
        launch_softmax_ce_amp_fwd_b200(node, mp, ctx, state);
        return;
    }
    cudaStream_t s = static_cast<cudaStream_t>(ctx.stream(StreamKind::COMP_1));
    const int si = state.get_or_register(s);
    state.output_stream_idx = si;
    state.streams[si].has_pending_work = true;
    const DTensor& logits = mp.get_dtensor(node.input_ids[0]);
    const DTensor& dl = mp.get_dtensor(node.output_ids[9]);
    // The probabilities (output [3]) exist only to carry the forward node's result to the backward node: with the two
    // fused nothing reads them, so they are not written and the pass moves 4 bytes per class instead of 12.
    check(trb200_softmax_ce_fused(ctx.ptr_at(node.input_ids[0]), logits.n_stride_cuda(),
                                  static_cast<const int32_t*>(ctx.ptr_at(node.input_ids[3])),
                                  static_cast<const float*>(ctx.ptr_at(node.input_ids[1])),
                                  static_cast<const float*>(ctx.ptr_at(node.input_ids[4])),
                                  nullptr, 0,
                                  ctx.ptr_at(node.output_ids[9]), dl.n_stride_cuda(),
                                  static_cast<float*>(ctx.ptr_at(node.output_ids[6])),
                                  static_cast<float*>(ctx.ptr_at(node.output_ids[0])),
                                  static_cast<float*>(ctx.ptr_at(node.output_ids[1])), logits.n(), logits.c(), s),
          "SOFTMAX_CE_AMP_FWD (fused with its backward)");
    cudaEventRecord(state.streams[si].last_done_event, s);
}

void launch_softmax_ce_amp_bwd_fused_b200(const GraphNode& node, const MemoryPlan& mp, const DeviceContext& ctx,
                                          MultiStreamCaptureState& state) {
    if (node.input_ids.size() < 7) {                    // not patched: compute d_logits from the stored probabilities
        launch_softmax_ce_amp_bwd_b200(node, mp, ctx, state);
        return;
    }
    // patched graph: the forward node has written d_logits already; only keep the stream bookkeeping consistent
    cudaStream_t s = static_cast<cudaStream_t>(ctx.stream(StreamKind::COMP_1));
    const int si = state.get_or_register(s);
    const int out_idx = state.output_stream_idx;
    if (out_idx >= 0 && state.streams[out_idx].stream != s)
        cudaStreamWaitEvent(s, state.streams[out_idx].last_done_event, 0);
    state.output_stream_idx = si;
}

// CBR_AMP_FWD (cbr_op.cpp:1013-1250): conv + batch statistics, bn_finalize, BN apply + ReLU + bit mask.
// input_ids:  [0]=X [1]=W16 [2]=gamma [3]=beta [4]=prev running mean [5]=prev running var
// output_ids: [0]=conv_output [1]=sum [2]=sq_sum [3]=bn_output (its first 2*K floats hold eq_scale then eq_bias,
//             cbr_op.cpp:1105-1108, 1168-1171) [4]=saved_mean [5]=saved_inv_var [6]=relu_output [7]=mask
//             [8]=next running mean [9]=next running var
// Convolution, statistics and finalize run on COMP_1 (two launches), the apply stage on COMP_3 as in the
// reference; the reference's separate finalize hop over COMP_2 has nothing left to do.
void launch_cbr_amp_fwd_b200(const GraphNode& node, const MemoryPlan& mp, const DeviceContext& ctx,
                             MultiStreamCaptureState& state) {
    const CBRParams& cbrp = node.params.cbr();
    cudaStream_t s_conv = static_cast<cudaStream_t>(ctx.stream(StreamKind::COMP_1));
    cudaStream_t s_apply = static_cast<cudaStream_t>(ctx.stream(StreamKind::COMP_3));
    const int i_conv = state.get_or_register(s_conv);
    const int i_apply = state.get_or_register(s_apply);
    const int out_idx = state.output_stream_idx;
    if (out_idx >= 0 && state.streams[out_idx].stream != s_conv)
        cudaStreamWaitEvent(s_conv, state.streams[out_idx].last_done_event, 0);

    const DTensor& dt_x = mp.get_dtensor(node.input_ids[0]);
    const DTensor& dt_w = mp.get_dtensor(node.input_ids[1]);
    const trb200_conv_desc d = conv_desc(dt_x, dt_w, cbrp.conv);
    const int K = d.k;
    float* eq_scale = static_cast<float*>(ctx.ptr_at(node.output_ids[3]));
    float* eq_bias = eq_scale + K;
    float* next_mean = static_cast<float*>(ctx.ptr_at(node.output_ids[8]));
    float* next_var = static_cast<float*>(ctx.ptr_at(node.output_ids[9]));
    const float* prev_mean = static_cast<const float*>(ctx.ptr_at(node.input_ids[4]));
    const float* prev_var = static_cast<const float*>(ctx.ptr_at(node.input_ids[5]));
    // the library updates running statistics in place: start the "next" tensors from the "prev" ones
    if (next_mean != prev_mean) cudaMemcpyAsync(next_mean, prev_mean, sizeof(float) * K, cudaMemcpyDeviceToDevice, s_conv);
    if (next_var != prev_var) cudaMemcpyAsync(next_var, prev_var, sizeof(float) * K, cudaMemcpyDeviceToDevice, s_conv);

    const size_t need = trb200_conv_fprop_bn_stats_workspace_bytes(&d);
    ctx.ensure_workspace_grow(StreamKind::COMP_1, need);
    check(trb200_conv_fprop_bn_stats(&d, ctx.ptr_at(node.input_ids[0]), ctx.ptr_at(node.input_ids[1]),
                                     ctx.ptr_at(node.output_ids[0]),
                                     static_cast<const float*>(ctx.ptr_at(node.input_ids[2])),
                                     static_cast<const float*>(ctx.ptr_at(node.input_ids[3])), cbrp.bn.eps,
                                     cbrp.bn.momentum, static_cast<float*>(ctx.ptr_at(node.output_ids[1])),
                                     static_cast<float*>(ctx.ptr_at(node.output_ids[2])),
                                     static_cast<float*>(ctx.ptr_at(node.output_ids[4])),
                                     static_cast<float*>(ctx.ptr_at(node.output_ids[5])), eq_scale, eq_bias, next_mean,
                                     next_var, ctx.workspace(StreamKind::COMP_1), ctx.workspace_size(StreamKind::COMP_1),
                                     s_conv),
          "CBR_AMP_FWD conv + statistics");
    cudaEventRecord(state.streams[i_conv].last_done_event, s_conv);
    state.streams[i_conv].has_pending_work = true;

    if (s_apply != s_conv) cudaStreamWaitEvent(s_apply, state.streams[i_conv].last_done_event, 0);
    const DTensor& dt_y = mp.get_dtensor(node.output_ids[0]);
    check(trb200_bn_apply_relu_mask(ctx.ptr_at(node.output_ids[0]), eq_scale, eq_bias, ctx.ptr_at(node.output_ids[6]),
                                    ctx.ptr_at(node.output_ids[7]), (int64_t)dt_y.n() * dt_y.h() * dt_y.w(), K, s_apply),
          "CBR_AMP_FWD BN apply + ReLU");
    cudaEventRecord(state.streams[i_apply].last_done_event, s_apply);
    state.streams[i_apply].has_pending_work = true;
    state.output_stream_idx = i_apply;
}

// FC_AMP_FWD (fc_op.cpp:259-347).  input_ids: [0]=x [1]=w16 [2]=bias (fp32); output_ids: [0]=y
void launch_fc_amp_fwd_b200(const GraphNode& node, const MemoryPlan& mp, const DeviceContext& ctx,
                            MultiStreamCaptureState& state) {
    const auto* p = std::get_if<FCParams>(&node.params.data);
    const bool has_bias = p ? p->bias : true;
    const DTensor& dt_x = mp.get_dtensor(node.input_ids[0]);
    const DTensor& dt_w = mp.get_dtensor(node.input_ids[1]);
    cudaStream_t s = static_cast<cudaStream_t>(ctx.stream(StreamKind::COMP_1));
    const int si = state.get_or_register(s);
    const int out_idx = state.output_stream_idx;
    if (out_idx >= 0 && state.streams[out_idx].stream != s)
        cudaStreamWaitEvent(s, state.streams[out_idx].last_done_event, 0);
    state.output_stream_idx = si;
    state.streams[si].has_pending_work = true;
    const int batch = dt_x.n(), in_f = dt_x.h() * dt_x.w() * dt_x.c(), out_f = dt_w.n();
    const size_t need = trb200_fc_amp_workspace_bytes(batch, in_f, out_f);
    ctx.ensure_workspace_grow(StreamKind::COMP_1, need);
    check(trb200_fc_amp_fwd(ctx.ptr_at(node.input_ids[0]), ctx.ptr_at(node.input_ids[1]),
                            has_bias ? static_cast<const float*>(ctx.ptr_at(node.input_ids[2])) : nullptr,
                            ctx.ptr_at(node.output_ids[0]), batch, in_f, out_f, 0, 0.f, 0, 0,
                            ctx.workspace(StreamKind::COMP_1), ctx.workspace_size(StreamKind::COMP_1), s),
          "FC_AMP_FWD");
    cudaEventRecord(state.streams[si].last_done_event, s);
}

// FC_AMP_BWD (fc_op.cpp:349-480).  input_ids: [0]=dy [1]=w16 ... [last]=x; output_ids: [0]=dx [1]=dW (fp32) [2]=db
void launch_fc_amp_bwd_b200(const GraphNode& node, const MemoryPlan& mp, const DeviceContext& ctx,
                            MultiStreamCaptureState& state) {
    const auto* p = std::get_if<FCParams>(&node.params.data);
    const bool has_bias = p ? p->bias : true;
    const int x_idx = static_cast<int>(node.input_ids.size()) - 1;
    const DTensor& dt_dy = mp.get_dtensor(node.input_ids[0]);
    const DTensor& dt_x = mp.get_dtensor(node.input_ids[x_idx]);
    cudaStream_t s = static_cast<cudaStream_t>(ctx.stream(StreamKind::COMP_1));
    const int si = state.get_or_register(s);
    const int out_idx = state.output_stream_idx;
    if (out_idx >= 0 && state.streams[out_idx].stream != s)
        cudaStreamWaitEvent(s, state.streams[out_idx].last_done_event, 0);
    state.output_stream_idx = si;
    state.streams[si].has_pending_work = true;
    const int batch = dt_dy.n(), out_f = dt_dy.c(), in_f = dt_x.h() * dt_x.w() * dt_x.c();
    const size_t need = trb200_fc_amp_workspace_bytes(batch, in_f, out_f);
    ctx.ensure_workspace_grow(StreamKind::COMP_1, need);
    check(trb200_fc_amp_bwd(ctx.ptr_at(node.input_ids[0]), ctx.ptr_at(node.input_ids[1]), ctx.ptr_at(node.input_ids[x_idx]),
                            ctx.ptr_at(node.output_ids[0]), ctx.ptr_at(node.output_ids[1]), 1,
                            has_bias ? static_cast<float*>(ctx.ptr_at(node.output_ids[2])) : nullptr, nullptr, 1.f,
                            batch, in_f, out_f, ctx.workspace(StreamKind::COMP_1), ctx.workspace_size(StreamKind::COMP_1), s),
          "FC_AMP_BWD");
    cudaEventRecord(state.streams[si].last_done_event, s);
}

// RANGE_SUM_ALLREDUCE / RANGE_MEAN_ALLREDUCE / RANGE_BN_STATS_ALLREDUCE (allreduce_op.cpp:37-105): in-place float
// sum over the ranks with NCCL on the UPDATE stream, over each (start region, end region) byte span of the node,
// followed for the mean flavours by the 1/world scale (trb200_scale_f32 = tr_scale_fp32_kernel).  The collective
// stays NCCL's; how many spans a step has, and therefore how much of it overlaps with backward, is the graph
// builder's choice (the reference cuts two, compiler.cpp:1836-1847; spans of 50 MB or more that end at tensor ends, in backward
// order, overlap almost fully).
void launch_allreduce_b200(const GraphNode& node, const MemoryPlan& mp, const DeviceContext& ctx,
                           MultiStreamCaptureState& state) {
    cudaStream_t s = static_cast<cudaStream_t>(ctx.stream(StreamKind::UPDATE));
    const int si = state.get_or_register(s);
    const int out_idx = state.output_stream_idx;
    if (out_idx >= 0 && state.streams[out_idx].stream != s)
        cudaStreamWaitEvent(s, state.streams[out_idx].last_done_event, 0);
    state.output_stream_idx = si;
    state.streams[si].has_pending_work = true;
    const int world = GlobalRegistry::instance().world_size();
    if (world > 1) {
#ifdef TR_USE_NCCL
        const bool mean = node.range_op == RangeOp::RANGE_MEAN_ALLREDUCE || node.range_op == RangeOp::RANGE_BN_STATS_ALLREDUCE;
        for (size_t i = 0; i < node.input_ranges.size() && i < node.output_ranges.size(); ++i) {
            const auto src_b = mp.resolve_region_bounds(static_cast<Region>(node.input_ranges[i].start_region_id),
                                                        static_cast<Region>(node.input_ranges[i].end_region_id));
            const auto dst_b = mp.resolve_region_bounds(static_cast<Region>(node.output_ranges[i].start_region_id),
                                                        static_cast<Region>(node.output_ranges[i].end_region_id));
            if (src_b.second == 0 || dst_b.second == 0) continue;
            void* src = ArenaKeeper::instance().ptr_at(ctx.rank_for_context(), src_b.first);
            void* dst = ArenaKeeper::instance().ptr_at(ctx.rank_for_context(), dst_b.first);
            const size_t count = std::min(src_b.second, dst_b.second) / sizeof(float);
            if (count == 0) continue;
            if (src != dst && cudaMemcpyAsync(dst, src, count * sizeof(float), cudaMemcpyDeviceToDevice, s) != cudaSuccess)
                TR_DEVICE_ERROR("RANGE_ALLREDUCE pre-copy failed");
            const ncclResult_t res = ncclAllReduce(dst, dst, count, ncclFloat32, ncclSum,
                                                   static_cast<ncclComm_t>(ctx.nccl_comm()), s);
            if (res != ncclSuccess) TR_DEVICE_ERROR("ncclAllReduce failed: " << ncclGetErrorString(res));
            if (mean)
                check(trb200_scale_f32(static_cast<float*>(dst), static_cast<int64_t>(count), 1.0f / static_cast<float>(world), s),
                      "RANGE_MEAN_ALLREDUCE scale");
        }
#else
        TR_DEVICE_ERROR("RANGE_ALLREDUCE with " << world << " ranks in a build without TR_USE_NCCL");
#endif
    }
    cudaEventRecord(state.streams[si].last_done_event, s);
}

// RANGE_GRAD_SCALING (grad_scaling_op.cu:15-22; launcher grad_scaling_op.cpp:31-57): input_ids [0]=has_nan flag,
// [1]=scaling, on COMP_1
void launch_grad_scaling_b200(const GraphNode& node, const MemoryPlan&, const DeviceContext& ctx,
                              MultiStreamCaptureState& state) {
    cudaStream_t s = static_cast<cudaStream_t>(ctx.stream(StreamKind::COMP_1));
    const int si = state.get_or_register(s);
    const int out_idx = state.output_stream_idx;
    if (out_idx >= 0 && state.streams[out_idx].stream != s)
        cudaStreamWaitEvent(s, state.streams[out_idx].last_done_event, 0);
    state.output_stream_idx = si;
    state.streams[si].has_pending_work = true;
    if (node.input_ids.size() < 2) TR_DEVICE_ERROR("RANGE_GRAD_SCALING requires 2 input_ids: [has_nan, scaling]");
    check(trb200_grad_scaling(static_cast<int32_t*>(ctx.ptr_at(node.input_ids[0])),
                              static_cast<float*>(ctx.ptr_at(node.input_ids[1])), 0, s),
          "RANGE_GRAD_SCALING");
    cudaEventRecord(state.streams[si].last_done_event, s);
}

}  // namespace
}  // namespace tr

extern "C" void tr_b200_register_ops(void) {
    using namespace tr;
    g_compute_op_table[static_cast<size_t>(ComputeOp::CBR_AMP_BWD)].launch_cuda = launch_cbr_amp_bwd_b200;
    g_compute_op_table[static_cast<size_t>(ComputeOp::CBR_AMP_BWD_FIRST_LAYER)].launch_cuda =
        launch_cbr_amp_bwd_first_layer_b200;
    // the fused pair falls back to the two separate launchers on a graph whose softmax nodes are not patched
    g_compute_op_table[static_cast<size_t>(ComputeOp::SOFTMAX_CE_AMP_FWD)].launch_cuda = launch_softmax_ce_amp_fwd_fused_b200;
    g_compute_op_table[static_cast<size_t>(ComputeOp::SOFTMAX_CE_AMP_BWD)].launch_cuda = launch_softmax_ce_amp_bwd_fused_b200;
    g_compute_op_table[static_cast<size_t>(ComputeOp::CBR_AMP_FWD)].launch_cuda = launch_cbr_amp_fwd_b200;
    g_compute_op_table[static_cast<size_t>(ComputeOp::FC_AMP_FWD)].launch_cuda = launch_fc_amp_fwd_b200;
    g_compute_op_table[static_cast<size_t>(ComputeOp::FC_AMP_BWD)].launch_cuda = launch_fc_amp_bwd_b200;
    g_range_op_table[static_cast<size_t>(RangeOp::RANGE_SUM_ALLREDUCE)].launch_cuda = launch_allreduce_b200;
    g_range_op_table[static_cast<size_t>(RangeOp::RANGE_MEAN_ALLREDUCE)].launch_cuda = launch_allreduce_b200;
    g_range_op_table[static_cast<size_t>(RangeOp::RANGE_BN_STATS_ALLREDUCE)].launch_cuda = launch_allreduce_b200;
    g_range_op_table[static_cast<size_t>(RangeOp::RANGE_GRAD_SCALING)].launch_cuda = launch_grad_scaling_b200;
}
