// Operator-registry adapter: the reference's launch_cuda(node, mp, ctx, state)
// signature on one side, the trb200 C ABI on the other.
//
//   tr_b200_register_ops() overwrites the launch_cuda entries of
//     CBR_AMP_BWD, CBR_AMP_BWD_FIRST_LAYER      (reference: cbr_op.cpp:1359-1651, 1866-1908)
//     SOFTMAX_CE_AMP_FWD, SOFTMAX_CE_AMP_BWD    (reference: softmax_ce_op.cpp:409-455, 591-627)
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

}  // namespace
}  // namespace tr

extern "C" void tr_b200_register_ops(void) {
    using namespace tr;
    g_compute_op_table[static_cast<size_t>(ComputeOp::CBR_AMP_BWD)].launch_cuda = launch_cbr_amp_bwd_b200;
    g_compute_op_table[static_cast<size_t>(ComputeOp::CBR_AMP_BWD_FIRST_LAYER)].launch_cuda =
        launch_cbr_amp_bwd_first_layer_b200;
    g_compute_op_table[static_cast<size_t>(ComputeOp::SOFTMAX_CE_AMP_FWD)].launch_cuda = launch_softmax_ce_amp_fwd_b200;
    g_compute_op_table[static_cast<size_t>(ComputeOp::SOFTMAX_CE_AMP_BWD)].launch_cuda = launch_softmax_ce_amp_bwd_b200;
}
