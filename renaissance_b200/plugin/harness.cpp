// A small stand-in for the reference's SimpleTask + CapturedGraph, enough to drive
// the registered operators the way the reference does (tests only):
//   register ops -> warm-up call per node outside capture (captured_graph.cpp:241-279)
//   -> stream capture of the node list through g_compute_op_table (capture_cuda.cpp:37-176,
//   thread-local capture mode, cross-stream join at the end) -> cudaGraphLaunch.
// C interface (ctypes): handles are opaque pointers, errors come back as -1 with the
// exception text in trbh_last_error().
#include "tr_shim.h"

#include <cstring>
#include <memory>

extern "C" void tr_b200_register_ops(void);

#ifdef TR_USE_NCCL
#include <nccl.h>
#endif

namespace tr {
ComputeOpEntry g_compute_op_table[static_cast<size_t>(ComputeOp::COUNT)];
RangeOpEntry g_range_op_table[static_cast<size_t>(RangeOp::COUNT)];
}

namespace {

struct Harness {
    tr::MemoryPlan mp;
    tr::DeviceContext ctx;
    std::vector<tr::GraphNode> nodes;
    cudaStream_t streams[5] = {};
    cudaGraph_t graph = nullptr;
    cudaGraphExec_t exec = nullptr;
    ~Harness() {
        if (exec) cudaGraphExecDestroy(exec);
        if (graph) cudaGraphDestroy(graph);
        for (auto s : streams)
            if (s) cudaStreamDestroy(s);
    }
};

thread_local std::string g_err;

template <class F>
int guarded(F&& f) {
    try {
        f();
        return 0;
    } catch (const std::exception& e) {
        g_err = e.what();
        return -1;
    }
}

void run_nodes(Harness& h, tr::MultiStreamCaptureState& state) {
    for (const auto& node : h.nodes) {
        if (node.kind == tr::GraphNode::Kind::RANGE) {
            auto& entry = tr::g_range_op_table[static_cast<size_t>(node.range_op)];
            if (!entry.launch_cuda) TR_DEVICE_ERROR("no launch_cuda registered for range op " << static_cast<int>(node.range_op));
            entry.launch_cuda(node, h.mp, h.ctx, state);
        } else {
            auto& entry = tr::g_compute_op_table[static_cast<size_t>(node.compute_op)];
            if (!entry.launch_cuda) TR_DEVICE_ERROR("no launch_cuda registered for op " << static_cast<int>(node.compute_op));
            entry.launch_cuda(node, h.mp, h.ctx, state);
        }
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) TR_DEVICE_ERROR("CUDA error after node: " << cudaGetErrorString(e));
    }
}

}  // namespace

extern "C" {

const char* trbh_last_error(void) { return g_err.c_str(); }

void* trbh_create(void) {
    auto* h = new Harness();
    for (int i = 0; i < 5; ++i) {
        cudaStreamCreateWithFlags(&h->streams[i], cudaStreamNonBlocking);     // device_context.cpp:74-156
        h->ctx.set_stream(static_cast<tr::StreamKind>(i), h->streams[i]);
    }
    tr_b200_register_ops();
    return h;
}

void trbh_destroy(void* hp) { delete static_cast<Harness*>(hp); }

// dtype: 0 fp32, 1 fp16, 2 int8, 3 int32; row_stride 0 = compact
int trbh_add_tensor(void* hp, int id, void* dev_ptr, int n, int h, int w, int c, int dtype, long long row_stride) {
    return guarded([&] {
        auto* H = static_cast<Harness*>(hp);
        tr::DTensor t;
        t.id = id;
        t.shape.dims[0] = n; t.shape.dims[1] = h; t.shape.dims[2] = w; t.shape.dims[3] = c;
        t.dtype = static_cast<tr::DType>(dtype);
        t.row_stride = row_stride;
        H->mp.add(t);
        H->ctx.bind(id, dev_ptr);
    });
}

// op: 1 CBR_AMP_BWD, 2 CBR_AMP_BWD_FIRST_LAYER, 3 SOFTMAX_CE_AMP_FWD, 4 SOFTMAX_CE_AMP_BWD, 5 CBR_AMP_FWD,
// 6 FC_AMP_FWD, 7 FC_AMP_BWD (for the FC ops `out_channels` = out_features and `kernel` != 0 means "has bias")
int trbh_add_node(void* hp, int op, const int* in_ids, int n_in, const int* out_ids, int n_out, int out_channels,
                  int kernel, int stride, int pad) {
    return guarded([&] {
        auto* H = static_cast<Harness*>(hp);
        tr::GraphNode node;
        node.compute_op = static_cast<tr::ComputeOp>(op);
        node.input_ids.assign(in_ids, in_ids + n_in);
        node.output_ids.assign(out_ids, out_ids + n_out);
        if (op == 6 || op == 7) {
            tr::FCParams p;
            p.out_features = out_channels;
            p.bias = kernel != 0;
            node.params = tr::OpParams(p);
        }
        if (op == 1 || op == 2 || op == 5) {
            tr::CBRParams p;
            p.conv.out_channels = out_channels;
            p.conv.kernel_h = p.conv.kernel_w = kernel;
            p.conv.stride_h = p.conv.stride_w = stride;
            p.conv.pad_h = p.conv.pad_w = pad;
            node.params = tr::OpParams(p);
        }
        H->nodes.push_back(std::move(node));
    });
}

// A RANGE node over one byte span of the rank's arena.  range_op: 1 BN_STATS_ALLREDUCE, 2 SUM_ALLREDUCE,
// 3 MEAN_ALLREDUCE (the span is registered as region pair (region, region)); 5 GRAD_SCALING takes ids instead.
int trbh_add_range_node(void* hp, int range_op, int region, unsigned long long offset, unsigned long long size,
                        const int* in_ids, int n_in) {
    return guarded([&] {
        auto* H = static_cast<Harness*>(hp);
        tr::GraphNode node;
        node.kind = tr::GraphNode::Kind::RANGE;
        node.range_op = static_cast<tr::RangeOp>(range_op);
        if (size) {
            H->mp.add_region_span(region, region, offset, size);
            tr::MemRange r;
            r.offset = offset; r.size = size; r.start_region_id = region; r.end_region_id = region;
            node.input_ranges.push_back(r);
            node.output_ranges.push_back(r);
        }
        if (n_in) node.input_ids.assign(in_ids, in_ids + n_in);
        H->nodes.push_back(std::move(node));
    });
}

// the rank's arena base (ArenaKeeper::ptr_at adds a node's byte offset to it) and its place in the job
int trbh_set_rank(void* hp, int rank, int world, void* arena_base) {
    return guarded([&] {
        auto* H = static_cast<Harness*>(hp);
        H->ctx.set_rank(rank);
        tr::GlobalRegistry::instance().set_world_size(world);
        tr::ArenaKeeper::instance().set_base(rank, arena_base);
    });
}

// NCCL communicator of the rank: rank 0 calls trbh_nccl_unique_id (128 bytes out), every rank trbh_nccl_init with it
int trbh_nccl_unique_id(void* out128) {
#ifdef TR_USE_NCCL
    return guarded([&] {
        ncclUniqueId id;
        if (ncclGetUniqueId(&id) != ncclSuccess) TR_DEVICE_ERROR("ncclGetUniqueId failed");
        static_assert(sizeof(id) == 128, "ncclUniqueId is 128 bytes");
        std::memcpy(out128, &id, sizeof(id));
    });
#else
    (void)out128;
    g_err = "built without TR_USE_NCCL";
    return -1;
#endif
}

int trbh_nccl_init(void* hp, int world, int rank, const void* id128) {
#ifdef TR_USE_NCCL
    return guarded([&] {
        auto* H = static_cast<Harness*>(hp);
        ncclUniqueId id;
        std::memcpy(&id, id128, sizeof(id));
        ncclComm_t comm = nullptr;
        const ncclResult_t r = ncclCommInitRank(&comm, world, id, rank);
        if (r != ncclSuccess) TR_DEVICE_ERROR("ncclCommInitRank: " << ncclGetErrorString(r));
        H->ctx.set_nccl_comm(comm);
    });
#else
    (void)hp; (void)world; (void)rank; (void)id128;
    g_err = "built without TR_USE_NCCL";
    return -1;
#endif
}

int trbh_nccl_destroy(void* hp) {
#ifdef TR_USE_NCCL
    return guarded([&] {
        auto* H = static_cast<Harness*>(hp);
        if (H->ctx.nccl_comm()) ncclCommDestroy(static_cast<ncclComm_t>(H->ctx.nccl_comm()));
        H->ctx.set_nccl_comm(nullptr);
    });
#else
    (void)hp;
    return 0;
#endif
}

// the warm-up call of every node, outside capture, followed by a device sync
int trbh_warmup(void* hp) {
    return guarded([&] {
        auto* H = static_cast<Harness*>(hp);
        tr::MultiStreamCaptureState state;
        state.primary_stream = H->streams[1];
        for (int i = 1; i <= 3; ++i) state.get_or_register(H->streams[i]);
        run_nodes(*H, state);
        cudaError_t e = cudaDeviceSynchronize();
        state.cleanup_all_events();
        if (e != cudaSuccess) TR_DEVICE_ERROR("warm-up: " << cudaGetErrorString(e));
    });
}

// capture the node list on COMP_1 as the primary stream
int trbh_capture(void* hp) {
    return guarded([&] {
        auto* H = static_cast<Harness*>(hp);
        tr::MultiStreamCaptureState state;
        cudaStream_t primary = H->streams[1];
        state.primary_stream = primary;
        for (int i = 1; i <= 3; ++i) state.get_or_register(H->streams[i]);
        if (cudaStreamBeginCapture(primary, cudaStreamCaptureModeThreadLocal) != cudaSuccess)
            TR_DEVICE_ERROR("cudaStreamBeginCapture failed");
        try {
            run_nodes(*H, state);
            // finalize_cross_stream_barrier (capture_multi_stream.cpp:108-116)
            for (int i = 0; i < state.num_active; ++i) {
                if (state.streams[i].stream == primary || !state.streams[i].has_pending_work) continue;
                cudaStreamWaitEvent(primary, state.streams[i].last_done_event, 0);
            }
        } catch (...) {
            cudaGraph_t dead = nullptr;
            cudaStreamEndCapture(primary, &dead);
            if (dead) cudaGraphDestroy(dead);
            state.cleanup_all_events();
            throw;
        }
        cudaError_t e = cudaStreamEndCapture(primary, &H->graph);
        state.cleanup_all_events();
        if (e != cudaSuccess) TR_DEVICE_ERROR("cudaStreamEndCapture: " << cudaGetErrorString(e));
        e = cudaGraphInstantiate(&H->exec, H->graph, 0);
        if (e != cudaSuccess) TR_DEVICE_ERROR("cudaGraphInstantiate: " << cudaGetErrorString(e));
    });
}

int trbh_replay(void* hp) {
    return guarded([&] {
        auto* H = static_cast<Harness*>(hp);
        if (!H->exec) TR_DEVICE_ERROR("replay before capture");
        cudaError_t e = cudaGraphLaunch(H->exec, H->streams[1]);
        if (e == cudaSuccess) e = cudaStreamSynchronize(H->streams[1]);
        if (e != cudaSuccess) TR_DEVICE_ERROR("replay: " << cudaGetErrorString(e));
    });
}

size_t trbh_workspace_bytes(void* hp) {
    return static_cast<Harness*>(hp)->ctx.workspace_size(tr::StreamKind::COMP_1);
}

}  // extern "C"
