// Minimal stand-ins for the reference types that cross the operator boundary.
//
// The adapter in b200_ops.cpp is written against the reference's own interface:
// it is meant to be compiled inside the reference tree with
// -DTRB200_WITH_REFERENCE_HEADERS, where these names come from
//   include/renaissance/backend/op_registry.h        ComputeOpEntry, g_compute_op_table
//   include/renaissance/graph/computation_graph.h    GraphNode
//   include/renaissance/graph/op_kind.h              ComputeOp, OpParams, CBRParams, ConvParams
//   include/renaissance/graph/memory_plan.h          MemoryPlan::get_dtensor
//   include/renaissance/tensor/distributed_tensor.h  DTensor
//   include/renaissance/backend/device_context.h     DeviceContext
//   include/renaissance/graph/capture_multi_stream.h MultiStreamCaptureState
//   include/renaissance/core/tr_exception.h          TR_DEVICE_ERROR
//   include/renaissance/core/global_registry.h       GlobalRegistry::world_size
//   include/renaissance/backend/memory_arena.h       ArenaKeeper::ptr_at
//   include/renaissance/graph/shape_id.h             MemRange
// Outside that tree (this repository's tests) the same adapter compiles against
// the declarations below, which carry only the members the adapter touches, with
// the reference's names and meaning.
#pragma once

#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>
#include <sstream>
#include <stdexcept>
#include <string>
#include <unordered_map>
#include <variant>
#include <vector>

namespace tr {

// tr_exception.h:206-271: errors are C++ exceptions, thrown with a streamed message
class TRException : public std::runtime_error {
public:
    using std::runtime_error::runtime_error;
};
class DeviceError : public TRException {
public:
    using TRException::TRException;
};
#define TR_DEVICE_ERROR(msg_stream)                    \
    do {                                               \
        std::ostringstream tr_oss__;                   \
        tr_oss__ << msg_stream;                        \
        throw ::tr::DeviceError(tr_oss__.str());       \
    } while (0)

enum class DType : uint8_t { FP32, FP16, INT8, INT32 };                       // types.h:193
enum class StreamKind : uint8_t { TRANS, COMP_1, COMP_2, COMP_3, UPDATE };    // types.h:217

// op_kind.h: only the operators this plugin replaces keep their names here
enum class ComputeOp : int {
    UNKNOWN = 0,
    CBR_AMP_BWD,
    CBR_AMP_BWD_FIRST_LAYER,
    SOFTMAX_CE_AMP_FWD,
    SOFTMAX_CE_AMP_BWD,
    CBR_AMP_FWD,
    FC_AMP_FWD,
    FC_AMP_BWD,
    COUNT
};

// op_kind.h:335-380: the range operators this plugin replaces
enum class RangeOp : uint16_t {
    UNKNOWN = 0,
    RANGE_BN_STATS_ALLREDUCE,
    RANGE_SUM_ALLREDUCE,
    RANGE_MEAN_ALLREDUCE,
    RANGE_CHECK_NAN,
    RANGE_GRAD_SCALING,
    COUNT
};

enum class Region : uint8_t { FIRST = 0 };                                    // types.h:241-340 (opaque here)

struct MemRange {                                                             // shape_id.h:84-89
    uint64_t offset = 0;
    uint64_t size = 0;
    int32_t start_region_id = -1;
    int32_t end_region_id = -1;
};

struct ConvParams {                                                           // op_kind.h:22-29
    int out_channels = 0;
    int kernel_h = 1, kernel_w = 1;
    int stride_h = 1, stride_w = 1;
    int pad_h = 0, pad_w = 0;
    int dilation_h = 1, dilation_w = 1;
    int groups = 1;
};
struct BNParams {                                                             // op_kind.h:42-52
    float eps = 1e-5f;
    float momentum = 0.1f;
};
struct CBRParams {                                                            // op_kind.h:91-94
    ConvParams conv;
    BNParams bn;
};
struct LossParams {
    float label_smoothing = 0.f;
};
struct FCParams {                                                             // op_kind.h:54-57
    int out_features = 0;
    bool bias = true;
};
struct OpParams {                                                             // op_kind.h:385-448
    std::variant<std::monostate, ConvParams, BNParams, LossParams, CBRParams, FCParams> data;
    OpParams() = default;
    explicit OpParams(CBRParams p) : data(std::move(p)) {}
    explicit OpParams(LossParams p) : data(std::move(p)) {}
    explicit OpParams(FCParams p) : data(std::move(p)) {}
    const CBRParams& cbr() const { return std::get<CBRParams>(data); }
};

struct GraphNode {                                                            // computation_graph.h:38-57
    enum class Kind : uint8_t { COMPUTE, RANGE };
    Kind kind = Kind::COMPUTE;
    union {
        ComputeOp compute_op;
        RangeOp range_op;
    };
    OpParams params;
    std::vector<int32_t> input_ids;
    std::vector<int32_t> output_ids;
    std::vector<MemRange> input_ranges;     // RANGE nodes: byte ranges of the arena, fixed at compile time
    std::vector<MemRange> output_ranges;
    GraphNode() : compute_op(ComputeOp::UNKNOWN) {}
};

struct Shape {
    int32_t dims[4] = {1, 1, 1, 1};
    int32_t n() const { return dims[0]; }
    int32_t h() const { return dims[1]; }
    int32_t w() const { return dims[2]; }
    int32_t c() const { return dims[3]; }
};

struct DTensor {                                                              // distributed_tensor.h:47-445
    int32_t id = -1;
    Shape shape;
    DType dtype = DType::FP16;
    int64_t row_stride = 0;          // elements between consecutive n (padded channel count * w * h)
    int32_t n() const { return shape.n(); }
    int32_t h() const { return shape.h(); }
    int32_t w() const { return shape.w(); }
    int32_t c() const { return shape.c(); }
    int64_t n_stride_cuda() const { return row_stride ? row_stride : (int64_t)h() * w() * c(); }
};

class MemoryPlan {                                                            // memory_plan.h:236-276
public:
    const DTensor& get_dtensor(int32_t id) const {
        auto it = tensors_.find(id);
        if (it == tensors_.end()) TR_DEVICE_ERROR("MemoryPlan: unknown DTensor id " << id);
        return it->second;
    }
    void add(const DTensor& t) { tensors_[t.id] = t; }
    // memory_plan.h:273-274: byte (offset, size) of the span from the start of one region to the end of another
    std::pair<uint64_t, uint64_t> resolve_region_bounds(Region start, Region end) const {
        auto it = regions_.find((static_cast<uint32_t>(start) << 8) | static_cast<uint32_t>(end));
        if (it == regions_.end()) return {0, 0};
        return it->second;
    }
    void add_region_span(int start, int end, uint64_t offset, uint64_t size) {
        regions_[(static_cast<uint32_t>(start) << 8) | static_cast<uint32_t>(end)] = {offset, size};
    }

private:
    std::unordered_map<int32_t, DTensor> tensors_;
    std::unordered_map<uint32_t, std::pair<uint64_t, uint64_t>> regions_;
};

class GlobalRegistry {                                                        // global_registry.h:57-257
public:
    static GlobalRegistry& instance() {
        static GlobalRegistry g;
        return g;
    }
    int world_size() const { return world_size_; }
    void set_world_size(int w) { world_size_ = w; }

private:
    int world_size_ = 1;
};

class ArenaKeeper {                                                           // memory_arena.h:196-276
public:
    static ArenaKeeper& instance() {
        static ArenaKeeper a;
        return a;
    }
    void* ptr_at(int rank, size_t offset) const noexcept {
        return (rank >= 0 && rank < 8 && base_[rank]) ? static_cast<char*>(base_[rank]) + offset : nullptr;
    }
    void set_base(int rank, void* base) {
        if (rank >= 0 && rank < 8) base_[rank] = base;
    }

private:
    void* base_[8] = {};
};

class DeviceContext {                                                         // device_context.h:32-116
public:
    void* ptr_at(int dtensor_id) const noexcept {
        auto it = ptrs_.find(dtensor_id);
        return it == ptrs_.end() ? nullptr : it->second;
    }
    void* stream(StreamKind kind) const { return streams_[static_cast<int>(kind)]; }
    void* workspace(StreamKind kind) const { return ws_[static_cast<int>(kind)].ptr; }
    size_t workspace_size(StreamKind kind) const { return ws_[static_cast<int>(kind)].size; }
    // device_context.cpp:379-428: cudaFree + cudaMalloc when too small; legal only outside capture
    void ensure_workspace_grow(StreamKind kind, size_t req) const {
        WSpace& w = ws_[static_cast<int>(kind)];
        if (req <= w.size) return;
        cudaStreamCaptureStatus st = cudaStreamCaptureStatusNone;
        cudaStreamIsCapturing(static_cast<cudaStream_t>(stream(kind)), &st);
        if (st != cudaStreamCaptureStatusNone)
            TR_DEVICE_ERROR("ensure_workspace_grow(" << req << ") inside stream capture: the warm-up call must size it");
        if (w.ptr) cudaFree(w.ptr);
        if (cudaMalloc(&w.ptr, req) != cudaSuccess) TR_DEVICE_ERROR("workspace cudaMalloc(" << req << ") failed");
        w.size = req;
    }
    void* nccl_comm() const noexcept { return nccl_comm_; }                   // device_context.h:91-92
    void set_nccl_comm(void* comm) noexcept { nccl_comm_ = comm; }
    int rank_for_context() const noexcept { return rank_for_context_; }       // device_context.h:44-45
    void set_rank(int rank) noexcept { rank_for_context_ = rank; }
    // harness side
    void bind(int id, void* p) { ptrs_[id] = p; }
    void set_stream(StreamKind kind, cudaStream_t s) { streams_[static_cast<int>(kind)] = s; }
    ~DeviceContext() {
        for (auto& w : ws_)
            if (w.ptr) cudaFree(w.ptr);
    }

private:
    struct WSpace {
        void* ptr = nullptr;
        size_t size = 0;
    };
    std::unordered_map<int, void*> ptrs_;
    void* streams_[5] = {};
    mutable WSpace ws_[5];
    void* nccl_comm_ = nullptr;
    int rank_for_context_ = 0;
};

struct PerStreamState {                                                       // capture_multi_stream.h:25-29
    cudaStream_t stream = nullptr;
    cudaEvent_t last_done_event = nullptr;
    bool has_pending_work = false;
};

struct MultiStreamCaptureState {                                              // capture_multi_stream.h:31-46
    static constexpr int kMaxActiveStreams = 5;
    PerStreamState streams[kMaxActiveStreams] = {};
    int num_active = 0;
    cudaStream_t primary_stream = nullptr;
    int32_t output_stream_idx = -1;

    int find_stream_index(cudaStream_t s) const noexcept {
        for (int i = 0; i < num_active; ++i)
            if (streams[i].stream == s) return i;
        return -1;
    }
    int get_or_register(cudaStream_t s) {
        int i = find_stream_index(s);
        if (i >= 0) return i;
        if (num_active >= kMaxActiveStreams) TR_DEVICE_ERROR("MultiStreamCaptureState: more than 5 active streams");
        streams[num_active].stream = s;
        if (cudaEventCreateWithFlags(&streams[num_active].last_done_event, cudaEventDisableTiming) != cudaSuccess)
            TR_DEVICE_ERROR("cudaEventCreate failed");
        return num_active++;
    }
    void cleanup_all_events() {
        for (int i = 0; i < num_active; ++i)
            if (streams[i].last_done_event) {
                cudaEventDestroy(streams[i].last_done_event);
                streams[i].last_done_event = nullptr;
            }
    }
};

struct ComputeOpEntry {                                                       // op_registry.h:58-70
    ComputeOp op = ComputeOp::UNKNOWN;
    void (*launch_cuda)(const GraphNode& node, const MemoryPlan& mp, const DeviceContext& ctx,
                        MultiStreamCaptureState& state) = nullptr;
};

struct RangeOpEntry {                                                         // op_registry.h:71-82
    RangeOp op = RangeOp::UNKNOWN;
    void (*launch_cuda)(const GraphNode& node, const MemoryPlan& mp, const DeviceContext& ctx,
                        MultiStreamCaptureState& state) = nullptr;
};

extern ComputeOpEntry g_compute_op_table[];                                   // op_registry.h:84
extern RangeOpEntry g_range_op_table[];                                       // op_registry.h:85

}  // namespace tr
