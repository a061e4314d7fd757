// The expert-parallel MoE FFN step as host C++ over this library's own entry
// points: one call enqueues, on the caller's stream (and a second one for two
// pieces that can run beside it) and with no host readback,
//   add_rms_norm_dynamic_quant -> route plan -> count all-gather -> address
//   tables -> dispatch (rows stored straight into the owning rank's
//   expert-major buffer, peer memory when that rank is another GPU) ->
//   barrier -> grouped_matmul_swiglu_quant -> int8 down projection whose
//   epilogue stores every row where its home rank's combine reads it ->
//   barrier -> combine (MoeFinalizeRouting's weighted sum).
// The only collectives are the all-gather of the per-expert counts and two
// one-word all-reduces used as stream-ordered barriers; they run on an NCCL
// communicator this file creates.  NCCL is not a link-time dependency: its
// entry points are looked up in the process (a torch process has libnccl
// loaded already) the first time a communicator is asked for, and every
// function here that needs it reports W8A8_ERR_UNSUPPORTED when it is absent.
// Peer memory is only ever written with plain stores by the kernels; nothing
// here reads another GPU's memory.
#include <dlfcn.h>

#include <cstring>
#include <mutex>

#include "common.cuh"

namespace w8a8 {

// ---------------------------------------------------------------------------
// NCCL, resolved at run time.  Only the handful of calls the step needs; the
// types are spelled out so that no NCCL header is needed to build the library
// (ncclUniqueId is 128 opaque bytes; the enumerators are NCCL's public ones).
// ---------------------------------------------------------------------------
struct NcclUniqueId {
    char bytes[128];
};
using NcclComm = void*;
constexpr int NCCL_INT32 = 2;  // ncclInt32
constexpr int NCCL_INT64 = 4;  // ncclInt64
constexpr int NCCL_SUM = 0;    // ncclSum

struct NcclApi {
    int (*get_unique_id)(NcclUniqueId*) = nullptr;
    int (*comm_init_rank)(NcclComm*, int, NcclUniqueId, int) = nullptr;
    int (*comm_destroy)(NcclComm) = nullptr;
    int (*all_gather)(const void*, void*, size_t, int, NcclComm, cudaStream_t) = nullptr;
    int (*all_reduce)(const void*, void*, size_t, int, int, NcclComm, cudaStream_t) = nullptr;
    bool ok = false;
};

static const NcclApi& nccl()
{
    static NcclApi api;
    static std::once_flag once;
    std::call_once(once, [] {
        void* h = nullptr;
        for (const char* name : {"libnccl.so.2", "libnccl.so"}) {
            h = dlopen(name, RTLD_NOW | RTLD_GLOBAL);
            if (h != nullptr) {
                break;
            }
        }
        if (h == nullptr) {
            return;
        }
        api.get_unique_id = reinterpret_cast<decltype(api.get_unique_id)>(dlsym(h, "ncclGetUniqueId"));
        api.comm_init_rank = reinterpret_cast<decltype(api.comm_init_rank)>(dlsym(h, "ncclCommInitRank"));
        api.comm_destroy = reinterpret_cast<decltype(api.comm_destroy)>(dlsym(h, "ncclCommDestroy"));
        api.all_gather = reinterpret_cast<decltype(api.all_gather)>(dlsym(h, "ncclAllGather"));
        api.all_reduce = reinterpret_cast<decltype(api.all_reduce)>(dlsym(h, "ncclAllReduce"));
        api.ok = api.get_unique_id && api.comm_init_rank && api.comm_destroy && api.all_gather && api.all_reduce;
    });
    return api;
}

}  // namespace w8a8

using namespace w8a8;

extern "C" int w8a8_ep_unique_id(void* id128)
{
    if (id128 == nullptr) {
        return W8A8_ERR_INVALID;
    }
    if (!nccl().ok) {
        return W8A8_ERR_UNSUPPORTED;
    }
    NcclUniqueId id;
    if (nccl().get_unique_id(&id) != 0) {
        return W8A8_ERR_CUDA;
    }
    std::memcpy(id128, id.bytes, sizeof(id.bytes));
    return W8A8_OK;
}

extern "C" int w8a8_ep_comm_create(const void* id128, int world, int rank, void** comm)
{
    if (id128 == nullptr || comm == nullptr || world < 1 || rank < 0 || rank >= world) {
        return W8A8_ERR_INVALID;
    }
    if (!nccl().ok) {
        return W8A8_ERR_UNSUPPORTED;
    }
    NcclUniqueId id;
    std::memcpy(id.bytes, id128, sizeof(id.bytes));
    NcclComm c = nullptr;
    if (nccl().comm_init_rank(&c, world, id, rank) != 0 || c == nullptr) {
        return W8A8_ERR_CUDA;
    }
    *comm = c;
    return W8A8_OK;
}

extern "C" int w8a8_ep_comm_destroy(void* comm)
{
    if (comm == nullptr) {
        return W8A8_OK;
    }
    if (!nccl().ok) {
        return W8A8_ERR_UNSUPPORTED;
    }
    return nccl().comm_destroy(comm) == 0 ? W8A8_OK : W8A8_ERR_CUDA;
}

// ---------------------------------------------------------------------------
// workspace of one step (device memory, caller-owned)
// ---------------------------------------------------------------------------
namespace {

struct StepBuffers {
    int32_t* status;      // [4]: [0] receive-buffer overflow (sticky), [1] barrier token
    int8_t* xq;           // [T, hidden]
    float* xs;            // [T]
    int64_t* count;       // [E]
    int64_t* cumsum;      // [E]
    int64_t* pos;         // [T * topk]
    void* plan_ws;
    size_t plan_ws_bytes;
    int64_t* gathered;    // [P, E]
    uint64_t* row_dst;    // [E]
    uint64_t* scale_dst;  // [E]
    int64_t* my_base;     // [E]
    int64_t* group_list;  // [E / P]
    int64_t* seg_first;   // [(E / P) * P + 1]
    uint64_t* seg_ptr;    // [(E / P) * P]
    int8_t* h;            // [cap, inter]
    float* hs;            // [cap]
    uint64_t* out_ptrs;   // [cap]
    void* mm_ws;
    size_t mm_ws_bytes;
    size_t total;
};

size_t up256(size_t v) { return (v + 255) / 256 * 256; }

StepBuffers carve_step(void* base, int64_t T, int64_t topk, int64_t hidden, int64_t inter, int64_t E, int64_t P,
                       int64_t cap)
{
    StepBuffers b{};
    uint8_t* p = static_cast<uint8_t*>(base);
    size_t off = 0;
    auto take = [&](size_t bytes) {
        uint8_t* r = p + off;
        off += up256(bytes);
        return r;
    };
    const int64_t e_local = E / P, nseg = e_local * P;
    b.status = reinterpret_cast<int32_t*>(take(4 * sizeof(int32_t)));
    b.xq = reinterpret_cast<int8_t*>(take(static_cast<size_t>(T) * hidden));
    b.xs = reinterpret_cast<float*>(take(static_cast<size_t>(T) * 4));
    b.count = reinterpret_cast<int64_t*>(take(static_cast<size_t>(E) * 8));
    b.cumsum = reinterpret_cast<int64_t*>(take(static_cast<size_t>(E) * 8));
    b.pos = reinterpret_cast<int64_t*>(take(static_cast<size_t>(T) * topk * 8));
    b.plan_ws_bytes = w8a8_route_plan_workspace_size(T, topk, E);
    b.plan_ws = take(b.plan_ws_bytes);
    b.gathered = reinterpret_cast<int64_t*>(take(static_cast<size_t>(P) * E * 8));
    b.row_dst = reinterpret_cast<uint64_t*>(take(static_cast<size_t>(E) * 8));
    b.scale_dst = reinterpret_cast<uint64_t*>(take(static_cast<size_t>(E) * 8));
    b.my_base = reinterpret_cast<int64_t*>(take(static_cast<size_t>(E) * 8));
    b.group_list = reinterpret_cast<int64_t*>(take(static_cast<size_t>(e_local) * 8));
    b.seg_first = reinterpret_cast<int64_t*>(take(static_cast<size_t>(nseg + 1) * 8));
    b.seg_ptr = reinterpret_cast<uint64_t*>(take(static_cast<size_t>(nseg) * 8));
    b.h = reinterpret_cast<int8_t*>(take(static_cast<size_t>(cap) * inter));
    b.hs = reinterpret_cast<float*>(take(static_cast<size_t>(cap) * 4));
    b.out_ptrs = reinterpret_cast<uint64_t*>(take(static_cast<size_t>(cap) * 8));
    const size_t up = w8a8_grouped_matmul_swiglu_quant_workspace_size(cap, hidden, 2 * inter, e_local);
    const size_t down = w8a8_grouped_matmul_workspace_size(cap, hidden, inter, e_local);
    b.mm_ws_bytes = up > down ? up : down;
    b.mm_ws = take(b.mm_ws_bytes);
    b.total = off;
    return b;
}

bool step_shape_ok(const W8A8MoeFfnStep* s)
{
    return s != nullptr && s->world >= 1 && s->rank >= 0 && s->rank < s->world && s->num_experts >= s->world &&
           s->num_experts % s->world == 0 && s->topk >= 1 && s->tokens >= 0 && s->hidden > 0 && s->inter > 0 &&
           s->cap_rows > 0 && (s->dtype == W8A8_DT_F16 || s->dtype == W8A8_DT_BF16);
}

}  // namespace

extern "C" size_t w8a8_moe_ffn_step_workspace_size(const W8A8MoeFfnStep* s)
{
    if (!step_shape_ok(s)) {
        return 0;
    }
    return carve_step(nullptr, s->tokens, s->topk, s->hidden, s->inter, s->num_experts, s->world, s->cap_rows).total;
}

// one stream-ordered barrier across the ranks: every kernel enqueued before it on every rank has finished before
// anything enqueued after it on any rank starts
static int step_barrier(const W8A8MoeFfnStep* s, int32_t* token, cudaStream_t st)
{
    if (s->world == 1) {
        return W8A8_OK;
    }
    return nccl().all_reduce(token, token, 1, NCCL_INT32, NCCL_SUM, s->comm, st) == 0 ? W8A8_OK : W8A8_ERR_CUDA;
}

// A second stream per device for the two pieces of the step that depend on nothing the main stream is busy with
// (the normalisation + quantisation of the tokens beside the routing tables, and the row-pointer expansion beside
// the up projection), with the events that fork it from and join it to the caller's stream.  Made on first use,
// kept for the life of the process.  Fork and join are event waits, so a stream capture of the step follows
// both streams.
struct SideStream {
    cudaStream_t stream = nullptr;
    cudaEvent_t fork[2] = {nullptr, nullptr};
    cudaEvent_t join[2] = {nullptr, nullptr};
    bool ok = false;
};

static SideStream* side_stream()
{
    constexpr int MAX_DEVICES = 64;
    static SideStream streams[MAX_DEVICES];
    static std::mutex lock;
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) {
        return nullptr;
    }
    std::lock_guard<std::mutex> guard(lock);
    SideStream& s = streams[dev];
    if (!s.ok) {
        bool good = cudaStreamCreateWithFlags(&s.stream, cudaStreamNonBlocking) == cudaSuccess;
        for (int i = 0; i < 2 && good; ++i) {
            good = cudaEventCreateWithFlags(&s.fork[i], cudaEventDisableTiming) == cudaSuccess &&
                   cudaEventCreateWithFlags(&s.join[i], cudaEventDisableTiming) == cudaSuccess;
        }
        if (!good) {
            return nullptr;
        }
        s.ok = true;
    }
    return &s;
}

extern "C" int w8a8_moe_ffn_step(const W8A8MoeFfnStep* s, const void* x, const void* residual, const void* gamma,
                                 float epsilon, const int32_t* expert_idx, const float* probs, void* out, void* x_out,
                                 void* stream)
{
    if (!step_shape_ok(s)) {
        return W8A8_ERR_INVALID;
    }
    if (s->tokens == 0) {
        // the collectives still have to be entered by every rank; an empty rank is not supported by this entry point
        return s->world == 1 ? W8A8_OK : W8A8_ERR_UNSUPPORTED;
    }
    if (x == nullptr || residual == nullptr || gamma == nullptr || expert_idx == nullptr || probs == nullptr ||
        out == nullptr || x_out == nullptr || s->peer_base == nullptr || s->local_base == nullptr ||
        s->w_up == nullptr || s->s_up == nullptr || s->w_down == nullptr || s->s_down == nullptr) {
        return W8A8_ERR_INVALID;
    }
    if (s->world > 1 && (s->comm == nullptr || !nccl().ok)) {
        return s->comm == nullptr ? W8A8_ERR_INVALID : W8A8_ERR_UNSUPPORTED;
    }
    const int64_t T = s->tokens, topk = s->topk, hidden = s->hidden, inter = s->inter, E = s->num_experts;
    const int64_t P = s->world, e_local = E / P, nseg = e_local * P, cap = s->cap_rows;
    if (T * topk > s->home_rows) {
        return W8A8_ERR_LIMIT;  // the return buffer holds home_rows rows
    }
    const StepBuffers b = carve_step(s->workspace, T, topk, hidden, inter, E, P, cap);
    if (s->workspace == nullptr || s->workspace_bytes < b.total) {
        return W8A8_ERR_WORKSPACE;
    }
    if (!is_aligned(s->workspace, 256)) {
        return W8A8_ERR_ALIGN;
    }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int64_t elem = 2;
    uint8_t* local = static_cast<uint8_t*>(s->local_base);
    int8_t* xe = reinterpret_cast<int8_t*>(local + s->off_x);
    float* xe_scale = reinterpret_cast<float*>(local + s->off_s);
    void* back = local + s->off_back;

    SideStream* side = side_stream();
    if (side == nullptr) {
        return W8A8_ERR_CUDA;
    }
    // the tokens are normalised and quantised on the second stream while this one plans the routes, exchanges the
    // counts and builds the address tables (small kernels that wait on latency, not on bandwidth)
    if (cudaEventRecord(side->fork[0], st) != cudaSuccess ||
        cudaStreamWaitEvent(side->stream, side->fork[0], 0) != cudaSuccess) {
        return W8A8_ERR_CUDA;
    }
    int rc = w8a8_add_rms_norm_dynamic_quant(x, residual, gamma, b.xq, x_out, b.xs, T, hidden, epsilon, s->dtype, 0,
                                             side->stream);
    if (rc != W8A8_OK) {
        return rc;
    }
    if (cudaEventRecord(side->join[0], side->stream) != cudaSuccess) {
        return W8A8_ERR_CUDA;
    }
    rc = w8a8_route_plan(expert_idx, T, topk, E, b.count, b.cumsum, b.pos, b.plan_ws, b.plan_ws_bytes, st);
    if (rc != W8A8_OK) {
        return rc;
    }
    // every rank learns every rank's per-expert counts; they stay on the device
    if (P > 1) {
        if (nccl().all_gather(b.count, b.gathered, static_cast<size_t>(E), NCCL_INT64, s->comm, st) != 0) {
            return W8A8_ERR_CUDA;
        }
    } else if (cudaMemcpyAsync(b.gathered, b.count, static_cast<size_t>(E) * 8, cudaMemcpyDeviceToDevice, st) !=
               cudaSuccess) {
        return W8A8_ERR_CUDA;
    }
    rc = w8a8_ep_tables(b.gathered, P, E, s->rank, s->peer_base, s->off_x, s->off_s, s->off_back, hidden, hidden * elem,
                        cap, b.row_dst, b.scale_dst, b.my_base, b.group_list, b.seg_first, b.seg_ptr, b.status, st);
    if (rc != W8A8_OK) {
        return rc;
    }
    // the tables are complete: the second stream expands them into one output address per expanded row while this
    // one dispatches and runs the up projection
    if (cudaEventRecord(side->fork[1], st) != cudaSuccess ||
        cudaStreamWaitEvent(side->stream, side->fork[1], 0) != cudaSuccess) {
        return W8A8_ERR_CUDA;
    }
    rc = w8a8_expand_row_pointers(b.seg_first, b.seg_ptr, nseg, cap, hidden * elem, b.out_ptrs, side->stream);
    if (rc != W8A8_OK) {
        return rc;
    }
    if (cudaEventRecord(side->join[1], side->stream) != cudaSuccess ||
        cudaStreamWaitEvent(st, side->join[0], 0) != cudaSuccess) {  // the quantised tokens are ready
        return W8A8_ERR_CUDA;
    }
    // No barrier before the stores: this rank's all-gather has completed, so every other rank's stream has reached
    // its own all-gather of this step, which it enqueued after everything that read its buffers in the step before.
    rc = w8a8_dispatch_rows(b.xq, b.xs, expert_idx, b.pos, b.row_dst, b.scale_dst, b.my_base, T, topk, hidden, st);
    if (rc != W8A8_OK) {
        return rc;
    }
    rc = step_barrier(s, b.status + 1, st);  // every rank's rows have landed
    if (rc != W8A8_OK) {
        return rc;
    }
    rc = w8a8_grouped_matmul_swiglu_quant(xe, s->w_up, s->s_up, xe_scale, b.h, b.hs, cap, hidden, 2 * inter, e_local,
                                          b.group_list, 2, W8A8_W_KN, 0, b.mm_ws, b.mm_ws_bytes, st);
    if (rc != W8A8_OK) {
        return rc;
    }
    if (cudaStreamWaitEvent(st, side->join[1], 0) != cudaSuccess) {  // the output addresses are ready
        return W8A8_ERR_CUDA;
    }
    rc = w8a8_grouped_matmul_to_rows(b.h, s->w_down, nullptr, b.out_ptrs, b.hs, s->s_down, cap, hidden, inter, e_local,
                                     b.group_list, 2, W8A8_DT_I8, W8A8_DT_F32, s->dtype, W8A8_W_KN, b.mm_ws,
                                     b.mm_ws_bytes, st);
    if (rc != W8A8_OK) {
        return rc;
    }
    rc = step_barrier(s, b.status + 1, st);  // every rank's output rows have landed at home
    if (rc != W8A8_OK) {
        return rc;
    }
    return w8a8_combine(back, probs, b.pos, out, T, topk, hidden, s->dtype, st);
}

extern "C" int w8a8_moe_ffn_step_status(const W8A8MoeFfnStep* s, void* stream)
{
    if (!step_shape_ok(s) || s->workspace == nullptr) {
        return W8A8_ERR_INVALID;
    }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    int32_t v = 0;
    int32_t* flag = static_cast<int32_t*>(s->workspace);  // StepBuffers::status[0]
    if (cudaMemcpyAsync(&v, flag, sizeof(v), cudaMemcpyDeviceToHost, st) != cudaSuccess ||
        cudaMemsetAsync(flag, 0, sizeof(v), st) != cudaSuccess || cudaStreamSynchronize(st) != cudaSuccess) {
        return W8A8_ERR_CUDA;
    }
    return v != 0 ? 1 : 0;
}
