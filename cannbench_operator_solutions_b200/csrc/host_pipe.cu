// grouped_matmul_swiglu_quant for rows that start, and results that end, in
// pinned HOST memory: host C++ that cuts the rows into chunks and keeps three
// streams busy at once - chunk i+1 going up, chunk i computing, chunk i-1
// coming back - over double-buffered device staging, so the call costs about
// as long as the slower copy direction instead of copy + compute + copy.  Each
// chunk is one call of w8a8_grouped_matmul_swiglu_quant with the chunk's own
// cumulative group list cut from the caller's (a chunk may start and end inside
// an expert's rows; rows are independent, so the results equal one call over
// all rows bit for bit).  Weights and their scales stay on the device.
#include <new>
#include <vector>

#include "common.cuh"

struct W8A8HostPipe {
    const int8_t* w;
    const float* w_scale;
    int64_t K, N, E, chunk;
    int w_layout;
    cudaStream_t s_in, s_out;
    cudaEvent_t start, arrived[2], computed[2], returned[2];
    int8_t* x[2];
    float* xs[2];
    int8_t* y[2];
    float* ys[2];
    void* workspace;
    size_t workspace_bytes;
    int device;
};

namespace {

size_t up256(size_t v) { return (v + 255) / 256 * 256; }

struct PipeLayout {
    size_t x, xs, y, ys, ws, total;
};

PipeLayout pipe_layout(int64_t K, int64_t N, int64_t E, int64_t chunk)
{
    PipeLayout l{};
    l.x = up256(static_cast<size_t>(chunk) * K);
    l.xs = up256(static_cast<size_t>(chunk) * 4);
    l.y = up256(static_cast<size_t>(chunk) * (N / 2));
    l.ys = up256(static_cast<size_t>(chunk) * 4);
    l.ws = up256(w8a8_grouped_matmul_swiglu_quant_workspace_size(chunk, K, N, E));
    l.total = 2 * (l.x + l.xs + l.y + l.ys) + l.ws;
    return l;
}

bool ok(cudaError_t e) { return e == cudaSuccess; }

}  // namespace

extern "C" size_t w8a8_gmsq_host_pipe_device_bytes(int64_t K, int64_t N, int64_t E, int64_t chunk_rows)
{
    if (K <= 0 || N <= 0 || (N & 1) || E <= 0 || chunk_rows <= 0) {
        return 0;
    }
    return pipe_layout(K, N, E, chunk_rows).total;
}

extern "C" int w8a8_gmsq_host_pipe_create(W8A8HostPipe** pipe, const int8_t* w, const float* w_scale, int64_t K,
                                          int64_t N, int64_t E, int w_layout, int64_t chunk_rows, void* device_mem,
                                          size_t device_bytes)
{
    if (pipe == nullptr || w == nullptr || w_scale == nullptr || K <= 0 || N <= 0 || (N & 1) || E <= 0 ||
        chunk_rows <= 0 || (w_layout != W8A8_W_KN && w_layout != W8A8_W_NK)) {
        return W8A8_ERR_INVALID;
    }
    const PipeLayout l = pipe_layout(K, N, E, chunk_rows);
    if (device_mem == nullptr || device_bytes < l.total) {
        return W8A8_ERR_WORKSPACE;
    }
    if (!w8a8::is_aligned(device_mem, 256)) {
        return W8A8_ERR_ALIGN;
    }
    W8A8HostPipe* p = new (std::nothrow) W8A8HostPipe();
    if (p == nullptr) {
        return W8A8_ERR_CUDA;
    }
    p->w = w;
    p->w_scale = w_scale;
    p->K = K;
    p->N = N;
    p->E = E;
    p->chunk = chunk_rows;
    p->w_layout = w_layout;
    bool good = ok(cudaGetDevice(&p->device)) && ok(cudaStreamCreateWithFlags(&p->s_in, cudaStreamNonBlocking)) &&
                ok(cudaStreamCreateWithFlags(&p->s_out, cudaStreamNonBlocking)) &&
                ok(cudaEventCreateWithFlags(&p->start, cudaEventDisableTiming));
    for (int b = 0; b < 2 && good; ++b) {
        good = ok(cudaEventCreateWithFlags(&p->arrived[b], cudaEventDisableTiming)) &&
               ok(cudaEventCreateWithFlags(&p->computed[b], cudaEventDisableTiming)) &&
               ok(cudaEventCreateWithFlags(&p->returned[b], cudaEventDisableTiming));
    }
    if (!good) {
        delete p;  // streams / events made so far are few and die with the context
        return W8A8_ERR_CUDA;
    }
    uint8_t* base = static_cast<uint8_t*>(device_mem);
    size_t off = 0;
    for (int b = 0; b < 2; ++b) {
        p->x[b] = reinterpret_cast<int8_t*>(base + off);
        off += l.x;
        p->xs[b] = reinterpret_cast<float*>(base + off);
        off += l.xs;
        p->y[b] = reinterpret_cast<int8_t*>(base + off);
        off += l.y;
        p->ys[b] = reinterpret_cast<float*>(base + off);
        off += l.ys;
    }
    p->workspace = base + off;
    p->workspace_bytes = l.ws;
    *pipe = p;
    return W8A8_OK;
}

extern "C" int w8a8_gmsq_host_pipe_destroy(W8A8HostPipe* p)
{
    if (p == nullptr) {
        return W8A8_OK;
    }
    cudaStreamDestroy(p->s_in);
    cudaStreamDestroy(p->s_out);
    cudaEventDestroy(p->start);
    for (int b = 0; b < 2; ++b) {
        cudaEventDestroy(p->arrived[b]);
        cudaEventDestroy(p->computed[b]);
        cudaEventDestroy(p->returned[b]);
    }
    delete p;
    return W8A8_OK;
}

// x_host [M, K] int8, x_scale_host [M], y_host [M, N/2] int8, y_scale_host [M]: pinned host memory (pageable memory
// works but the copies then do not overlap).  group_list_host: cumulative, E entries, last == M.  The call returns
// once everything is enqueued; the results are complete when `stream` has caught up.
extern "C" int w8a8_gmsq_host_pipe_run(W8A8HostPipe* p, const int8_t* x_host, const float* x_scale_host,
                                       const int64_t* group_list_host, int64_t M, int8_t* y_host, float* y_scale_host,
                                       int flags, void* stream)
{
    if (p == nullptr || M < 0 || (flags & ~W8A8_F_ROUND_DIRECT) != 0) {
        return W8A8_ERR_INVALID;
    }
    if (M == 0) {
        return W8A8_OK;
    }
    if (x_host == nullptr || x_scale_host == nullptr || group_list_host == nullptr || y_host == nullptr ||
        y_scale_host == nullptr) {
        return W8A8_ERR_INVALID;
    }
    int64_t prev = 0;
    for (int64_t g = 0; g < p->E; ++g) {
        if (group_list_host[g] < prev || group_list_host[g] > M) {
            return W8A8_ERR_GROUP_LIST;
        }
        prev = group_list_host[g];
    }
    if (prev != M) {
        return W8A8_ERR_GROUP_LIST;
    }
    cudaStream_t main = static_cast<cudaStream_t>(stream);
    const int64_t K = p->K, H = p->N / 2;
    if (!ok(cudaEventRecord(p->start, main)) || !ok(cudaStreamWaitEvent(p->s_in, p->start, 0)) ||
        !ok(cudaStreamWaitEvent(p->s_out, p->start, 0))) {
        return W8A8_ERR_CUDA;
    }
    std::vector<int64_t> local;
    int64_t e0 = 0;
    int64_t i = 0;
    for (int64_t r0 = 0; r0 < M; r0 += p->chunk, ++i) {
        const int64_t r1 = (r0 + p->chunk < M) ? r0 + p->chunk : M;
        const int64_t rows = r1 - r0;
        const int b = static_cast<int>(i & 1);
        // the chunk's experts and its own cumulative list
        while (e0 < p->E && group_list_host[e0] <= r0) {
            ++e0;
        }
        local.clear();
        for (int64_t e1 = e0;; ++e1) {
            const int64_t end = group_list_host[e1] < r1 ? group_list_host[e1] : r1;
            local.push_back(end - r0);
            if (group_list_host[e1] >= r1) {
                break;
            }
        }
        const int64_t experts = static_cast<int64_t>(local.size());
        // copy-in stream: wait until the staging buffer's previous reader (chunk i-2) has computed
        if (i >= 2 && !ok(cudaStreamWaitEvent(p->s_in, p->computed[b], 0))) {
            return W8A8_ERR_CUDA;
        }
        if (!ok(cudaMemcpyAsync(p->x[b], x_host + r0 * K, static_cast<size_t>(rows) * K, cudaMemcpyHostToDevice,
                                p->s_in)) ||
            !ok(cudaMemcpyAsync(p->xs[b], x_scale_host + r0, static_cast<size_t>(rows) * 4, cudaMemcpyHostToDevice,
                                p->s_in)) ||
            !ok(cudaEventRecord(p->arrived[b], p->s_in)) || !ok(cudaStreamWaitEvent(main, p->arrived[b], 0))) {
            return W8A8_ERR_CUDA;
        }
        // compute stream: the result buffer must have been copied out (chunk i-2)
        if (i >= 2 && !ok(cudaStreamWaitEvent(main, p->returned[b], 0))) {
            return W8A8_ERR_CUDA;
        }
        const size_t w_stride = static_cast<size_t>(p->K) * p->N;
        const int rc = w8a8_grouped_matmul_swiglu_quant(p->x[b], p->w + static_cast<size_t>(e0) * w_stride,
                                                        p->w_scale + static_cast<size_t>(e0) * p->N, p->xs[b], p->y[b],
                                                        p->ys[b], rows, p->K, p->N, experts, local.data(), 0,
                                                        p->w_layout, flags, p->workspace, p->workspace_bytes, main);
        if (rc != W8A8_OK) {
            return rc;
        }
        if (!ok(cudaEventRecord(p->computed[b], main)) || !ok(cudaStreamWaitEvent(p->s_out, p->computed[b], 0)) ||
            !ok(cudaMemcpyAsync(y_host + r0 * H, p->y[b], static_cast<size_t>(rows) * H, cudaMemcpyDeviceToHost,
                                p->s_out)) ||
            !ok(cudaMemcpyAsync(y_scale_host + r0, p->ys[b], static_cast<size_t>(rows) * 4, cudaMemcpyDeviceToHost,
                                p->s_out)) ||
            !ok(cudaEventRecord(p->returned[b], p->s_out))) {
            return W8A8_ERR_CUDA;
        }
    }
    // the caller's stream is done when both result buffers have been copied out
    if (!ok(cudaStreamWaitEvent(main, p->returned[0], 0)) || (i >= 2 && !ok(cudaStreamWaitEvent(main, p->returned[1], 0)))) {
        return W8A8_ERR_CUDA;
    }
    return W8A8_OK;
}
