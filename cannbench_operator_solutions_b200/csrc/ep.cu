// Expert-parallel bookkeeping kernels for sm_100a: routing plan (stable
// counting sort by expert), row scatter into expert-major order, and the
// weighted combine.
//
// Layout contract: rows of one expert are contiguous and keep (token, k)
// order, which is what a rank-major all-to-all followed by the reference's
// MoeReRouting permutation yields (operators/moererouting/csrc/ops/
// moe_re_routing/op_kernel/moe_re_routing_launch.h:15-21).  Combine
// arithmetic: fp32, term = prob * row rounded, then added, ascending k,
// round-to-nearest-even store (operators/moefinalizerouting/csrc/ops/
// moe_finalize_routing/op_kernel/moe_finalize_routing_kernel.cpp:15-25,165-170).
//
// All three are HBM-bound byte movers: 128-bit accesses, a row read once and
// written topk times (scatter) or topk rows read and one written (combine).
#include "common.cuh"

namespace w8a8 {

constexpr int RP_BLOCK = 256;  // pairs per counting block

// workspace layout: int32 block_count[B][E] (becomes the exclusive prefix over
// blocks), then int64 base[E]
__global__ void __launch_bounds__(RP_BLOCK) rp_count_kernel(const int32_t* __restrict__ expert_idx, int64_t P,
                                                            int64_t E, int32_t* __restrict__ block_count,
                                                            int32_t* __restrict__ bad)
{
    const int64_t p = static_cast<int64_t>(blockIdx.x) * RP_BLOCK + threadIdx.x;
    if (p < P) {
        const int32_t e = expert_idx[p];
        if (e < 0 || e >= E) {
            atomicExch(bad, 1);
        } else {
            atomicAdd(&block_count[static_cast<int64_t>(blockIdx.x) * E + e], 1);
        }
    }
}

__global__ void __launch_bounds__(1024) rp_scan_kernel(int32_t* __restrict__ block_count, int64_t B, int64_t E,
                                                       int64_t* __restrict__ base, int64_t* __restrict__ count,
                                                       int64_t* __restrict__ cumsum)
{
    for (int64_t e = threadIdx.x; e < E; e += blockDim.x) {
        int64_t run = 0;
        for (int64_t b = 0; b < B; ++b) {
            const int32_t c = block_count[b * E + e];
            block_count[b * E + e] = static_cast<int32_t>(run);
            run += c;
        }
        count[e] = run;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int64_t run = 0;
        for (int64_t e = 0; e < E; ++e) {
            base[e] = run;
            run += count[e];
            cumsum[e] = run;
        }
    }
}

__global__ void __launch_bounds__(RP_BLOCK) rp_place_kernel(const int32_t* __restrict__ expert_idx, int64_t P,
                                                            int64_t E, const int32_t* __restrict__ block_prefix,
                                                            const int64_t* __restrict__ base,
                                                            int64_t* __restrict__ expanded_pos)
{
    __shared__ int32_t s_e[RP_BLOCK];
    const int64_t p = static_cast<int64_t>(blockIdx.x) * RP_BLOCK + threadIdx.x;
    int32_t e = -1;
    if (p < P) {
        e = expert_idx[p];
    }
    s_e[threadIdx.x] = e;
    __syncthreads();
    if (p < P) {
        if (e < 0 || e >= E) {
            expanded_pos[p] = -1;
            return;
        }
        int rank = 0;
        for (int j = 0; j < static_cast<int>(threadIdx.x); ++j) {
            rank += (s_e[j] == e) ? 1 : 0;
        }
        expanded_pos[p] = base[e] + block_prefix[static_cast<int64_t>(blockIdx.x) * E + e] + rank;
    }
}

// One CTA per token: the row is read once and written to its topk slots.
template <bool VEC>
__global__ void __launch_bounds__(256) scatter_rows_kernel(const uint8_t* __restrict__ src,
                                                           const float* __restrict__ src_scale,
                                                           uint8_t* __restrict__ dst, float* __restrict__ dst_scale,
                                                           const int64_t* __restrict__ pos, int64_t T, int topk,
                                                           int64_t row_bytes)
{
    for (int64_t i = blockIdx.x; i < T; i += gridDim.x) {
        const uint8_t* s = src + i * row_bytes;
        if constexpr (VEC) {
            const int64_t n16 = row_bytes / 16;
            for (int64_t c = threadIdx.x; c < n16; c += blockDim.x) {
                const uint4 v = __ldcs(reinterpret_cast<const uint4*>(s) + c);
                for (int k = 0; k < topk; ++k) {
                    const int64_t p = pos[i * topk + k];
                    if (p >= 0) {
                        __stcs(reinterpret_cast<uint4*>(dst + p * row_bytes) + c, v);
                    }
                }
            }
        } else {
            for (int64_t c = threadIdx.x; c < row_bytes; c += blockDim.x) {
                const uint8_t v = s[c];
                for (int k = 0; k < topk; ++k) {
                    const int64_t p = pos[i * topk + k];
                    if (p >= 0) {
                        dst[p * row_bytes + c] = v;
                    }
                }
            }
        }
        if (src_scale != nullptr && dst_scale != nullptr && static_cast<int>(threadIdx.x) < topk) {
            const int64_t p = pos[i * topk + threadIdx.x];
            if (p >= 0) {
                dst_scale[p] = src_scale[i];
            }
        }
    }
}

// dst[d] = src[index[d]] for whole rows (and their fp32 scales): the regroup
// step after an all-to-all (rank-major -> expert-major) and its inverse.
// One warp per row at a time; a lane keeps PERMUTE_UNROLL 16-byte loads in flight before it stores, which is
// what a pure copy needs to cover the HBM latency (a CTA-wide loop with one load per thread reached 0.66 of the
// copy bandwidth, this form is measured in the benchmark's moe_re_routing workload).
constexpr int PERMUTE_UNROLL = 8;

template <bool VEC>
__global__ void __launch_bounds__(256) permute_rows_kernel(const uint8_t* __restrict__ src,
                                                           const float* __restrict__ src_scale,
                                                           uint8_t* __restrict__ dst, float* __restrict__ dst_scale,
                                                           const int64_t* __restrict__ index, int64_t rows,
                                                           int64_t row_bytes)
{
    const int lane = threadIdx.x & 31;
    const int64_t warps = static_cast<int64_t>(gridDim.x) * (blockDim.x >> 5);
    for (int64_t d = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5); d < rows;
         d += warps) {
        const int64_t s = index[d];
        if (s < 0) {
            continue;
        }
        if constexpr (VEC) {
            const uint4* sp = reinterpret_cast<const uint4*>(src + s * row_bytes);
            uint4* dp = reinterpret_cast<uint4*>(dst + d * row_bytes);
            const int64_t n16 = row_bytes / 16;
            for (int64_t base = 0; base < n16; base += 32 * PERMUTE_UNROLL) {
                uint4 v[PERMUTE_UNROLL];
#pragma unroll
                for (int u = 0; u < PERMUTE_UNROLL; ++u) {
                    const int64_t c = base + u * 32 + lane;
                    if (c < n16) {
                        v[u] = __ldcs(sp + c);
                    }
                }
#pragma unroll
                for (int u = 0; u < PERMUTE_UNROLL; ++u) {
                    const int64_t c = base + u * 32 + lane;
                    if (c < n16) {
                        __stcs(dp + c, v[u]);
                    }
                }
            }
        } else {
            for (int64_t c = lane; c < row_bytes; c += 32) {
                dst[d * row_bytes + c] = src[s * row_bytes + c];
            }
        }
        if (lane == 0 && src_scale != nullptr && dst_scale != nullptr) {
            dst_scale[d] = src_scale[s];
        }
    }
}

// Fused dispatch: the quantised row of token i is written straight to the row it will occupy in the
// expert-major buffer of the rank that owns expert idx[i, k] -- a plain store, over NVLink when that rank is a
// peer.  row_dst[e] / scale_dst[e] point at the first row / scale this rank may write for expert e in the
// owner's buffer, my_base[e] is the position of this rank's first pair for expert e in its own expert-major
// order, pos[i, k] that pair's position: destination row = row_dst[e] + (pos - my_base[e]) rows.
// This replaces pack + all-to-all + regroup with one pass; the row is read once and stored topk times.
template <bool VEC>
__global__ void __launch_bounds__(256) dispatch_rows_kernel(const uint8_t* __restrict__ src,
                                                            const float* __restrict__ src_scale,
                                                            const int32_t* __restrict__ expert_idx,
                                                            const int64_t* __restrict__ pos,
                                                            const uint64_t* __restrict__ row_dst,
                                                            const uint64_t* __restrict__ scale_dst,
                                                            const int64_t* __restrict__ my_base, int64_t T, int topk,
                                                            int64_t row_bytes)
{
    __shared__ uint64_t s_dst[64];
    for (int64_t i = blockIdx.x; i < T; i += gridDim.x) {
        __syncthreads();
        if (static_cast<int>(threadIdx.x) < topk) {
            const int64_t pr = i * topk + threadIdx.x;
            const int32_t e = expert_idx[pr];
            const int64_t p = pos[pr];
            uint64_t d = 0;
            if (p >= 0 && row_dst[e] != 0) {  // a zero destination: the table builder found the buffers too small
                const int64_t off = p - my_base[e];
                d = row_dst[e] + static_cast<uint64_t>(off) * static_cast<uint64_t>(row_bytes);
                if (src_scale != nullptr) {
                    reinterpret_cast<float*>(scale_dst[e])[off] = src_scale[i];
                }
            }
            s_dst[threadIdx.x] = d;
        }
        __syncthreads();
        const uint8_t* s = src + i * row_bytes;
        if constexpr (VEC) {
            const int64_t n16 = row_bytes / 16;
            for (int64_t c = threadIdx.x; c < n16; c += blockDim.x) {
                const uint4 v = __ldcs(reinterpret_cast<const uint4*>(s) + c);
                for (int k = 0; k < topk; ++k) {
                    const uint64_t d = s_dst[k];
                    if (d != 0) {
                        reinterpret_cast<uint4*>(d)[c] = v;
                    }
                }
            }
        } else {
            for (int64_t c = threadIdx.x; c < row_bytes; c += blockDim.x) {
                const uint8_t v = s[c];
                for (int k = 0; k < topk; ++k) {
                    const uint64_t d = s_dst[k];
                    if (d != 0) {
                        reinterpret_cast<uint8_t*>(d)[c] = v;
                    }
                }
            }
        }
    }
}

// out[r] = seg_ptr[s] + (r - seg_first[s]) * row_bytes for the segment s with seg_first[s] <= r < seg_first[s+1]
__global__ void __launch_bounds__(256) expand_row_pointers_kernel(const int64_t* __restrict__ seg_first,
                                                                  const uint64_t* __restrict__ seg_ptr, int nseg,
                                                                  int64_t rows, int64_t row_bytes,
                                                                  uint64_t* __restrict__ out)
{
    const int64_t r = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (r >= rows) {
        return;
    }
    int lo = 0, hi = nseg;  // last segment whose first row is <= r (empty segments share a first row)
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (seg_first[mid] <= r) {
            lo = mid;
        } else {
            hi = mid;
        }
    }
    out[r] = seg_ptr[lo] + static_cast<uint64_t>(r - seg_first[lo]) * static_cast<uint64_t>(row_bytes);
}

// ---------------------------------------------------------------------------
// MoeReRouting with the count matrix in device memory
// (operators/moererouting/csrc/ops/moe_re_routing/op_kernel/moe_re_routing_kernel.cpp:15-24)
// ---------------------------------------------------------------------------
// Cells are numbered in destination order, s = j * N + i (expert-major, then source rank):
//   dst_first[s] = colStart(j) + sum_{i'<i} cnt[i'][j]      (non-decreasing in s, one extra entry = total)
//   src_first[s] = rowStart(i) + sum_{j'<j} cnt[i][j']
// One CTA builds both tables; the matrix is small (ranks x local experts) next to the token rows.
// hdr[1] = 1 when a count is negative or the counts sum to more than A rows; the later kernels then do nothing.
template <typename CntT>
__global__ void __launch_bounds__(1024) rr_table_kernel(const CntT* __restrict__ cnt, int64_t N, int64_t E,
                                                        int64_t A, int32_t* __restrict__ hdr,
                                                        int64_t* __restrict__ dst_first,
                                                        int64_t* __restrict__ src_first,
                                                        int64_t* __restrict__ col_start,
                                                        int64_t* __restrict__ row_start,
                                                        CntT* __restrict__ expert_num)
{
    __shared__ int s_bad;
    const int tid = threadIdx.x;
    if (tid == 0) {
        s_bad = 0;
    }
    __syncthreads();
    bool bad = false;
    for (int64_t j = tid; j < E; j += blockDim.x) {
        int64_t sum = 0;
        for (int64_t i = 0; i < N; ++i) {
            const int64_t c = static_cast<int64_t>(cnt[i * E + j]);
            bad |= (c < 0) || (c > A);
            sum += c;
        }
        col_start[j + 1] = sum;
    }
    for (int64_t i = tid; i < N; i += blockDim.x) {
        int64_t sum = 0;
        for (int64_t j = 0; j < E; ++j) {
            const int64_t c = static_cast<int64_t>(cnt[i * E + j]);
            sum += (c < 0 || c > A) ? 0 : c;
        }
        row_start[i + 1] = sum;
    }
    if (bad) {
        s_bad = 1;
    }
    __syncthreads();
    // The two scans are short (local experts, ranks); two threads run them side by side.
    if (tid == 0) {
        int64_t run = 0;
        col_start[0] = 0;
        int64_t next = col_start[1];
        for (int64_t j = 0; j < E; ++j) {
            const int64_t c = next;
            if (j + 1 < E) {
                next = col_start[j + 2];  // issued before the dependent store of this step
            }
            run += c;
            if (run > A) {
                s_bad = 1;
                run = A;  // keeps later sums in range; nothing is copied once the flag is set
            }
            col_start[j + 1] = run;
        }
    }
    if (tid == 32) {
        int64_t run = 0;
        row_start[0] = 0;
        int64_t next = row_start[1];
        for (int64_t i = 0; i < N; ++i) {
            const int64_t c = next;
            if (i + 1 < N) {
                next = row_start[i + 2];
            }
            run += c;
            row_start[i + 1] = run;
        }
    }
    __syncthreads();
    if (tid == 0) {
        dst_first[N * E] = s_bad ? 0 : col_start[E];
        hdr[0] = 0;
        hdr[1] = s_bad;
    }
    __syncthreads();
    if (s_bad) {
        return;
    }
    for (int64_t j = tid; j < E; j += blockDim.x) {
        int64_t run = col_start[j];
        for (int64_t i = 0; i < N; ++i) {
            dst_first[j * N + i] = run;
            run += static_cast<int64_t>(cnt[i * E + j]);
        }
        expert_num[j] = static_cast<CntT>(run - col_start[j]);
    }
    for (int64_t i = tid; i < N; i += blockDim.x) {
        int64_t run = row_start[i];
        for (int64_t j = 0; j < E; ++j) {
            src_first[j * N + i] = run;
            run += static_cast<int64_t>(cnt[i * E + j]);
        }
    }
}

// The same tables for a matrix of at most RR_SMALL_CELLS cells (the usual case: ranks x local experts), with the
// matrix and every prefix staged in shared memory: the sequential scans then cost a few cycles per step instead
// of a global-memory round trip.
constexpr int RR_SMALL_CELLS = 2048;

template <typename CntT>
__global__ void __launch_bounds__(1024) rr_table_small_kernel(const CntT* __restrict__ cnt, int N, int E, int64_t A,
                                                              int32_t* __restrict__ hdr,
                                                              int64_t* __restrict__ dst_first,
                                                              int64_t* __restrict__ src_first,
                                                              CntT* __restrict__ expert_num)
{
    __shared__ int64_t s_cnt[RR_SMALL_CELLS];
    // E + N <= cells + 1, so one array of cells + 2 entries holds both prefixes: columns first, rows after them
    __shared__ int64_t s_sums[RR_SMALL_CELLS + 2];
    int64_t* s_col = s_sums;          // E + 1 entries: exclusive prefix of the column sums
    int64_t* s_row = s_sums + E + 1;  // N + 1 entries: exclusive prefix of the row sums
    __shared__ int s_bad;
    const int tid = threadIdx.x;
    const int cells = N * E;
    if (tid == 0) {
        s_bad = 0;
    }
    __syncthreads();
    for (int c = tid; c < cells; c += blockDim.x) {
        const int64_t v = static_cast<int64_t>(cnt[c]);
        if (v < 0 || v > A) {
            s_bad = 1;
        }
        s_cnt[c] = (v < 0 || v > A) ? 0 : v;
    }
    __syncthreads();
    for (int j = tid; j < E; j += blockDim.x) {
        int64_t sum = 0;
        for (int i = 0; i < N; ++i) {
            sum += s_cnt[i * E + j];
        }
        s_col[j + 1] = sum;
    }
    for (int i = tid; i < N; i += blockDim.x) {
        int64_t sum = 0;
        for (int j = 0; j < E; ++j) {
            sum += s_cnt[i * E + j];
        }
        s_row[i + 1] = sum;
    }
    __syncthreads();
    if (tid == 0) {
        int64_t run = 0;
        s_col[0] = 0;
        for (int j = 0; j < E; ++j) {
            run += s_col[j + 1];
            s_col[j + 1] = run;
        }
        if (run > A) {
            s_bad = 1;
        }
    }
    if (tid == 32) {
        int64_t run = 0;
        s_row[0] = 0;
        for (int i = 0; i < N; ++i) {
            run += s_row[i + 1];
            s_row[i + 1] = run;
        }
    }
    __syncthreads();
    const bool bad = (s_bad != 0);
    if (tid == 0) {
        dst_first[cells] = bad ? 0 : s_col[E];
        hdr[0] = 0;
        hdr[1] = bad ? 1 : 0;
    }
    if (bad) {
        return;
    }
    for (int j = tid; j < E; j += blockDim.x) {
        int64_t run = s_col[j];
        for (int i = 0; i < N; ++i) {
            dst_first[j * N + i] = run;
            run += s_cnt[i * E + j];
        }
        expert_num[j] = static_cast<CntT>(run - s_col[j]);
    }
    for (int i = tid; i < N; i += blockDim.x) {
        int64_t run = s_row[i];
        for (int j = 0; j < E; ++j) {
            src_first[j * N + i] = run;
            run += s_cnt[i * E + j];
        }
    }
}

// index[d] = source row of destination row d (-1 past the routed rows); out_idx[d] the same as int32.
__global__ void __launch_bounds__(256) rr_index_kernel(const int32_t* __restrict__ hdr,
                                                       const int64_t* __restrict__ dst_first,
                                                       const int64_t* __restrict__ src_first, int64_t cells,
                                                       int64_t A, int64_t* __restrict__ index,
                                                       int32_t* __restrict__ out_idx)
{
    const int64_t d = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (d >= A) {
        return;
    }
    if (hdr[1] != 0 || d >= dst_first[cells]) {
        index[d] = -1;
        return;
    }
    int64_t lo = 0, hi = cells;  // last cell whose first row is <= d (empty cells share a first row)
    while (hi - lo > 1) {
        const int64_t mid = (lo + hi) >> 1;
        if (dst_first[mid] <= d) {
            lo = mid;
        } else {
            hi = mid;
        }
    }
    const int64_t s = src_first[lo] + (d - dst_first[lo]);
    index[d] = s;
    out_idx[d] = static_cast<int32_t>(s);
}

// ---------------------------------------------------------------------------
// MoeFinalizeRouting
// (operators/moefinalizerouting/csrc/ops/moe_finalize_routing/op_kernel/moe_finalize_routing_kernel.cpp:15-25)
// ---------------------------------------------------------------------------
// A 16-byte chunk of a row: 8 elements of a 16-bit type or 4 floats.  Chunks are kept in registers in their raw
// form (a uint4) while loads are in flight and unpacked to fp32 only when they are consumed.
template <int DT>
struct RowChunk {
    static constexpr int EL = (DT == W8A8_DT_F32) ? 4 : 8;

    template <bool VEC>
    static __device__ __forceinline__ uint4 load_raw(const void* base, int64_t row, int c, int64_t H)
    {
        if constexpr (DT == W8A8_DT_F32) {
            const float* r = static_cast<const float*>(base) + row * H;
            if constexpr (VEC) {
                return __ldcs(reinterpret_cast<const uint4*>(r) + c);
            } else {
                uint32_t w[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int64_t e = static_cast<int64_t>(c) * 4 + j;
                    w[j] = (e < H) ? __float_as_uint(r[e]) : 0u;
                }
                return make_uint4(w[0], w[1], w[2], w[3]);
            }
        } else {
            return load_chunk16<VEC>(static_cast<const uint16_t*>(base) + row * H, c, H);
        }
    }

    static __device__ __forceinline__ void unpack(const uint4& v, float (&f)[EL])
    {
        if constexpr (DT == W8A8_DT_F32) {
            f[0] = __uint_as_float(v.x), f[1] = __uint_as_float(v.y);
            f[2] = __uint_as_float(v.z), f[3] = __uint_as_float(v.w);
        } else {
            unpack2<DT>(v.x, f[0], f[1]);
            unpack2<DT>(v.y, f[2], f[3]);
            unpack2<DT>(v.z, f[4], f[5]);
            unpack2<DT>(v.w, f[6], f[7]);
        }
    }

    template <bool VEC>
    static __device__ __forceinline__ void load(const void* base, int64_t row, int c, int64_t H, float (&f)[EL])
    {
        unpack(load_raw<VEC>(base, row, c, H), f);
    }

    template <bool VEC>
    static __device__ __forceinline__ void store(void* base, int64_t row, int c, int64_t H, const float (&f)[EL])
    {
        if constexpr (DT == W8A8_DT_F32) {
            float* r = static_cast<float*>(base) + row * H;
            if constexpr (VEC) {
                __stcs(reinterpret_cast<float4*>(r) + c, make_float4(f[0], f[1], f[2], f[3]));
            } else {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int64_t e = static_cast<int64_t>(c) * 4 + j;
                    if (e < H) {
                        r[e] = f[j];
                    }
                }
            }
        } else {
            const uint4 o = make_uint4(pack2<DT>(f[0], f[1]), pack2<DT>(f[2], f[3]), pack2<DT>(f[4], f[5]),
                                       pack2<DT>(f[6], f[7]));
            store_chunk16<VEC>(static_cast<uint16_t*>(base) + row * H, c, H, o);
        }
    }
};

__device__ __forceinline__ float load_scalar_as_f32(const void* p, int64_t i, int dt)
{
    if (dt == W8A8_DT_F32) {
        return static_cast<const float*>(p)[i];
    }
    const uint32_t b = static_cast<const uint16_t*>(p)[i];
    return (dt == W8A8_DT_BF16) ? bits16_to_float<W8A8_DT_BF16>(b) : bits16_to_float<W8A8_DT_F16>(b);
}

// One CTA per output row.  The K (position, scale, expert) triples of the row are staged in shared memory once;
// every thread then owns 16-byte chunks of the hidden dimension and, for MFR_BATCH values of k at a time, issues
// all its row (and bias) loads before it touches the accumulator, so up to MFR_BATCH gathers are in flight per
// thread.  Arithmetic order per element: acc = fp32(skip1); acc += fp32(skip2); for ascending k:
// term = fp32(row) [+ fp32(bias)]; term *= scale; acc += term (no fused multiply-add); RNE store.
constexpr int MFR_BATCH = 8;
constexpr int MFR_MAX_STAGED_K = 128;

template <int DT, bool VEC, bool HAS_BIAS, typename IdxT>
__global__ void __launch_bounds__(256) mfr_kernel(const void* __restrict__ rows, const IdxT* __restrict__ esdr,
                                                  const void* __restrict__ skip1, const void* __restrict__ skip2,
                                                  const void* __restrict__ bias, const void* __restrict__ scales,
                                                  const int32_t* __restrict__ expert, void* __restrict__ out,
                                                  int64_t R, int64_t H, int K, int64_t E, int64_t num_dst,
                                                  int col_mode, int scale_dt)
{
    using C = RowChunk<DT>;
    constexpr int EL = C::EL;
    __shared__ int64_t s_pos[MFR_MAX_STAGED_K];
    __shared__ int64_t s_eid[MFR_MAX_STAGED_K];
    __shared__ float s_w[MFR_MAX_STAGED_K];
    const int nchunks = static_cast<int>((H + EL - 1) / EL);
    for (int64_t i = blockIdx.x; i < R; i += gridDim.x) {
        for (int k0 = 0; k0 < K; k0 += MFR_MAX_STAGED_K) {
            const int kn = min(K - k0, MFR_MAX_STAGED_K);
            __syncthreads();
            if (static_cast<int>(threadIdx.x) < kn) {
                const int k = k0 + threadIdx.x;
                int64_t p = esdr[col_mode ? (static_cast<int64_t>(k) * R + i) : (i * K + k)];
                if (p < 0 || p >= num_dst) {
                    p = -1;
                }
                int64_t eid = -1;
                if constexpr (HAS_BIAS) {
                    eid = expert[i * K + k];
                    if (eid < 0 || eid >= E) {
                        eid = -1;
                    }
                }
                s_pos[threadIdx.x] = p;
                s_eid[threadIdx.x] = eid;
                s_w[threadIdx.x] = (scales != nullptr) ? load_scalar_as_f32(scales, i * K + k, scale_dt) : 1.0f;
            }
            __syncthreads();
            for (int c = threadIdx.x; c < nchunks; c += blockDim.x) {
                float acc[EL];
                if (k0 == 0) {
                    if (skip1 != nullptr) {
                        C::template load<VEC>(skip1, i, c, H, acc);
                    } else {
#pragma unroll
                        for (int j = 0; j < EL; ++j) {
                            acc[j] = 0.0f;
                        }
                    }
                    if (skip2 != nullptr) {
                        float t[EL];
                        C::template load<VEC>(skip2, i, c, H, t);
#pragma unroll
                        for (int j = 0; j < EL; ++j) {
                            acc[j] = __fadd_rn(acc[j], t[j]);
                        }
                    }
                } else {
                    // more than MFR_MAX_STAGED_K terms: the partial sum so far is in `out` as fp32 only when the
                    // output type is fp32; other types take the single-pass route below (K is limited by the host)
                    C::template load<VEC>(out, i, c, H, acc);
                }
                for (int kb = 0; kb < kn; kb += MFR_BATCH) {
                    uint4 v[MFR_BATCH];
                    uint4 b[HAS_BIAS ? MFR_BATCH : 1];
#pragma unroll
                    for (int u = 0; u < MFR_BATCH; ++u) {
                        const int k = kb + u;
                        if (k < kn && s_pos[k] >= 0) {
                            v[u] = C::template load_raw<VEC>(rows, s_pos[k], c, H);
                            if constexpr (HAS_BIAS) {
                                if (s_eid[k] >= 0) {
                                    b[u] = C::template load_raw<VEC>(bias, s_eid[k], c, H);
                                }
                            }
                        }
                    }
#pragma unroll
                    for (int u = 0; u < MFR_BATCH; ++u) {
                        const int k = kb + u;
                        if (k < kn && s_pos[k] >= 0) {
                            const bool add_bias = HAS_BIAS && s_eid[k] >= 0;
                            const float w = s_w[k];
                            float vf[EL];
                            float bf[EL];
                            C::unpack(v[u], vf);
                            if constexpr (HAS_BIAS) {
                                if (add_bias) {
                                    C::unpack(b[u], bf);
                                }
                            }
#pragma unroll
                            for (int j = 0; j < EL; ++j) {
                                float term = vf[j];
                                if (add_bias) {
                                    term = __fadd_rn(term, bf[j]);
                                }
                                if (scales != nullptr) {
                                    term = __fmul_rn(term, w);
                                }
                                acc[j] = __fadd_rn(acc[j], term);
                            }
                        }
                    }
                }
                C::template store<VEC>(out, i, c, H, acc);
            }
        }
    }
}

// ---------------------------------------------------------------------------
// Expert-parallel address tables, computed on the device from the all-gathered count matrix C[P, E]
// (C[i][e] = rows rank i routes to global expert e; expert e lives on rank e / (E / P)).
// Everything dispatch_rows, the grouped matmuls and the row-pointer expansion need, with no host readback:
//   row_dst[e], scale_dst[e]  where this rank's first row / scale for expert e goes in the owner's buffers
//   my_base[e]                position of this rank's first pair for expert e in its own expert-major order
//   group_list[j]             cumulative rows of this rank's local experts (all source ranks)
//   seg_first / seg_ptr       one segment per (local expert, source rank): first local row, and the address in
//                             the source rank's return buffer where the segment's first output row goes
//   status[0]                 1 when some rank would receive more rows than the buffers hold
// One CTA; thread i < P walks rank i's counts, thread e < E a column.
// ---------------------------------------------------------------------------
constexpr int EP_MAX_RANKS = 64;
constexpr int EP_MAX_CELLS = 2048;  // P * E, held in shared memory

__global__ void __launch_bounds__(1024) ep_tables_kernel(const int64_t* __restrict__ counts, int P, int E, int rank,
                                                         const uint64_t* __restrict__ peer_base, uint64_t off_x,
                                                         uint64_t off_s, uint64_t off_back, int64_t row_bytes,
                                                         int64_t back_row_bytes, int64_t cap_rows,
                                                         uint64_t* __restrict__ row_dst,
                                                         uint64_t* __restrict__ scale_dst,
                                                         int64_t* __restrict__ my_base,
                                                         int64_t* __restrict__ group_list,
                                                         int64_t* __restrict__ seg_first,
                                                         uint64_t* __restrict__ seg_ptr, int32_t* __restrict__ status)
{
    // The whole matrix is staged in shared memory first (one coalesced pass), so that the sequential prefix loops
    // below run on shared memory instead of waiting for a global load per step.  Row counts fit 32 bits (a rank's
    // buffers hold fewer than 2^31 rows; larger counts set the overflow flag).
    __shared__ int32_t s_cnt[EP_MAX_CELLS];   // [P][E]
    __shared__ int32_t s_base[EP_MAX_CELLS];  // [P][E]: rank i's exclusive prefix over experts
    __shared__ int32_t s_seg[EP_MAX_CELLS];   // [E/P][P]: first local row of each (local expert, source rank) segment
    __shared__ int32_t s_col[1024];           // rows per expert over all ranks
    __shared__ int32_t s_before[1024];        // rows of lower ranks inside each expert
    __shared__ int32_t s_exbase[1024];        // expert's first row in its owner's buffer
    __shared__ int s_bad;
    const int tid = threadIdx.x;
    const int e_local = E / P;
    const int cells = P * E;
    if (tid == 0) {
        s_bad = 0;
    }
    __syncthreads();
    const int64_t limit = cap_rows < 0x7fffffffLL ? cap_rows : 0x7fffffffLL;
    for (int c = tid; c < cells; c += blockDim.x) {
        const int64_t v = counts[c];
        if (v < 0 || v > limit) {
            s_bad = 1;
        }
        s_cnt[c] = (v < 0 || v > limit) ? 0 : static_cast<int32_t>(v);
    }
    __syncthreads();
    if (tid < P) {
        int64_t run = 0;
        for (int e = 0; e < E; ++e) {
            s_base[tid * E + e] = static_cast<int32_t>(run);
            run += s_cnt[tid * E + e];
        }
        if (run > 0x7fffffffLL) {
            s_bad = 1;
        }
    }
    for (int e = tid; e < E; e += blockDim.x) {
        int64_t col = 0, before = 0;
        for (int i = 0; i < P; ++i) {
            const int32_t c = s_cnt[i * E + e];
            if (i < rank) {
                before += c;
            }
            col += c;
        }
        if (col > limit) {
            s_bad = 1;
            col = 0;
            before = 0;
        }
        s_col[e] = static_cast<int32_t>(col);
        s_before[e] = static_cast<int32_t>(before);
    }
    __syncthreads();
    if (tid < P) {  // thread o: the experts of owner o
        int64_t run = 0;
        for (int j = 0; j < e_local; ++j) {
            const int e = tid * e_local + j;
            s_exbase[e] = static_cast<int32_t>(run < 0x7fffffffLL ? run : 0);
            run += s_col[e];
            if (tid == rank) {
                group_list[j] = run;
            }
        }
        if (run > cap_rows) {
            s_bad = 1;
        }
    }
    if (tid == 32) {  // segments in (local expert, source rank) order: exclusive prefix of their lengths
        int64_t run = 0;
        for (int j = 0; j < e_local; ++j) {
            const int e = rank * e_local + j;
            for (int i = 0; i < P; ++i) {
                s_seg[j * P + i] = static_cast<int32_t>(run < 0x7fffffffLL ? run : 0);
                run += s_cnt[i * E + e];
            }
        }
    }
    __syncthreads();
    // Too many rows for some rank's buffers: nothing may be stored anywhere.  Every rank sees the same counts, so
    // every rank takes this branch together: zero destinations (dispatch skips them) and empty groups.
    const bool bad = (s_bad != 0);
    const int nseg = e_local * P;
    for (int e = tid; e < E; e += blockDim.x) {
        const int owner = e / e_local;
        const uint64_t first = static_cast<uint64_t>(s_exbase[e]) + static_cast<uint64_t>(s_before[e]);
        row_dst[e] = bad ? 0 : peer_base[owner] + off_x + first * static_cast<uint64_t>(row_bytes);
        scale_dst[e] = bad ? 0 : peer_base[owner] + off_s + first * 4u;
        my_base[e] = s_base[rank * E + e];
    }
    for (int sidx = tid; sidx < nseg; sidx += blockDim.x) {
        const int j = sidx / P, i = sidx - j * P;
        const int e = rank * e_local + j;
        seg_first[sidx] = bad ? 0 : s_seg[sidx];
        seg_ptr[sidx] = bad ? 0
                            : peer_base[i] + off_back +
                                  static_cast<uint64_t>(s_base[i * E + e]) * static_cast<uint64_t>(back_row_bytes);
    }
    if (bad) {
        for (int j = tid; j < e_local; j += blockDim.x) {
            group_list[j] = 0;
        }
    }
    if (tid == 0) {
        // the last local expert's cumulative count is the number of rows this rank holds
        int64_t total = 0;
        for (int j = 0; j < e_local; ++j) {
            total += s_col[rank * e_local + j];
        }
        seg_first[nseg] = bad ? 0 : total;
        // sticky: a later good step must not hide an overflowed one; the reader clears it
        if (bad) {
            status[0] = 1;
        }
    }
}

static inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

}  // namespace w8a8

extern "C" size_t w8a8_route_plan_workspace_size(int64_t T, int64_t topk, int64_t E)
{
    if (T < 0 || topk <= 0 || E <= 0) {
        return 0;
    }
    const int64_t P = T * topk;
    const int64_t B = (P + w8a8::RP_BLOCK - 1) / w8a8::RP_BLOCK;
    size_t bytes = 256;  // error word
    bytes += w8a8::align_up(static_cast<size_t>(B > 0 ? B : 1) * static_cast<size_t>(E) * sizeof(int32_t), 256);
    bytes += w8a8::align_up(static_cast<size_t>(E) * sizeof(int64_t), 256);
    return bytes;
}

extern "C" int w8a8_route_plan(const int32_t* expert_idx, int64_t T, int64_t topk, int64_t E, int64_t* count,
                               int64_t* cumsum, int64_t* expanded_pos, void* workspace, size_t workspace_bytes,
                               void* stream)
{
    if (T < 0 || topk <= 0 || E <= 0 || count == nullptr || cumsum == nullptr) {
        return W8A8_ERR_INVALID;
    }
    if (T > 0 && (expert_idx == nullptr || expanded_pos == nullptr)) {
        return W8A8_ERR_INVALID;
    }
    const size_t need = w8a8_route_plan_workspace_size(T, topk, E);
    if (workspace == nullptr || workspace_bytes < need) {
        return W8A8_ERR_WORKSPACE;
    }
    if (!w8a8::is_aligned(workspace, 256)) {
        return W8A8_ERR_ALIGN;
    }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int64_t P = T * topk;
    const int64_t B = (P + w8a8::RP_BLOCK - 1) / w8a8::RP_BLOCK;
    uint8_t* ws = static_cast<uint8_t*>(workspace);
    int32_t* bad = reinterpret_cast<int32_t*>(ws);
    int32_t* block_count = reinterpret_cast<int32_t*>(ws + 256);
    const size_t bc_bytes = w8a8::align_up(static_cast<size_t>(B > 0 ? B : 1) * E * sizeof(int32_t), 256);
    int64_t* base = reinterpret_cast<int64_t*>(ws + 256 + bc_bytes);
    if (cudaMemsetAsync(ws, 0, 256 + bc_bytes, st) != cudaSuccess) {
        return W8A8_ERR_CUDA;
    }
    if (B > 0) {
        w8a8::rp_count_kernel<<<static_cast<unsigned>(B), w8a8::RP_BLOCK, 0, st>>>(expert_idx, P, E, block_count, bad); w8a8::note_launch();
    }
    w8a8::rp_scan_kernel<<<1, 1024, 0, st>>>(block_count, B, E, base, count, cumsum); w8a8::note_launch();
    if (B > 0) {
        w8a8::rp_place_kernel<<<static_cast<unsigned>(B), w8a8::RP_BLOCK, 0, st>>>(expert_idx, P, E, block_count, base,
                                                                                  expanded_pos); w8a8::note_launch();
    }
    return (cudaGetLastError() == cudaSuccess) ? W8A8_OK : W8A8_ERR_CUDA;
}

extern "C" int w8a8_scatter_rows(const void* src, const float* src_scale, void* dst, float* dst_scale,
                                 const int64_t* expanded_pos, int64_t T, int64_t topk, int64_t row_bytes,
                                 void* stream)
{
    if (T < 0 || topk <= 0 || topk > 256 || row_bytes <= 0) {
        return W8A8_ERR_INVALID;
    }
    if (T == 0) {
        return W8A8_OK;
    }
    if (src == nullptr || dst == nullptr || expanded_pos == nullptr) {
        return W8A8_ERR_INVALID;
    }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const bool vec = (row_bytes % 16 == 0) && w8a8::is_aligned(src, 16) && w8a8::is_aligned(dst, 16);
    const int64_t cap = static_cast<int64_t>(w8a8::sm_count()) * 8;
    const unsigned grid = static_cast<unsigned>(T < cap ? T : cap);
    if (vec) {
        w8a8::scatter_rows_kernel<true><<<grid, 256, 0, st>>>(static_cast<const uint8_t*>(src), src_scale,
                                                             static_cast<uint8_t*>(dst), dst_scale, expanded_pos, T,
                                                             static_cast<int>(topk), row_bytes); w8a8::note_launch();
    } else {
        w8a8::scatter_rows_kernel<false><<<grid, 256, 0, st>>>(static_cast<const uint8_t*>(src), src_scale,
                                                              static_cast<uint8_t*>(dst), dst_scale, expanded_pos, T,
                                                              static_cast<int>(topk), row_bytes); w8a8::note_launch();
    }
    return (cudaGetLastError() == cudaSuccess) ? W8A8_OK : W8A8_ERR_CUDA;
}

extern "C" int w8a8_permute_rows(const void* src, const float* src_scale, void* dst, float* dst_scale,
                                 const int64_t* index, int64_t rows, int64_t row_bytes, void* stream)
{
    if (rows < 0 || row_bytes <= 0) {
        return W8A8_ERR_INVALID;
    }
    if (rows == 0) {
        return W8A8_OK;
    }
    if (src == nullptr || dst == nullptr || index == nullptr) {
        return W8A8_ERR_INVALID;
    }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const bool vec = (row_bytes % 16 == 0) && w8a8::is_aligned(src, 16) && w8a8::is_aligned(dst, 16);
    const int64_t cap = static_cast<int64_t>(w8a8::sm_count()) * 8;  // 8 CTAs of 8 warps fill an SM
    const int64_t want = (rows + 7) / 8;                             // one warp per row
    const unsigned grid = static_cast<unsigned>(want < cap ? want : cap);
    if (vec) {
        w8a8::permute_rows_kernel<true><<<grid, 256, 0, st>>>(static_cast<const uint8_t*>(src), src_scale,
                                                             static_cast<uint8_t*>(dst), dst_scale, index, rows,
                                                             row_bytes); w8a8::note_launch();
    } else {
        w8a8::permute_rows_kernel<false><<<grid, 256, 0, st>>>(static_cast<const uint8_t*>(src), src_scale,
                                                              static_cast<uint8_t*>(dst), dst_scale, index, rows,
                                                              row_bytes); w8a8::note_launch();
    }
    return (cudaGetLastError() == cudaSuccess) ? W8A8_OK : W8A8_ERR_CUDA;
}

extern "C" int w8a8_dispatch_rows(const void* src, const float* src_scale, const int32_t* expert_idx,
                                  const int64_t* expanded_pos, const uint64_t* row_dst, const uint64_t* scale_dst,
                                  const int64_t* my_base, int64_t T, int64_t topk, int64_t row_bytes, void* stream)
{
    if (T < 0 || topk <= 0 || topk > 64 || row_bytes <= 0) {
        return W8A8_ERR_INVALID;
    }
    if (T == 0) {
        return W8A8_OK;
    }
    if (src == nullptr || expert_idx == nullptr || expanded_pos == nullptr || row_dst == nullptr ||
        my_base == nullptr || (src_scale != nullptr && scale_dst == nullptr)) {
        return W8A8_ERR_INVALID;
    }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    // destination rows are row_bytes apart from 16-byte aligned bases when the sources are
    const bool vec = (row_bytes % 16 == 0) && w8a8::is_aligned(src, 16);
    const int64_t cap = static_cast<int64_t>(w8a8::sm_count()) * 8;
    const unsigned grid = static_cast<unsigned>(T < cap ? T : cap);
    if (vec) {
        w8a8::dispatch_rows_kernel<true><<<grid, 256, 0, st>>>(static_cast<const uint8_t*>(src), src_scale, expert_idx,
                                                              expanded_pos, row_dst, scale_dst, my_base, T,
                                                              static_cast<int>(topk), row_bytes); w8a8::note_launch();
    } else {
        w8a8::dispatch_rows_kernel<false><<<grid, 256, 0, st>>>(static_cast<const uint8_t*>(src), src_scale,
                                                               expert_idx, expanded_pos, row_dst, scale_dst, my_base,
                                                               T, static_cast<int>(topk), row_bytes); w8a8::note_launch();
    }
    return (cudaGetLastError() == cudaSuccess) ? W8A8_OK : W8A8_ERR_CUDA;
}

extern "C" int w8a8_expand_row_pointers(const int64_t* seg_first, const uint64_t* seg_ptr, int64_t nseg, int64_t rows,
                                        int64_t row_bytes, uint64_t* out, void* stream)
{
    if (nseg <= 0 || rows < 0 || row_bytes <= 0 || nseg >= (int64_t(1) << 30)) {
        return W8A8_ERR_INVALID;
    }
    if (rows == 0) {
        return W8A8_OK;
    }
    if (seg_first == nullptr || seg_ptr == nullptr || out == nullptr) {
        return W8A8_ERR_INVALID;
    }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const unsigned grid = static_cast<unsigned>((rows + 255) / 256);
    w8a8::expand_row_pointers_kernel<<<grid, 256, 0, st>>>(seg_first, seg_ptr, static_cast<int>(nseg), rows, row_bytes,
                                                           out); w8a8::note_launch();
    return (cudaGetLastError() == cudaSuccess) ? W8A8_OK : W8A8_ERR_CUDA;
}

extern "C" int w8a8_combine(const void* rows, const float* probs, const int64_t* expanded_pos, void* out, int64_t T,
                            int64_t topk, int64_t H, int dtype, void* stream)
{
    if (dtype != W8A8_DT_F16 && dtype != W8A8_DT_BF16) {
        return W8A8_ERR_INVALID;
    }
    if (T < 0 || topk <= 0 || H <= 0) {
        return W8A8_ERR_INVALID;
    }
    if (T == 0) {
        return W8A8_OK;
    }
    if (rows == nullptr || probs == nullptr || expanded_pos == nullptr || out == nullptr) {
        return W8A8_ERR_INVALID;
    }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const bool vec = (H % 8 == 0) && w8a8::is_aligned(rows, 16) && w8a8::is_aligned(out, 16);
    const int64_t cap = static_cast<int64_t>(w8a8::sm_count()) * 8;
    const unsigned grid = static_cast<unsigned>(T < cap ? T : cap);
    // The scales-only, row-arranged case of the finalize kernel with 64-bit positions (no upper bound on them).
    if (topk > w8a8::MFR_MAX_STAGED_K) {
        return W8A8_ERR_LIMIT;
    }
    auto kern = (dtype == W8A8_DT_BF16)
                    ? (vec ? w8a8::mfr_kernel<W8A8_DT_BF16, true, false, int64_t>
                           : w8a8::mfr_kernel<W8A8_DT_BF16, false, false, int64_t>)
                    : (vec ? w8a8::mfr_kernel<W8A8_DT_F16, true, false, int64_t>
                           : w8a8::mfr_kernel<W8A8_DT_F16, false, false, int64_t>);
    kern<<<grid, 256, 0, st>>>(rows, expanded_pos, nullptr, nullptr, nullptr, probs, nullptr, out, T, H,
                               static_cast<int>(topk), 0, INT64_MAX, 0, W8A8_DT_F32); w8a8::note_launch();
    return (cudaGetLastError() == cudaSuccess) ? W8A8_OK : W8A8_ERR_CUDA;
}

// workspace: 256-byte header | dst_first[N*E+1] | src_first[N*E] | col_start[E+1] | row_start[N+1] | index[A]
extern "C" size_t w8a8_moe_re_routing_workspace_size(int64_t A, int64_t N, int64_t E)
{
    if (A < 0 || N <= 0 || E <= 0) {
        return 0;
    }
    const size_t cells = static_cast<size_t>(N) * static_cast<size_t>(E);
    size_t bytes = 256;
    bytes += w8a8::align_up((cells + 1) * sizeof(int64_t), 256);
    bytes += w8a8::align_up(cells * sizeof(int64_t), 256);
    bytes += w8a8::align_up(static_cast<size_t>(E + 1) * sizeof(int64_t), 256);
    bytes += w8a8::align_up(static_cast<size_t>(N + 1) * sizeof(int64_t), 256);
    bytes += w8a8::align_up(static_cast<size_t>(A > 0 ? A : 1) * sizeof(int64_t), 256);
    return bytes;
}

extern "C" int w8a8_moe_re_routing(const void* tokens, const void* counts, const float* scales, void* out_tokens,
                                   float* out_scales, int32_t* out_idx, void* expert_token_num, int64_t A,
                                   int64_t row_bytes, int64_t N, int64_t E, int count_bytes, void* workspace,
                                   size_t workspace_bytes, void* stream)
{
    if (A < 0 || row_bytes <= 0 || N <= 0 || E <= 0 || (count_bytes != 4 && count_bytes != 8)) {
        return W8A8_ERR_INVALID;
    }
    if (A > INT32_MAX) {
        return W8A8_ERR_LIMIT;  // permute_token_idx is int32
    }
    if (counts == nullptr || expert_token_num == nullptr) {
        return W8A8_ERR_INVALID;
    }
    if (A > 0 && (tokens == nullptr || out_tokens == nullptr || out_idx == nullptr)) {
        return W8A8_ERR_INVALID;
    }
    if (workspace == nullptr || workspace_bytes < w8a8_moe_re_routing_workspace_size(A, N, E)) {
        return W8A8_ERR_WORKSPACE;
    }
    if (!w8a8::is_aligned(workspace, 256) || !w8a8::is_aligned(counts, static_cast<size_t>(count_bytes))) {
        return W8A8_ERR_ALIGN;
    }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const size_t cells = static_cast<size_t>(N) * static_cast<size_t>(E);
    uint8_t* ws = static_cast<uint8_t*>(workspace);
    int32_t* hdr = reinterpret_cast<int32_t*>(ws);
    ws += 256;
    int64_t* dst_first = reinterpret_cast<int64_t*>(ws);
    ws += w8a8::align_up((cells + 1) * sizeof(int64_t), 256);
    int64_t* src_first = reinterpret_cast<int64_t*>(ws);
    ws += w8a8::align_up(cells * sizeof(int64_t), 256);
    int64_t* col_start = reinterpret_cast<int64_t*>(ws);
    ws += w8a8::align_up(static_cast<size_t>(E + 1) * sizeof(int64_t), 256);
    int64_t* row_start = reinterpret_cast<int64_t*>(ws);
    ws += w8a8::align_up(static_cast<size_t>(N + 1) * sizeof(int64_t), 256);
    int64_t* index = reinterpret_cast<int64_t*>(ws);

    if (cells <= static_cast<size_t>(w8a8::RR_SMALL_CELLS)) {
        if (count_bytes == 4) {
            w8a8::rr_table_small_kernel<int32_t><<<1, 1024, 0, st>>>(
                static_cast<const int32_t*>(counts), static_cast<int>(N), static_cast<int>(E), A, hdr, dst_first,
                src_first, static_cast<int32_t*>(expert_token_num)); w8a8::note_launch();
        } else {
            w8a8::rr_table_small_kernel<int64_t><<<1, 1024, 0, st>>>(
                static_cast<const int64_t*>(counts), static_cast<int>(N), static_cast<int>(E), A, hdr, dst_first,
                src_first, static_cast<int64_t*>(expert_token_num)); w8a8::note_launch();
        }
    } else if (count_bytes == 4) {
        w8a8::rr_table_kernel<int32_t><<<1, 1024, 0, st>>>(static_cast<const int32_t*>(counts), N, E, A, hdr,
                                                          dst_first, src_first, col_start, row_start,
                                                          static_cast<int32_t*>(expert_token_num)); w8a8::note_launch();
    } else {
        w8a8::rr_table_kernel<int64_t><<<1, 1024, 0, st>>>(static_cast<const int64_t*>(counts), N, E, A, hdr,
                                                          dst_first, src_first, col_start, row_start,
                                                          static_cast<int64_t*>(expert_token_num)); w8a8::note_launch();
    }
    if (cudaGetLastError() != cudaSuccess) {
        return W8A8_ERR_CUDA;
    }
    if (A == 0) {
        return W8A8_OK;
    }
    const unsigned blocks = static_cast<unsigned>((A + 255) / 256);
    w8a8::rr_index_kernel<<<blocks, 256, 0, st>>>(hdr, dst_first, src_first, static_cast<int64_t>(cells), A, index,
                                                  out_idx); w8a8::note_launch();
    if (cudaGetLastError() != cudaSuccess) {
        return W8A8_ERR_CUDA;
    }
    return w8a8_permute_rows(tokens, scales, out_tokens, (scales != nullptr) ? out_scales : nullptr, index, A,
                             row_bytes, stream);
}

template <int DT>
static int launch_mfr(const void* rows, const int32_t* esdr, const void* skip1, const void* skip2, const void* bias,
                      const void* scales, const int32_t* expert, void* out, int64_t R, int64_t H, int64_t K, int64_t E,
                      int64_t num_dst, int col_mode, int scale_dt, bool vec, cudaStream_t st)
{
    const int64_t cap = static_cast<int64_t>(w8a8::sm_count()) * 8;
    const unsigned grid = static_cast<unsigned>(R < cap ? R : cap);
    const bool has_bias = (bias != nullptr) && (expert != nullptr);
    auto kern = vec ? (has_bias ? w8a8::mfr_kernel<DT, true, true, int32_t> : w8a8::mfr_kernel<DT, true, false, int32_t>)
                    : (has_bias ? w8a8::mfr_kernel<DT, false, true, int32_t>
                                : w8a8::mfr_kernel<DT, false, false, int32_t>);
    kern<<<grid, 256, 0, st>>>(rows, esdr, skip1, skip2, bias, scales, expert, out, R, H, static_cast<int>(K), E,
                               num_dst, col_mode, scale_dt); w8a8::note_launch();
    return (cudaGetLastError() == cudaSuccess) ? W8A8_OK : W8A8_ERR_CUDA;
}

extern "C" int w8a8_moe_finalize_routing(const void* rows, const int32_t* src_to_dst_row, const void* skip1,
                                         const void* skip2, const void* bias, const void* scales,
                                         const int32_t* expert_for_source_row, void* out, int64_t num_rows, int64_t H,
                                         int64_t K, int64_t E, int64_t num_dst, int drop_pad_mode, int dtype,
                                         int scale_dtype, void* stream)
{
    if (dtype != W8A8_DT_F16 && dtype != W8A8_DT_BF16 && dtype != W8A8_DT_F32) {
        return W8A8_ERR_INVALID;
    }
    if (scales != nullptr && scale_dtype != W8A8_DT_F16 && scale_dtype != W8A8_DT_BF16 &&
        scale_dtype != W8A8_DT_F32) {
        return W8A8_ERR_INVALID;
    }
    if (num_rows < 0 || H <= 0 || K <= 0 || E < 0 || num_dst < 0) {
        return W8A8_ERR_INVALID;
    }
    if (K > w8a8::MFR_MAX_STAGED_K && dtype != W8A8_DT_F32) {
        return W8A8_ERR_LIMIT;  // a 16-bit output cannot carry the fp32 partial sum between passes
    }
    if (num_rows == 0) {
        return W8A8_OK;
    }
    if (rows == nullptr || src_to_dst_row == nullptr || out == nullptr) {
        return W8A8_ERR_INVALID;
    }
    const size_t elem = (dtype == W8A8_DT_F32) ? 4 : 2;
    const void* ptrs[5] = {rows, skip1, skip2, bias, out};
    bool vec = (H * static_cast<int64_t>(elem)) % 16 == 0;
    for (const void* q : ptrs) {
        if (q != nullptr && !w8a8::is_aligned(q, elem)) {
            return W8A8_ERR_ALIGN;
        }
        vec = vec && (q == nullptr || w8a8::is_aligned(q, 16));
    }
    const int col_mode = (drop_pad_mode <= 1) ? 1 : 0;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    switch (dtype) {
    case W8A8_DT_F16:
        return launch_mfr<W8A8_DT_F16>(rows, src_to_dst_row, skip1, skip2, bias, scales, expert_for_source_row, out,
                                       num_rows, H, K, E, num_dst, col_mode, scale_dtype, vec, st);
    case W8A8_DT_BF16:
        return launch_mfr<W8A8_DT_BF16>(rows, src_to_dst_row, skip1, skip2, bias, scales, expert_for_source_row, out,
                                        num_rows, H, K, E, num_dst, col_mode, scale_dtype, vec, st);
    default:
        return launch_mfr<W8A8_DT_F32>(rows, src_to_dst_row, skip1, skip2, bias, scales, expert_for_source_row, out,
                                       num_rows, H, K, E, num_dst, col_mode, scale_dtype, vec, st);
    }
}

extern "C" int w8a8_ep_tables(const int64_t* counts, int64_t P, int64_t E, int64_t rank, const uint64_t* peer_base,
                              uint64_t off_x, uint64_t off_s, uint64_t off_back, int64_t row_bytes,
                              int64_t back_row_bytes, int64_t cap_rows, uint64_t* row_dst, uint64_t* scale_dst,
                              int64_t* my_base, int64_t* group_list, int64_t* seg_first, uint64_t* seg_ptr,
                              int32_t* status, void* stream)
{
    if (P <= 0 || E <= 0 || E % P != 0 || rank < 0 || rank >= P || row_bytes <= 0 || back_row_bytes <= 0 ||
        cap_rows < 0) {
        return W8A8_ERR_INVALID;
    }
    if (P > w8a8::EP_MAX_RANKS || E > 1024 || P * E > w8a8::EP_MAX_CELLS) {
        return W8A8_ERR_LIMIT;
    }
    if (counts == nullptr || peer_base == nullptr || row_dst == nullptr || scale_dst == nullptr ||
        my_base == nullptr || group_list == nullptr || seg_first == nullptr || seg_ptr == nullptr ||
        status == nullptr) {
        return W8A8_ERR_INVALID;
    }
    w8a8::ep_tables_kernel<<<1, 1024, 0, static_cast<cudaStream_t>(stream)>>>(
        counts, static_cast<int>(P), static_cast<int>(E), static_cast<int>(rank), peer_base, off_x, off_s, off_back,
        row_bytes, back_row_bytes, cap_rows, row_dst, scale_dst, my_base, group_list, seg_first, seg_ptr, status); w8a8::note_launch();
    return (cudaGetLastError() == cudaSuccess) ? W8A8_OK : W8A8_ERR_CUDA;
}
