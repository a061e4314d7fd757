// MoeGatingTopKSoftmax for sm_100a: per-row softmax over the experts, the k largest probabilities with their
// expert indices, and the flattened row index j * rows + r.
//
// Arithmetic follows operators/moegatingtopksoftmax/csrc/ops/moe_gating_top_k_softmax/op_kernel/
// moe_gating_kernel.cpp of the reference catalog: everything in fp32 (:28), row maximum (:305-312), x - max
// (:327), exp (:329), row sum (:333-339), descending sort of the exponentials with their indices (:344-368),
// division of the selected values by the row sum (:390), round-to-nearest-even cast to the input type (:392);
// a finished row reports `inner` as every expert index and keeps y and row_idx (:21, :285-300).
//
// Two choices the reference leaves to its hardware are fixed here and shared bit for bit with the CPU oracle:
// exp is the canonical fp32 sequence of common.cuh, and the row sum is taken in a 32-lane order (lane t adds
// elements t, t+32, ... in ascending order, then a butterfly over lane distances 16, 8, 4, 2, 1).  Equal
// exponentials are ordered by ascending expert index.
//
// Mapping: one warp per row, the row held in registers (lane t owns elements t + 32 v).  Each lane ranks its own
// elements once (larger exponential first, equal ones by ascending index) and parks them in that order in shared
// memory; the k selections are then k rounds of "largest head of the 32 lists" - two `redux.sync`, one 8-byte
// shared-memory load and a counter per round - instead of a scan of the lane's elements per round.  The operator
// moves rows * inner input elements and 10 k bytes of output per row; at router sizes (inner <= 1024) it is bound
// by the exp arithmetic, not by HBM.
#include "common.cuh"

namespace w8a8 {

template <int DT>
__device__ __forceinline__ float gating_load(const void* x, int64_t i)
{
    if constexpr (DT == W8A8_DT_F32) {
        return static_cast<const float*>(x)[i];
    } else {
        return bits16_to_float<DT>(static_cast<const uint16_t*>(x)[i]);
    }
}

template <int DT>
__device__ __forceinline__ void gating_store(void* y, int64_t i, float v)
{
    if constexpr (DT == W8A8_DT_F32) {
        static_cast<float*>(y)[i] = v;
    } else {
        static_cast<uint16_t*>(y)[i] = float_to_bits16<DT>(v);
    }
}

constexpr int GATING_WARPS = 4;

// FULL: inner == 32 * VPT, so no element needs a bounds check.
template <int DT, int VPT, bool FULL>
__global__ void __launch_bounds__(GATING_WARPS * 32) gating_kernel(const void* __restrict__ x,
                                                                   const uint8_t* __restrict__ finished,
                                                                   void* __restrict__ y,
                                                                   int32_t* __restrict__ expert_idx,
                                                                   int32_t* __restrict__ row_idx, int64_t rows,
                                                                   int inner, int k)
{
    __shared__ int2 lists[GATING_WARPS][(VPT + 1) * 32];
    const int lane = threadIdx.x & 31;
    int2* list = lists[threadIdx.x >> 5];
    const int64_t warps = static_cast<int64_t>(gridDim.x) * GATING_WARPS;
    for (int64_t r = static_cast<int64_t>(blockIdx.x) * GATING_WARPS + (threadIdx.x >> 5); r < rows; r += warps) {
        float v[VPT];
        float m = -INFINITY;
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            const int c = lane + 32 * i;
            v[i] = (FULL || c < inner) ? gating_load<DT>(x, r * inner + c) : -INFINITY;
            m = fmaxf(m, v[i]);
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
            m = fmaxf(m, __shfl_xor_sync(FULL_MASK, m, off));
        }
        float s = 0.0f;
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            const int c = lane + 32 * i;
            if (FULL || c < inner) {
                v[i] = canonical_expf(__fsub_rn(v[i], m));
                s = __fadd_rn(s, v[i]);
            } else {
                v[i] = -1.0f;  // below every exponential: never selected
            }
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
            s = __fadd_rn(s, __shfl_xor_sync(FULL_MASK, s, off));
        }
        const bool fin = (finished != nullptr) && (finished[r] != 0);
        // Selection keys: exponentials are >= 0, so their bit patterns order like integers; what can never be
        // selected (a NaN, which fmaxf drops, and the padding past `inner`) gets the bits of -1, a negative integer.
        int key[VPT];
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            key[i] = __float_as_int(fmaxf(v[i], -1.0f));
        }
        // position of each element in the lane's own order: larger key first, equal keys by ascending i
        int pos[VPT];
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            pos[i] = 0;
        }
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
#pragma unroll
            for (int j = i + 1; j < VPT; ++j) {
                const bool first = key[i] >= key[j];  // i stays in front of j
                pos[j] += first ? 1 : 0;
                pos[i] += first ? 0 : 1;
            }
        }
        // list[p * 32 + lane] = the lane's p-th element as (key, expert index); one more entry that ends the list
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            list[pos[i] * 32 + lane] = make_int2(key[i], lane + 32 * i);
        }
        list[VPT * 32 + lane] = make_int2(-1, 0);
        // Lane j keeps the j-th selection and the lanes store together after every 32 rounds: one division and one
        // store instruction per 32 results instead of one per result.
        int keep_top = -1;
        int keep_win = 0;
        int taken = 0;  // how many of this lane's elements have been selected
        for (int j = 0; j < k; ++j) {
            const int2 head = list[taken * 32 + lane];
            const int top = __reduce_max_sync(FULL_MASK, head.x);
            // the largest exponential, and among equal ones the smallest expert index; with nothing selectable left
            // (only after NaNs) the result is a NaN with index 0
            const unsigned cand = (head.x == top && top >= 0) ? static_cast<unsigned>(head.y) : 0xffffffffu;
            const unsigned win = __reduce_min_sync(FULL_MASK, cand);
            taken += (cand == win && top >= 0) ? 1 : 0;
            if (lane == (j & 31)) {
                keep_top = top;
                keep_win = (top >= 0) ? static_cast<int>(win) : 0;
            }
            if ((j & 31) == 31 || j == k - 1) {
                const int jj = (j & ~31) + lane;  // the round this lane holds
                if (jj <= j) {
                    const float e = (keep_top >= 0) ? __int_as_float(keep_top) : NAN;
                    const int64_t o = r * k + jj;
                    gating_store<DT>(y, o, __fdiv_rn(e, s));
                    expert_idx[o] = fin ? inner : keep_win;
                    row_idx[o] = static_cast<int32_t>(static_cast<int64_t>(jj) * rows + r);
                }
            }
        }
    }
}

template <int DT, int VPT>
static cudaError_t launch_gating(const void* x, const uint8_t* finished, void* y, int32_t* expert_idx,
                                 int32_t* row_idx, int64_t rows, int inner, int k, cudaStream_t st)
{
    const int64_t want = (rows + GATING_WARPS - 1) / GATING_WARPS;
    const int64_t cap = static_cast<int64_t>(sm_count()) * 16;
    const unsigned grid = static_cast<unsigned>(want < cap ? want : cap);
    if (inner == 32 * VPT) {
        gating_kernel<DT, VPT, true><<<grid, GATING_WARPS * 32, 0, st>>>(x, finished, y, expert_idx, row_idx, rows, inner, k);
    } else {
        gating_kernel<DT, VPT, false><<<grid, GATING_WARPS * 32, 0, st>>>(x, finished, y, expert_idx, row_idx, rows, inner, k);
    }
    w8a8::note_launch();
    return cudaGetLastError();
}

template <int DT>
static cudaError_t dispatch_gating(const void* x, const uint8_t* finished, void* y, int32_t* expert_idx,
                                   int32_t* row_idx, int64_t rows, int inner, int k, cudaStream_t st)
{
    if (inner <= 32) {
        return launch_gating<DT, 1>(x, finished, y, expert_idx, row_idx, rows, inner, k, st);
    }
    if (inner <= 64) {
        return launch_gating<DT, 2>(x, finished, y, expert_idx, row_idx, rows, inner, k, st);
    }
    if (inner <= 128) {
        return launch_gating<DT, 4>(x, finished, y, expert_idx, row_idx, rows, inner, k, st);
    }
    if (inner <= 256) {
        return launch_gating<DT, 8>(x, finished, y, expert_idx, row_idx, rows, inner, k, st);
    }
    if (inner <= 512) {
        return launch_gating<DT, 16>(x, finished, y, expert_idx, row_idx, rows, inner, k, st);
    }
    return launch_gating<DT, 32>(x, finished, y, expert_idx, row_idx, rows, inner, k, st);
}

}  // namespace w8a8

extern "C" int w8a8_moe_gating_top_k_softmax(const void* x, const uint8_t* finished, void* y, int32_t* expert_idx,
                                             int32_t* row_idx, int64_t rows, int64_t inner, int64_t k, int dtype,
                                             void* stream)
{
    if (dtype != W8A8_DT_F16 && dtype != W8A8_DT_BF16 && dtype != W8A8_DT_F32) {
        return W8A8_ERR_INVALID;
    }
    if (rows < 0 || inner <= 0 || k <= 0 || k > inner) {
        return W8A8_ERR_INVALID;
    }
    if (inner > W8A8_GATING_MAX_EXPERTS || rows * k > INT32_MAX) {
        return W8A8_ERR_LIMIT;
    }
    if (rows == 0) {
        return W8A8_OK;
    }
    if (x == nullptr || y == nullptr || expert_idx == nullptr || row_idx == nullptr) {
        return W8A8_ERR_INVALID;
    }
    const size_t elem = (dtype == W8A8_DT_F32) ? 4 : 2;
    if (!w8a8::is_aligned(x, elem) || !w8a8::is_aligned(y, elem)) {
        return W8A8_ERR_ALIGN;
    }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int in = static_cast<int>(inner), kk = static_cast<int>(k);
    cudaError_t e;
    switch (dtype) {
    case W8A8_DT_F16:
        e = w8a8::dispatch_gating<W8A8_DT_F16>(x, finished, y, expert_idx, row_idx, rows, in, kk, st);
        break;
    case W8A8_DT_BF16:
        e = w8a8::dispatch_gating<W8A8_DT_BF16>(x, finished, y, expert_idx, row_idx, rows, in, kk, st);
        break;
    default:
        e = w8a8::dispatch_gating<W8A8_DT_F32>(x, finished, y, expert_idx, row_idx, rows, in, kk, st);
        break;
    }
    return (e == cudaSuccess) ? W8A8_OK : W8A8_ERR_CUDA;
}
