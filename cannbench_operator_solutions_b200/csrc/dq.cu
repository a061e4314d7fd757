// DynamicQuant for sm_100a: per-row absmax int8 quantisation, one HBM pass.
//
// Arithmetic follows operators/dynamicquant/csrc/ops/dynamic_quant/op_kernel/
// dynamic_quant_kernel.cpp of the reference catalog: row maximum of |x|
// (:203-239), clamp at 1e-12 (:240), scale = amax * (1/127) (:249),
// inv = (1/amax) * 127 (:256-257), y = x * inv (:260-276), fp32 -> fp16 ->
// int8 with round-to-nearest-even twice (:279-282).
//
// Mapping: one CTA per row at a time (grid-stride over rows).  Thread t owns
// the 16-byte chunks t, t+T, ... of the row and keeps them in registers
// between the reduction and the quantisation, so x is read once and y
// written once.  The row maximum is taken on the raw 16-bit patterns
// (|x| as an unsigned integer), which needs no conversion and propagates
// NaN; a warp `redux` plus one shared-memory exchange finishes it.
#include "common.cuh"

namespace w8a8 {

template <int DT, int THREADS, int CPT, bool VEC, bool DIRECT>
__global__ void __launch_bounds__(THREADS) dq_rows_kernel(const uint16_t* __restrict__ x, int8_t* __restrict__ y,
                                                          float* __restrict__ scale, int64_t M, int64_t N)
{
    constexpr int WARPS = THREADS / 32;
    __shared__ uint32_t s_max[2][WARPS];
    const int tid = threadIdx.x;
    const int nchunks = static_cast<int>((N + 7) / 8);
    int parity = 0;
    for (int64_t row = blockIdx.x; row < M; row += gridDim.x, parity ^= 1) {
        const uint16_t* xr = x + row * N;
        uint4 v[CPT];
        uint32_t m2 = 0;
#pragma unroll
        for (int i = 0; i < CPT; ++i) {
            const int c = tid + i * THREADS;
            v[i] = (c < nchunks) ? load_chunk16<VEC>(xr, c, N) : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int i = 0; i < CPT; ++i) {
            m2 = chunk_absmax16(v[i], m2);
        }
        uint32_t m = max(m2 & 0xffffu, m2 >> 16);
        m = __reduce_max_sync(FULL_MASK, m);
        if ((tid & 31) == 0) {
            s_max[parity][tid >> 5] = m;
        }
        __syncthreads();
#pragma unroll
        for (int w = 0; w < WARPS; ++w) {
            m = max(m, s_max[parity][w]);
        }
        float amax = bits16_to_float<DT>(m);
        if (amax < 1e-12f) {
            amax = 1e-12f;
        }
        if (tid == 0) {
            scale[row] = __fmul_rn(amax, INV127);
        }
        const float inv = __fmul_rn(__frcp_rn(amax), 127.0f);
        int8_t* yr = y + row * N;
        // inv is a finite positive number unless the row held inf or NaN;
        // then every product is 0 or NaN and the row quantises to zeros.
        const bool regular = (__float_as_uint(amax) < 0x7f800000u);
#pragma unroll
        for (int i = 0; i < CPT; ++i) {
            const int c = tid + i * THREADS;
            if (c < nchunks) {
                uint32_t lo = 0, hi = 0;
                if (regular) {
                    float f[8];
                    unpack2<DT>(v[i].x, f[0], f[1]);
                    unpack2<DT>(v[i].y, f[2], f[3]);
                    unpack2<DT>(v[i].z, f[4], f[5]);
                    unpack2<DT>(v[i].w, f[6], f[7]);
                    lo = narrow4_fast<DIRECT>(__fmul_rn(f[0], inv), __fmul_rn(f[1], inv), __fmul_rn(f[2], inv),
                                              __fmul_rn(f[3], inv));
                    hi = narrow4_fast<DIRECT>(__fmul_rn(f[4], inv), __fmul_rn(f[5], inv), __fmul_rn(f[6], inv),
                                              __fmul_rn(f[7], inv));
                }
                store_chunk8<VEC>(yr, c, N, lo, hi);
            }
        }
    }
}

// Rows longer than the register-resident kernels cover: two passes over the
// row (the second one normally hits L2), same arithmetic.
template <int DT, bool DIRECT>
__global__ void __launch_bounds__(1024) dq_long_rows_kernel(const uint16_t* __restrict__ x, int8_t* __restrict__ y,
                                                            float* __restrict__ scale, int64_t M, int64_t N)
{
    __shared__ uint32_t s_max[2][32];
    const int tid = threadIdx.x;
    int parity = 0;
    for (int64_t row = blockIdx.x; row < M; row += gridDim.x, parity ^= 1) {
        const uint16_t* xr = x + row * N;
        uint32_t m = 0;
        for (int64_t j = tid; j < N; j += 1024) {
            m = max(m, static_cast<uint32_t>(xr[j]) & 0x7fffu);
        }
        m = __reduce_max_sync(FULL_MASK, m);
        if ((tid & 31) == 0) {
            s_max[parity][tid >> 5] = m;
        }
        __syncthreads();
        for (int w = 0; w < 32; ++w) {
            m = max(m, s_max[parity][w]);
        }
        float amax = bits16_to_float<DT>(m);
        if (amax < 1e-12f) {
            amax = 1e-12f;
        }
        if (tid == 0) {
            scale[row] = __fmul_rn(amax, INV127);
        }
        const float inv = __fmul_rn(__frcp_rn(amax), 127.0f);
        int8_t* yr = y + row * N;
        for (int64_t j = tid; j < N; j += 1024) {
            const float v = __fmul_rn(bits16_to_float<DT>(xr[j]), inv);
            yr[j] = static_cast<int8_t>(narrow1_general<DIRECT>(v));
        }
    }
}

template <int DT, int THREADS, int CPT, bool VEC, bool DIRECT>
static cudaError_t launch_rows(const void* x, int8_t* y, float* scale, int64_t M, int64_t N, cudaStream_t st)
{
    auto kern = dq_rows_kernel<DT, THREADS, CPT, VEC, DIRECT>;
    int per_sm = 1;
    cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, THREADS, 0);
    if (e != cudaSuccess) {
        return e;
    }
    if (per_sm < 1) {
        per_sm = 1;
    }
    const int64_t cap = static_cast<int64_t>(sm_count()) * per_sm;
    const unsigned grid = static_cast<unsigned>(M < cap ? M : cap);
    kern<<<grid, THREADS, 0, st>>>(static_cast<const uint16_t*>(x), y, scale, M, N); w8a8::note_launch();
    return cudaGetLastError();
}

template <int DT, bool VEC, bool DIRECT>
static cudaError_t dispatch_cpt(const void* x, int8_t* y, float* scale, int64_t M, int64_t N, cudaStream_t st)
{
    const int64_t chunks = (N + 7) / 8;
    if (chunks <= 128) {
        return launch_rows<DT, 128, 1, VEC, DIRECT>(x, y, scale, M, N, st);
    }
    if (chunks <= 256) {
        return launch_rows<DT, 256, 1, VEC, DIRECT>(x, y, scale, M, N, st);
    }
    if (chunks <= 512) {
        return launch_rows<DT, 256, 2, VEC, DIRECT>(x, y, scale, M, N, st);
    }
    if (chunks <= 1024) {
        return launch_rows<DT, 256, 4, VEC, DIRECT>(x, y, scale, M, N, st);
    }
    if (chunks <= 2048) {
        return launch_rows<DT, 256, 8, VEC, DIRECT>(x, y, scale, M, N, st);
    }
    if (chunks <= 8192) {
        return launch_rows<DT, 1024, 8, VEC, DIRECT>(x, y, scale, M, N, st);
    }
    const int64_t cap = static_cast<int64_t>(sm_count()) * 2;
    const unsigned grid = static_cast<unsigned>(M < cap ? M : cap);
    dq_long_rows_kernel<DT, DIRECT><<<grid, 1024, 0, st>>>(static_cast<const uint16_t*>(x), y, scale, M, N); w8a8::note_launch();
    return cudaGetLastError();
}

template <int DT>
static cudaError_t dispatch(const void* x, int8_t* y, float* scale, int64_t M, int64_t N, bool vec, bool direct,
                            cudaStream_t st)
{
    if (vec) {
        return direct ? dispatch_cpt<DT, true, true>(x, y, scale, M, N, st)
                      : dispatch_cpt<DT, true, false>(x, y, scale, M, N, st);
    }
    return direct ? dispatch_cpt<DT, false, true>(x, y, scale, M, N, st)
                  : dispatch_cpt<DT, false, false>(x, y, scale, M, N, st);
}

}  // namespace w8a8

extern "C" int w8a8_dynamic_quant(const void* x, int8_t* y, float* scale, int64_t M, int64_t N, int dtype, int flags,
                                  void* stream)
{
    if (dtype != W8A8_DT_F16 && dtype != W8A8_DT_BF16) {
        return W8A8_ERR_INVALID;
    }
    if (M < 0 || N <= 0 || (flags & ~W8A8_F_ROUND_DIRECT) != 0) {
        return W8A8_ERR_INVALID;
    }
    if (M == 0) {
        return W8A8_OK;
    }
    if (x == nullptr || y == nullptr || scale == nullptr) {
        return W8A8_ERR_INVALID;
    }
    if (!w8a8::is_aligned(x, 2) || !w8a8::is_aligned(scale, 4)) {
        return W8A8_ERR_ALIGN;
    }
    const bool vec = (N % 8 == 0) && w8a8::is_aligned(x, 16) && w8a8::is_aligned(y, 8);
    const bool direct = (flags & W8A8_F_ROUND_DIRECT) != 0;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const cudaError_t e = (dtype == W8A8_DT_BF16)
                              ? w8a8::dispatch<W8A8_DT_BF16>(x, y, scale, M, N, vec, direct, st)
                              : w8a8::dispatch<W8A8_DT_F16>(x, y, scale, M, N, vec, direct, st);
    return (e == cudaSuccess) ? W8A8_OK : W8A8_ERR_CUDA;
}
