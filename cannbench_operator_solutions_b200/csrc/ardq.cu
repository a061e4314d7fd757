// AddRmsNormDynamicQuant for sm_100a: residual add + RMSNorm + per-row absmax
// int8 quantisation in one HBM pass (two reads, three writes per element).
//
// Arithmetic follows operators/addrmsnormdynamicquant/csrc/ops/
// add_rms_norm_dynamic_quant/op_kernel/add_rms_norm_dynamic_quant_kernel.cpp
// of the reference catalog: fp32 add (:232-247), xOut rounded to the storage
// type only for the store (:251-265), z = xOut * gamma (:268-270), sum of
// squares and max|z| (:275-278), mean = sum * (1/N), + eps, sqrt (:280-282),
// rstd = 1/rms, m = maxAbs * rstd, clamp at 1e-12 only when m < 1e-12,
// scale = m * (1/127), k = rstd / scale (:286-298), y = narrow(z * k)
// (:308-314).
//
// Reduction order (the definition the CPU oracle shares): 256 lanes; lane t
// owns the 8-element chunks t, t+256, ... and folds their squares in element
// order with fmaf; lanes combine inside each warp by an xor butterfly
// (16, 8, 4, 2, 1) and the eight warp sums are added left to right.
//
// Mapping: one 256-thread CTA per row at a time; the row's z values stay in
// registers between the reductions and the quantisation.
#include "common.cuh"

namespace w8a8 {

constexpr int ARDQ_THREADS = 256;

template <int DT, int CPT, bool VEC, bool DIRECT>
__global__ void __launch_bounds__(ARDQ_THREADS)
    ardq_rows_kernel(const uint16_t* __restrict__ x1, const uint16_t* __restrict__ x2,
                     const uint16_t* __restrict__ gamma, int8_t* __restrict__ y, uint16_t* __restrict__ x_out,
                     float* __restrict__ scale_out, int64_t rows, int64_t N, float eps, float inv_n)
{
    constexpr int WARPS = ARDQ_THREADS / 32;
    __shared__ float s_sum[2][WARPS];
    __shared__ uint32_t s_max[2][WARPS];
    const int tid = threadIdx.x;
    const int nchunks = static_cast<int>((N + 7) / 8);
    int parity = 0;
    for (int64_t row = blockIdx.x; row < rows; row += gridDim.x, parity ^= 1) {
        const uint16_t* r1 = x1 + row * N;
        const uint16_t* r2 = x2 + row * N;
        uint16_t* ro = x_out + row * N;
        uint4 a[CPT], b[CPT];
#pragma unroll
        for (int i = 0; i < CPT; ++i) {
            const int c = tid + i * ARDQ_THREADS;
            const bool in = c < nchunks;
            a[i] = in ? load_chunk16<VEC>(r1, c, N) : make_uint4(0, 0, 0, 0);
            b[i] = in ? load_chunk16<VEC>(r2, c, N) : make_uint4(0, 0, 0, 0);
        }
        float z[CPT][8];
        float acc = 0.0f;
        uint32_t mb = 0;
#pragma unroll
        for (int i = 0; i < CPT; ++i) {
            const int c = tid + i * ARDQ_THREADS;
            if (c < nchunks) {
                const uint4 g = load_chunk16_cached<VEC>(gamma, c, N);
                const uint32_t aw[4] = {a[i].x, a[i].y, a[i].z, a[i].w};
                const uint32_t bw[4] = {b[i].x, b[i].y, b[i].z, b[i].w};
                const uint32_t gw[4] = {g.x, g.y, g.z, g.w};
                uint32_t ow[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    float a0, a1, b0, b1, g0, g1;
                    unpack2<DT>(aw[j], a0, a1);
                    unpack2<DT>(bw[j], b0, b1);
                    unpack2<DT>(gw[j], g0, g1);
                    const float s0 = __fadd_rn(a0, b0);
                    const float s1 = __fadd_rn(a1, b1);
                    ow[j] = pack2<DT>(s0, s1);
                    acc = fmaf(s0, s0, acc);
                    acc = fmaf(s1, s1, acc);
                    const float z0 = __fmul_rn(s0, g0);
                    const float z1 = __fmul_rn(s1, g1);
                    z[i][2 * j] = z0;
                    z[i][2 * j + 1] = z1;
                    mb = max(mb, __float_as_uint(z0) & 0x7fffffffu);
                    mb = max(mb, __float_as_uint(z1) & 0x7fffffffu);
                }
                store_chunk16<VEC>(ro, c, N, make_uint4(ow[0], ow[1], ow[2], ow[3]));
            } else {
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    z[i][j] = 0.0f;
                }
            }
        }
        // warp butterfly for the sum, redux for the maximum
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1) {
            acc = __fadd_rn(acc, __shfl_xor_sync(FULL_MASK, acc, off));
        }
        mb = __reduce_max_sync(FULL_MASK, mb);
        if ((tid & 31) == 0) {
            s_sum[parity][tid >> 5] = acc;
            s_max[parity][tid >> 5] = mb;
        }
        __syncthreads();
        float sum = s_sum[parity][0];
#pragma unroll
        for (int w = 1; w < WARPS; ++w) {
            sum = __fadd_rn(sum, s_sum[parity][w]);
        }
#pragma unroll
        for (int w = 0; w < WARPS; ++w) {
            mb = max(mb, s_max[parity][w]);
        }
        const float mean = __fmul_rn(sum, inv_n);
        const float rms = __fsqrt_rn(__fadd_rn(mean, eps));
        const float max_abs = __uint_as_float(mb);
        const float rstd = __frcp_rn(rms);
        const float m = __fmul_rn(max_abs, rstd);
        const float sm = (m < 1e-12f) ? 1e-12f : m;
        const float sc = __fmul_rn(sm, INV127);
        const float k = __fdiv_rn(rstd, sc);
        if (tid == 0) {
            scale_out[row] = sc;
        }
        // k finite and non-zero implies every z is finite and |z*k| <= 127(1+ulp):
        // the conversion-free narrowing applies.  Otherwise (inf / NaN rows,
        // eps == 0 on an all-zero row) take the general narrowing.
        const uint32_t kb = __float_as_uint(k) & 0x7fffffffu;
        const bool regular = (kb != 0u) && (kb < 0x7f800000u);
        int8_t* yr = y + row * N;
#pragma unroll
        for (int i = 0; i < CPT; ++i) {
            const int c = tid + i * ARDQ_THREADS;
            if (c < nchunks) {
                float q[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    q[j] = __fmul_rn(z[i][j], k);
                }
                uint32_t lo, hi;
                if (regular) {
                    lo = narrow4_fast<DIRECT>(q[0], q[1], q[2], q[3]);
                    hi = narrow4_fast<DIRECT>(q[4], q[5], q[6], q[7]);
                } else {
                    lo = narrow4_general<DIRECT>(q[0], q[1], q[2], q[3]);
                    hi = narrow4_general<DIRECT>(q[4], q[5], q[6], q[7]);
                }
                store_chunk8<VEC>(yr, c, N, lo, hi);
            }
        }
    }
}

template <int DT, int CPT, bool VEC, bool DIRECT>
static cudaError_t launch(const void* x1, const void* x2, const void* gamma, int8_t* y, void* x_out, float* scale_out,
                          int64_t rows, int64_t N, float eps, cudaStream_t st)
{
    auto kern = ardq_rows_kernel<DT, CPT, VEC, DIRECT>;
    int per_sm = 1;
    cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, ARDQ_THREADS, 0);
    if (e != cudaSuccess) {
        return e;
    }
    if (per_sm < 1) {
        per_sm = 1;
    }
    const int64_t cap = static_cast<int64_t>(sm_count()) * per_sm;
    const unsigned grid = static_cast<unsigned>(rows < cap ? rows : cap);
    const float inv_n = 1.0f / static_cast<float>(N);
    kern<<<grid, ARDQ_THREADS, 0, st>>>(static_cast<const uint16_t*>(x1), static_cast<const uint16_t*>(x2),
                                        static_cast<const uint16_t*>(gamma), y, static_cast<uint16_t*>(x_out),
                                        scale_out, rows, N, eps, inv_n); w8a8::note_launch();
    return cudaGetLastError();
}

template <int DT, bool VEC, bool DIRECT>
static cudaError_t dispatch_cpt(const void* x1, const void* x2, const void* gamma, int8_t* y, void* x_out,
                                float* scale_out, int64_t rows, int64_t N, float eps, cudaStream_t st)
{
    const int64_t chunks = (N + 7) / 8;
    if (chunks <= 256) {
        return launch<DT, 1, VEC, DIRECT>(x1, x2, gamma, y, x_out, scale_out, rows, N, eps, st);
    }
    if (chunks <= 512) {
        return launch<DT, 2, VEC, DIRECT>(x1, x2, gamma, y, x_out, scale_out, rows, N, eps, st);
    }
    if (chunks <= 1024) {
        return launch<DT, 4, VEC, DIRECT>(x1, x2, gamma, y, x_out, scale_out, rows, N, eps, st);
    }
    return launch<DT, 8, VEC, DIRECT>(x1, x2, gamma, y, x_out, scale_out, rows, N, eps, st);
}

template <int DT>
static cudaError_t dispatch(const void* x1, const void* x2, const void* gamma, int8_t* y, void* x_out,
                            float* scale_out, int64_t rows, int64_t N, float eps, bool vec, bool direct,
                            cudaStream_t st)
{
    if (vec) {
        return direct ? dispatch_cpt<DT, true, true>(x1, x2, gamma, y, x_out, scale_out, rows, N, eps, st)
                      : dispatch_cpt<DT, true, false>(x1, x2, gamma, y, x_out, scale_out, rows, N, eps, st);
    }
    return direct ? dispatch_cpt<DT, false, true>(x1, x2, gamma, y, x_out, scale_out, rows, N, eps, st)
                  : dispatch_cpt<DT, false, false>(x1, x2, gamma, y, x_out, scale_out, rows, N, eps, st);
}

}  // namespace w8a8

extern "C" int w8a8_add_rms_norm_dynamic_quant(const void* x1, const void* x2, const void* gamma, int8_t* y,
                                               void* x_out, float* scale_out, int64_t rows, int64_t N, float epsilon,
                                               int dtype, int flags, void* stream)
{
    if (dtype != W8A8_DT_F16 && dtype != W8A8_DT_BF16) {
        return W8A8_ERR_INVALID;
    }
    // the reference rejects rows longer than 16384
    // (add_rms_norm_dynamic_quant_plugin.cpp:82)
    if (rows < 0 || N <= 0 || N > 16384 || (flags & ~W8A8_F_ROUND_DIRECT) != 0) {
        return W8A8_ERR_INVALID;
    }
    if (rows == 0) {
        return W8A8_OK;
    }
    if (x1 == nullptr || x2 == nullptr || gamma == nullptr || y == nullptr || x_out == nullptr ||
        scale_out == nullptr) {
        return W8A8_ERR_INVALID;
    }
    if (!w8a8::is_aligned(x1, 2) || !w8a8::is_aligned(x2, 2) || !w8a8::is_aligned(gamma, 2) ||
        !w8a8::is_aligned(x_out, 2) || !w8a8::is_aligned(scale_out, 4)) {
        return W8A8_ERR_ALIGN;
    }
    const bool vec = (N % 8 == 0) && w8a8::is_aligned(x1, 16) && w8a8::is_aligned(x2, 16) &&
                     w8a8::is_aligned(gamma, 16) && w8a8::is_aligned(x_out, 16) && w8a8::is_aligned(y, 8);
    const bool direct = (flags & W8A8_F_ROUND_DIRECT) != 0;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const cudaError_t e =
        (dtype == W8A8_DT_BF16)
            ? w8a8::dispatch<W8A8_DT_BF16>(x1, x2, gamma, y, x_out, scale_out, rows, N, epsilon, vec, direct, st)
            : w8a8::dispatch<W8A8_DT_F16>(x1, x2, gamma, y, x_out, scale_out, rows, N, epsilon, vec, direct, st);
    return (e == cudaSuccess) ? W8A8_OK : W8A8_ERR_CUDA;
}
