// DequantSwigluQuant for sm_100a: dequantise a [M, 2H] matmul result, SwiGLU, smooth scale, per-token int8
// quantisation, one HBM pass.
//
// Arithmetic follows operators/dequantswigluquant/csrc/ops/dequant_swiglu_quant/op_kernel/dqsq_kernel.cpp of the
// reference catalog, in the order its vector instructions run:
//   int32 input:  a = float(x[:, :H]) * weight_scale[:H], b = float(x[:, H:]) * weight_scale[H:]   (:335-347)
//   16-bit input: a, b = float(x) halves                                                            (:298-329)
//   quant_scale multiplies the half that is NOT the gate input, before the gate is formed          (:349-363)
//   int32 input:  a *= activation_scale[row], b *= activation_scale[row]                            (:386-410)
//   gate = b (activate_left == 0) or a: out = (a * b) / (1 + exp(gate * -1))                        (:415-428)
//   m = max |out| (not-greater-than-zero, NaN included, counts as 0), s = max(m * (1/127), 1e-12)   (:434-499)
//   y = narrow(clamp(out / s, -128, 127)), fp32 -> fp16 -> int8 with round-to-nearest-even twice    (:509-524)
// The reference scales by out / s in its batched short-row layout (:482) and by out * (1 / s) otherwise
// (:500-504).  Its batched layout needs a padded half-row of at most 1984 elements (:97) and, per tile, fewer
// 64-column chunks than rows (:272), which depends on its on-chip buffer tiling; this build divides when the
// padded half-row is at most 1984 elements long and multiplies by the reciprocal for longer rows, so the two
// can differ by one int8 step on the rare element where the two roundings disagree.  exp is the canonical fp32
// sequence shared with the CPU oracle; a NaN activation quantises to 0.
//
// Mapping: one CTA of 256 threads per row (grid-stride).  Thread t owns 16-byte chunks t, t+256, ... of both
// halves and keeps the fp32 results in registers between the row maximum and the quantisation, so x is read
// once and y written once: 8H + H + 4 bytes per row for int32 input, 4H + H + 4 for 16-bit input.
#include "common.cuh"

namespace w8a8 {

constexpr int DQSQ_X_I32 = 0;
constexpr int DQSQ_X_F16 = 1;
constexpr int DQSQ_X_BF16 = 2;
constexpr int DQSQ_THREADS = 256;

template <int XT>
struct DqsqChunk {
    static constexpr int EL = (XT == DQSQ_X_I32) ? 4 : 8;

    // 16 raw bytes starting at element `first` of the row
    static __device__ __forceinline__ uint4 load_raw(const void* row, int64_t first)
    {
        constexpr size_t ELEM = (XT == DQSQ_X_I32) ? 4 : 2;
        return __ldcs(reinterpret_cast<const uint4*>(static_cast<const uint8_t*>(row) + first * ELEM));
    }

    static __device__ __forceinline__ void unpack(const uint4& v, float (&f)[EL])
    {
        if constexpr (XT == DQSQ_X_I32) {
            f[0] = static_cast<float>(static_cast<int32_t>(v.x)), f[1] = static_cast<float>(static_cast<int32_t>(v.y));
            f[2] = static_cast<float>(static_cast<int32_t>(v.z)), f[3] = static_cast<float>(static_cast<int32_t>(v.w));
        } else {
            constexpr int DT = (XT == DQSQ_X_F16) ? W8A8_DT_F16 : W8A8_DT_BF16;
            unpack2<DT>(v.x, f[0], f[1]);
            unpack2<DT>(v.y, f[2], f[3]);
            unpack2<DT>(v.z, f[4], f[5]);
            unpack2<DT>(v.w, f[6], f[7]);
        }
    }

    static __device__ __forceinline__ float load1(const void* row, int64_t i)
    {
        if constexpr (XT == DQSQ_X_I32) {
            return static_cast<float>(static_cast<const int32_t*>(row)[i]);
        } else if constexpr (XT == DQSQ_X_F16) {
            return bits16_to_float<W8A8_DT_F16>(static_cast<const uint16_t*>(row)[i]);
        } else {
            return bits16_to_float<W8A8_DT_BF16>(static_cast<const uint16_t*>(row)[i]);
        }
    }
};

// one output element, in the reference's operation order
template <int XT>
__device__ __forceinline__ float dqsq_element(float a, float b, float wa, float wb, float qs, float as, bool has_q,
                                              bool left)
{
    if constexpr (XT == DQSQ_X_I32) {
        a = __fmul_rn(a, wa);
        b = __fmul_rn(b, wb);
    }
    if (has_q) {
        if (left) {
            b = __fmul_rn(b, qs);
        } else {
            a = __fmul_rn(a, qs);
        }
    }
    if constexpr (XT == DQSQ_X_I32) {
        a = __fmul_rn(a, as);
        b = __fmul_rn(b, as);
    }
    const float gate = left ? a : b;
    const float den = __fadd_rn(canonical_expf(__fmul_rn(gate, -1.0f)), 1.0f);
    return __fdiv_rn(__fmul_rn(a, b), den);
}

// The same element with the two halves named by role (g: the half the gate is formed from, o: the other one) and the
// smooth scale always applied (1 when the caller gave none; a multiplication by 1 is exact): a * b commutes, and
// gate * -1 is a sign flip, so the bits are those of dqsq_element without its per-element case distinctions.
template <int XT>
__device__ __forceinline__ float dqsq_element_by_role(float g, float o, float wg, float wo, float qs, float as)
{
    if constexpr (XT == DQSQ_X_I32) {
        g = __fmul_rn(g, wg);
        o = __fmul_rn(o, wo);
    }
    o = __fmul_rn(o, qs);
    if constexpr (XT == DQSQ_X_I32) {
        g = __fmul_rn(g, as);
        o = __fmul_rn(o, as);
    }
    const float den = __fadd_rn(canonical_expf(-g), 1.0f);
    return __fdiv_rn(__fmul_rn(g, o), den);
}

__device__ __forceinline__ float dqsq_block_max(float m, float* s_red, int parity)
{
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        m = fmaxf(m, __shfl_xor_sync(FULL_MASK, m, off));
    }
    float* slot = s_red + parity * (DQSQ_THREADS / 32);
    if ((threadIdx.x & 31) == 0) {
        slot[threadIdx.x >> 5] = m;
    }
    __syncthreads();
#pragma unroll
    for (int w = 0; w < DQSQ_THREADS / 32; ++w) {
        m = fmaxf(m, slot[w]);
    }
    return m;
}

// out / s, or out * (1 / s) with `s` already holding the reciprocal
__device__ __forceinline__ float dqsq_scaled(float o, float s, bool divide)
{
    return divide ? __fdiv_rn(o, s) : __fmul_rn(o, s);
}

template <bool DIVIDE>
__device__ __forceinline__ uint32_t dqsq_quant4(const float* o, float s, bool direct)
{
    constexpr bool divide = DIVIDE;
    float v[4];
    bool any_nan = false;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const float q = dqsq_scaled(o[j], s, divide);
        any_nan |= (q != q);
        v[j] = fmaxf(fminf(q, 127.0f), -128.0f);
    }
    uint32_t packed = direct ? narrow4_fast<true>(v[0], v[1], v[2], v[3]) : narrow4_fast<false>(v[0], v[1], v[2], v[3]);
    if (any_nan) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float q = dqsq_scaled(o[j], s, divide);
            if (q != q) {
                packed &= ~(0xffu << (8 * j));
            }
        }
    }
    return packed;
}

// Register-resident rows: H a multiple of the chunk length, at most DQSQ_THREADS * EL * CPT long.
template <int XT, int CPT, bool DIVIDE>
__global__ void __launch_bounds__(DQSQ_THREADS, (CPT <= 2) ? 4 : 1) dqsq_rows_kernel(const void* __restrict__ x,
                                                                 const float* __restrict__ weight_scale,
                                                                 const float* __restrict__ activation_scale,
                                                                 const float* __restrict__ quant_scale,
                                                                 int8_t* __restrict__ y, float* __restrict__ scale,
                                                                 int64_t M, int64_t H, int left, int direct, int)
{
    using C = DqsqChunk<XT>;
    constexpr int EL = C::EL;
    __shared__ float s_red[2 * (DQSQ_THREADS / 32)];
    const int tid = threadIdx.x;
    const int nchunks = static_cast<int>(H / EL);
    const size_t elem = (XT == DQSQ_X_I32) ? 4 : 2;
    const bool has_q = (quant_scale != nullptr);
    // where the gate half and the other half start, in the row and in weight_scale
    const int64_t g_off = left ? 0 : H, o_off = left ? H : 0;
    int parity = 0;
    for (int64_t row = blockIdx.x; row < M; row += gridDim.x, parity ^= 1) {
        const uint8_t* xr = static_cast<const uint8_t*>(x) + static_cast<size_t>(row) * 2 * H * elem;
        const float as = (XT == DQSQ_X_I32) ? activation_scale[row] : 1.0f;
        // every load of the row is issued before the first is used
        uint4 ca[CPT], cb[CPT];
#pragma unroll
        for (int i = 0; i < CPT; ++i) {
            const int c = tid + i * DQSQ_THREADS;
            if (c < nchunks) {
                ca[i] = C::load_raw(xr, g_off + static_cast<int64_t>(c) * EL);
                cb[i] = C::load_raw(xr, o_off + static_cast<int64_t>(c) * EL);
            }
        }
        float out[CPT][EL];
        float m = 0.0f;
#pragma unroll
        for (int i = 0; i < CPT; ++i) {
            const int c = tid + i * DQSQ_THREADS;
            if (c < nchunks) {
                const int64_t j0 = static_cast<int64_t>(c) * EL;
                float a[EL], b[EL];
                C::unpack(ca[i], a);
                C::unpack(cb[i], b);
                // per-channel vectors are re-read by every row: cached 128-bit loads (the launcher checks alignment)
                float wa[EL], wb[EL], qs[EL];
#pragma unroll
                for (int q = 0; q < EL / 4; ++q) {
                    float4 t = make_float4(1.0f, 1.0f, 1.0f, 1.0f);
                    if constexpr (XT == DQSQ_X_I32) {
                        t = __ldg(reinterpret_cast<const float4*>(weight_scale + g_off + j0) + q);
                    }
                    wa[4 * q] = t.x, wa[4 * q + 1] = t.y, wa[4 * q + 2] = t.z, wa[4 * q + 3] = t.w;
                    if constexpr (XT == DQSQ_X_I32) {
                        t = __ldg(reinterpret_cast<const float4*>(weight_scale + o_off + j0) + q);
                    }
                    wb[4 * q] = t.x, wb[4 * q + 1] = t.y, wb[4 * q + 2] = t.z, wb[4 * q + 3] = t.w;
                    t = has_q ? __ldg(reinterpret_cast<const float4*>(quant_scale + j0) + q)
                              : make_float4(1.0f, 1.0f, 1.0f, 1.0f);
                    qs[4 * q] = t.x, qs[4 * q + 1] = t.y, qs[4 * q + 2] = t.z, qs[4 * q + 3] = t.w;
                }
#pragma unroll
                for (int j = 0; j < EL; ++j) {
                    out[i][j] = dqsq_element_by_role<XT>(a[j], b[j], wa[j], wb[j], qs[j], as);
                    m = fmaxf(m, fabsf(out[i][j]));
                }
            }
        }
        m = dqsq_block_max(m, s_red, parity);
        float s = __fmul_rn(m, INV127);
        if (s < 1e-12f) {
            s = 1e-12f;
        }
        if (tid == 0) {
            scale[row] = s;
        }
        const float qf = DIVIDE ? s : __fdiv_rn(1.0f, s);
        int8_t* yr = y + row * H;
#pragma unroll
        for (int i = 0; i < CPT; ++i) {
            const int c = tid + i * DQSQ_THREADS;
            if (c < nchunks) {
                const int64_t j0 = static_cast<int64_t>(c) * EL;
                if constexpr (EL == 4) {
                    *reinterpret_cast<uint32_t*>(yr + j0) = dqsq_quant4<DIVIDE>(out[i], qf, direct != 0);
                } else {
                    const uint2 o = make_uint2(dqsq_quant4<DIVIDE>(out[i], qf, direct != 0),
                                               dqsq_quant4<DIVIDE>(out[i] + 4, qf, direct != 0));
                    *reinterpret_cast<uint2*>(yr + j0) = o;
                }
            }
        }
    }
}

// Any H and any alignment: two passes over the row, the second recomputes the activations (normally from L2).
template <int XT>
__global__ void __launch_bounds__(DQSQ_THREADS) dqsq_long_rows_kernel(const void* __restrict__ x,
                                                                      const float* __restrict__ weight_scale,
                                                                      const float* __restrict__ activation_scale,
                                                                      const float* __restrict__ quant_scale,
                                                                      int8_t* __restrict__ y, float* __restrict__ scale,
                                                                      int64_t M, int64_t H, int left, int direct, int divide)
{
    using C = DqsqChunk<XT>;
    __shared__ float s_red[2 * (DQSQ_THREADS / 32)];
    const size_t elem = (XT == DQSQ_X_I32) ? 4 : 2;
    const bool has_q = (quant_scale != nullptr);
    int parity = 0;
    for (int64_t row = blockIdx.x; row < M; row += gridDim.x, parity ^= 1) {
        const uint8_t* xr = static_cast<const uint8_t*>(x) + static_cast<size_t>(row) * 2 * H * elem;
        const float as = (XT == DQSQ_X_I32) ? activation_scale[row] : 1.0f;
        auto element = [&](int64_t j) {
            const float wa = (XT == DQSQ_X_I32) ? weight_scale[j] : 1.0f;
            const float wb = (XT == DQSQ_X_I32) ? weight_scale[H + j] : 1.0f;
            const float qs = has_q ? quant_scale[j] : 1.0f;
            return dqsq_element<XT>(C::load1(xr, j), C::load1(xr, H + j), wa, wb, qs, as, has_q, left != 0);
        };
        float m = 0.0f;
        for (int64_t j = threadIdx.x; j < H; j += DQSQ_THREADS) {
            m = fmaxf(m, fabsf(element(j)));
        }
        m = dqsq_block_max(m, s_red, parity);
        float s = __fmul_rn(m, INV127);
        if (s < 1e-12f) {
            s = 1e-12f;
        }
        if (threadIdx.x == 0) {
            scale[row] = s;
        }
        const float qf = divide ? s : __fdiv_rn(1.0f, s);
        for (int64_t j = threadIdx.x; j < H; j += DQSQ_THREADS) {
            const float q = dqsq_scaled(element(j), qf, divide != 0);
            const float v = fmaxf(fminf(q, 127.0f), -128.0f);
            y[row * H + j] = (q != q) ? static_cast<int8_t>(0)
                                      : static_cast<int8_t>(direct ? narrow1_general<true>(v) : narrow1_general<false>(v));
        }
    }
}

template <int XT>
static cudaError_t dispatch_dqsq(const void* x, const float* ws, const float* as, const float* qs, int8_t* y,
                                 float* scale, int64_t M, int64_t H, int left, int direct, bool vec, cudaStream_t st)
{
    constexpr int EL = DqsqChunk<XT>::EL;
    // padded half-row length of the reference's layout choice: H rounded up to 32 bytes of the input type
    constexpr int64_t PAD = (XT == DQSQ_X_I32) ? 8 : 16;
    const int divide = ((H + PAD - 1) / PAD * PAD <= 1984) ? 1 : 0;
    const int64_t chunks = (H + EL - 1) / EL;
    using Kern = void (*)(const void*, const float*, const float*, const float*, int8_t*, float*, int64_t, int64_t, int,
                          int, int);
    Kern kern = dqsq_long_rows_kernel<XT>;
    if (vec && chunks <= DQSQ_THREADS) {
        kern = divide ? dqsq_rows_kernel<XT, 1, true> : dqsq_rows_kernel<XT, 1, false>;
    } else if (vec && chunks <= 2 * DQSQ_THREADS) {
        kern = divide ? dqsq_rows_kernel<XT, 2, true> : dqsq_rows_kernel<XT, 2, false>;
    } else if (vec && chunks <= 4 * DQSQ_THREADS) {
        kern = dqsq_rows_kernel<XT, 4, false>;  // rows this long always take the reciprocal form
    } else if (vec && chunks <= 8 * DQSQ_THREADS) {
        kern = dqsq_rows_kernel<XT, 8, false>;
    }
    // one wave: as many CTAs as are resident at once, each walking rows with a grid stride
    int per_sm = 1;
    const cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, DQSQ_THREADS, 0);
    if (e != cudaSuccess) {
        return e;
    }
    const int64_t cap = static_cast<int64_t>(sm_count()) * (per_sm < 1 ? 1 : per_sm);
    const unsigned grid = static_cast<unsigned>(M < cap ? M : cap);
    kern<<<grid, DQSQ_THREADS, 0, st>>>(x, ws, as, qs, y, scale, M, H, left, direct, divide); w8a8::note_launch();
    return cudaGetLastError();
}

}  // namespace w8a8

extern "C" int w8a8_dequant_swiglu_quant(const void* x, const float* weight_scale, const float* activation_scale,
                                         const float* quant_scale, int8_t* y, float* scale, int64_t M, int64_t H,
                                         int x_dtype, int activate_left, int flags, void* stream)
{
    if (x_dtype != W8A8_DT_I32 && x_dtype != W8A8_DT_F16 && x_dtype != W8A8_DT_BF16) {
        return W8A8_ERR_INVALID;
    }
    if (M < 0 || H <= 0 || (flags & ~W8A8_F_ROUND_DIRECT) != 0) {
        return W8A8_ERR_INVALID;
    }
    const bool is_i32 = (x_dtype == W8A8_DT_I32);
    if (is_i32 != (weight_scale != nullptr) || is_i32 != (activation_scale != nullptr)) {
        return W8A8_ERR_INVALID;  // both scales with int32 input, neither with 16-bit input
    }
    if (M == 0) {
        return W8A8_OK;
    }
    if (x == nullptr || y == nullptr || scale == nullptr) {
        return W8A8_ERR_INVALID;
    }
    const size_t elem = is_i32 ? 4 : 2;
    if (!w8a8::is_aligned(x, elem) || !w8a8::is_aligned(scale, 4) || !w8a8::is_aligned(weight_scale, 4) ||
        !w8a8::is_aligned(activation_scale, 4) || !w8a8::is_aligned(quant_scale, 4)) {
        return W8A8_ERR_ALIGN;
    }
    const int64_t el = is_i32 ? 4 : 8;
    const bool vec = (H % el == 0) && w8a8::is_aligned(x, 16) && w8a8::is_aligned(y, 8) && (H * elem) % 16 == 0 &&
                     w8a8::is_aligned(weight_scale, 16) && w8a8::is_aligned(quant_scale, 16);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int left = activate_left ? 1 : 0;
    const int direct = (flags & W8A8_F_ROUND_DIRECT) ? 1 : 0;
    cudaError_t e;
    if (is_i32) {
        e = w8a8::dispatch_dqsq<w8a8::DQSQ_X_I32>(x, weight_scale, activation_scale, quant_scale, y, scale, M, H, left,
                                                  direct, vec, st);
    } else if (x_dtype == W8A8_DT_F16) {
        e = w8a8::dispatch_dqsq<w8a8::DQSQ_X_F16>(x, nullptr, nullptr, quant_scale, y, scale, M, H, left, direct, vec,
                                                  st);
    } else {
        e = w8a8::dispatch_dqsq<w8a8::DQSQ_X_BF16>(x, nullptr, nullptr, quant_scale, y, scale, M, H, left, direct, vec,
                                                   st);
    }
    return (e == cudaSuccess) ? W8A8_OK : W8A8_ERR_CUDA;
}
