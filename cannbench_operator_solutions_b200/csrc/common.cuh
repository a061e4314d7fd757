// Shared device helpers for the W8A8 quantised-FFN kernels (sm_100a).
//
// The whole library is compiled with -fmad=false: the operators' results
// depend on which multiplies and adds are rounded separately, so every fused
// multiply-add in these sources is an explicit fmaf().
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/w8a8ffn.h"

namespace w8a8 {

constexpr unsigned FULL_MASK = 0xffffffffu;
constexpr float INV127 = 1.0f / 127.0f;

// ---------------------------------------------------------------------------
// 16-bit float <-> fp32
// ---------------------------------------------------------------------------
template <int DT>
__device__ __forceinline__ void unpack2(uint32_t p, float& lo, float& hi)
{
    if constexpr (DT == W8A8_DT_BF16) {
        lo = __uint_as_float(p << 16);
        hi = __uint_as_float(p & 0xffff0000u);
    } else {
        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&p));
        lo = f.x;
        hi = f.y;
    }
}

template <int DT>
__device__ __forceinline__ uint32_t pack2(float lo, float hi)
{
    if constexpr (DT == W8A8_DT_BF16) {
        const __nv_bfloat162 b = __floats2bfloat162_rn(lo, hi);
        return *reinterpret_cast<const uint32_t*>(&b);
    } else {
        const __half2 h = __floats2half2_rn(lo, hi);
        return *reinterpret_cast<const uint32_t*>(&h);
    }
}

template <int DT>
__device__ __forceinline__ float bits16_to_float(uint32_t b)
{
    if constexpr (DT == W8A8_DT_BF16) {
        return __uint_as_float(b << 16);
    } else {
        return __half2float(__ushort_as_half(static_cast<unsigned short>(b)));
    }
}

template <int DT>
__device__ __forceinline__ uint16_t float_to_bits16(float v)
{
    if constexpr (DT == W8A8_DT_BF16) {
        return __bfloat16_as_ushort(__float2bfloat16_rn(v));
    } else {
        return __half_as_ushort(__float2half_rn(v));
    }
}

// fp32 exp shared with the CPU oracle: Cody-Waite reduction by ln2 in two
// pieces, degree-5 polynomial (the classic single-precision coefficients
// published with the Cephes library), two-step power-of-two scaling.  Built
// from IEEE mul / add / fma only, so host and device agree bit for bit.
// This is the defining sequence; the kernels call canonical_expf below, which
// returns the same bits with fewer instructions.
__device__ __forceinline__ float canonical_expf_as_defined(float x)
{
    if (x != x) {
        return x;
    }
    x = (x > 89.0f) ? 89.0f : x;
    x = (x < -104.0f) ? -104.0f : x;
    const float n = rintf(__fmul_rn(x, 1.44269504088896341f));
    float r = fmaf(n, -0.693359375f, x);
    r = fmaf(n, 2.12194440e-4f, r);
    float p = 1.9875691500e-4f;
    p = fmaf(p, r, 1.3981999507e-3f);
    p = fmaf(p, r, 8.3334519073e-3f);
    p = fmaf(p, r, 4.1665795894e-2f);
    p = fmaf(p, r, 1.6666665459e-1f);
    p = fmaf(p, r, 5.0000001201e-1f);
    const float r2 = __fmul_rn(r, r);
    float e = fmaf(p, r2, r);
    e = __fadd_rn(e, 1.0f);
    const int ni = static_cast<int>(n);
    const int n1 = ni >> 1;
    const int n2 = ni - n1;
    const float s1 = __int_as_float((n1 + 127) << 23);
    const float s2 = __int_as_float((n2 + 127) << 23);
    return __fmul_rn(__fmul_rn(e, s1), s2);
}

// The same function, bit for bit on every input (w8a8_selftest_exp sweeps all 2^32), arranged for the issue
// slots it costs in the SwiGLU epilogues and the router softmax:
//  - rint and the float -> int conversion (conversion-pipe instructions, a quarter of the fp32 rate) become an
//    add and a subtract of 1.5 * 2^23, whose sum holds the integer in its low mantissa bits (|n| <= 151);
//    a product that rounds to -0 gives n = +0 instead of -0, which the two fma that use n turn into the same r;
//  - e lies in [0.70, 1.42] and n1 = n >> 1 in [-75, 64], so the first of the two multiplications by powers of
//    two is exact and lands on a normal number: it becomes an integer add to e's exponent field.  The second
//    multiplication stays, because it is the one that rounds (subnormal results) or overflows.
__device__ __forceinline__ float canonical_expf(float x)
{
    const float xc = fminf(fmaxf(x, -104.0f), 89.0f);  // a NaN comes out as -104 here and is put back at the end
    const float t = __fadd_rn(__fmul_rn(xc, 1.44269504088896341f), 12582912.0f);
    const float n = __fsub_rn(t, 12582912.0f);
    const int ni = __float_as_int(t) - 0x4B400000;
    float r = fmaf(n, -0.693359375f, xc);
    r = fmaf(n, 2.12194440e-4f, r);
    float p = 1.9875691500e-4f;
    p = fmaf(p, r, 1.3981999507e-3f);
    p = fmaf(p, r, 8.3334519073e-3f);
    p = fmaf(p, r, 4.1665795894e-2f);
    p = fmaf(p, r, 1.6666665459e-1f);
    p = fmaf(p, r, 5.0000001201e-1f);
    const float r2 = __fmul_rn(r, r);
    float e = fmaf(p, r2, r);
    e = __fadd_rn(e, 1.0f);
    const int n1 = ni >> 1;
    const int n2 = ni - n1;
    const float e1 = __int_as_float(__float_as_int(e) + (n1 << 23));
    const float s2 = __int_as_float((n2 << 23) + 0x3f800000);
    const float out = __fmul_rn(e1, s2);
    return (x != x) ? x : out;
}

// silu(l) = l / (1 + exp(-l)), the operation sequence of the reference
// (gmsq_vec_kernel.cpp:213-217).
__device__ __forceinline__ float canonical_silu(float l)
{
    const float e = __fadd_rn(canonical_expf(-l), 1.0f);
    return __fdiv_rn(l, e);
}

// ---------------------------------------------------------------------------
// fp32 -> int8 narrowing.
//
// "As written" (the reference's two casts): fp32 -> fp16 RNE, then fp16 ->
// int8 RNE.  For |v| <= 128 the second step is done without a conversion
// instruction: adding 1536 (= 1.5 * 2^10, where fp16 has unit spacing)
// rounds to the nearest integer, ties to even, and leaves the two's
// complement byte in the low 8 bits of the sum's bit pattern.
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t narrow4_fp16_fast(float a, float b, float c, float d)
{
    const __half2 magic = __floats2half2_rn(1536.0f, 1536.0f);
    __half2 h01 = __hadd2(__floats2half2_rn(a, b), magic);
    __half2 h23 = __hadd2(__floats2half2_rn(c, d), magic);
    return __byte_perm(*reinterpret_cast<uint32_t*>(&h01), *reinterpret_cast<uint32_t*>(&h23), 0x6420);
}

// Direct fp32 -> int8 RNE for |v| <= 128: 1.5 * 2^23 trick.
__device__ __forceinline__ uint32_t narrow4_direct_fast(float a, float b, float c, float d)
{
    const float magic = 12582912.0f;
    const uint32_t ua = __float_as_uint(__fadd_rn(a, magic));
    const uint32_t ub = __float_as_uint(__fadd_rn(b, magic));
    const uint32_t uc = __float_as_uint(__fadd_rn(c, magic));
    const uint32_t ud = __float_as_uint(__fadd_rn(d, magic));
    const uint32_t ab = __byte_perm(ua, ub, 0x0040);
    const uint32_t cd = __byte_perm(uc, ud, 0x0040);
    return __byte_perm(ab, cd, 0x5410);
}

// Fully general narrowing: any fp32 including NaN (-> 0), inf and values
// outside the int8 range (saturate).
template <bool DIRECT>
__device__ __forceinline__ int narrow1_general(float v)
{
    int r;
    if constexpr (DIRECT) {
        r = (v != v) ? 0 : __float2int_rn(fminf(fmaxf(v, -128.0f), 127.0f));
    } else {
        const __half h = __float2half_rn(v);
        const float hv = __half2float(h);
        r = (hv != hv) ? 0 : __float2int_rn(fminf(fmaxf(hv, -128.0f), 127.0f));
    }
    return r;
}

template <bool DIRECT>
__device__ __forceinline__ uint32_t narrow4_general(float a, float b, float c, float d)
{
    const uint32_t ua = static_cast<uint32_t>(narrow1_general<DIRECT>(a)) & 0xffu;
    const uint32_t ub = static_cast<uint32_t>(narrow1_general<DIRECT>(b)) & 0xffu;
    const uint32_t uc = static_cast<uint32_t>(narrow1_general<DIRECT>(c)) & 0xffu;
    const uint32_t ud = static_cast<uint32_t>(narrow1_general<DIRECT>(d)) & 0xffu;
    return ua | (ub << 8) | (uc << 16) | (ud << 24);
}

template <bool DIRECT>
__device__ __forceinline__ uint32_t narrow4_fast(float a, float b, float c, float d)
{
    if constexpr (DIRECT) {
        return narrow4_direct_fast(a, b, c, d);
    } else {
        return narrow4_fp16_fast(a, b, c, d);
    }
}

// ---------------------------------------------------------------------------
// One 8-element chunk of a 16-bit row: 128-bit streaming load when the row
// is 16-byte aligned and a multiple of 8 long, element-wise otherwise
// (missing elements read as +0, the identity of both row reductions).
// ---------------------------------------------------------------------------
template <bool VEC>
__device__ __forceinline__ uint4 load_chunk16(const uint16_t* row, int c, int64_t N)
{
    if constexpr (VEC) {
        return __ldcs(reinterpret_cast<const uint4*>(row) + c);
    } else {
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int64_t e = static_cast<int64_t>(c) * 8 + 2 * i;
            const uint32_t lo = (e < N) ? row[e] : 0u;
            const uint32_t hi = (e + 1 < N) ? row[e + 1] : 0u;
            w[i] = lo | (hi << 16);
        }
        return make_uint4(w[0], w[1], w[2], w[3]);
    }
}

// gamma-like vectors are re-read by every row: keep them cacheable
template <bool VEC>
__device__ __forceinline__ uint4 load_chunk16_cached(const uint16_t* row, int c, int64_t N)
{
    if constexpr (VEC) {
        return __ldg(reinterpret_cast<const uint4*>(row) + c);
    } else {
        return load_chunk16<false>(row, c, N);
    }
}

template <bool VEC>
__device__ __forceinline__ void store_chunk16(uint16_t* row, int c, int64_t N, uint4 v)
{
    if constexpr (VEC) {
        __stcs(reinterpret_cast<uint4*>(row) + c, v);
    } else {
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int64_t e = static_cast<int64_t>(c) * 8 + 2 * i;
            if (e < N) {
                row[e] = static_cast<uint16_t>(w[i] & 0xffffu);
            }
            if (e + 1 < N) {
                row[e + 1] = static_cast<uint16_t>(w[i] >> 16);
            }
        }
    }
}

template <bool VEC>
__device__ __forceinline__ void store_chunk8(int8_t* row, int c, int64_t N, uint32_t lo, uint32_t hi)
{
    if constexpr (VEC) {
        __stcs(reinterpret_cast<uint2*>(row) + c, make_uint2(lo, hi));
    } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int64_t e = static_cast<int64_t>(c) * 8 + i;
            if (e < N) {
                const uint32_t w = (i < 4) ? lo : hi;
                row[e] = static_cast<int8_t>((w >> (8 * (i & 3))) & 0xffu);
            }
        }
    }
}

// Largest |.| bit pattern of the eight 16-bit values in a chunk, compared as
// unsigned integers: orders finite magnitudes, inf above them, NaN above inf.
__device__ __forceinline__ uint32_t chunk_absmax16(uint4 v, uint32_t m2)
{
    m2 = __vmaxu2(m2, v.x & 0x7fff7fffu);
    m2 = __vmaxu2(m2, v.y & 0x7fff7fffu);
    m2 = __vmaxu2(m2, v.z & 0x7fff7fffu);
    m2 = __vmaxu2(m2, v.w & 0x7fff7fffu);
    return m2;
}

inline bool is_aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; }

int sm_count();  // cached multiprocessor count of the current device
void note_launch();  // counts one kernel launch of this library (w8a8_kernel_launch_count)

}  // namespace w8a8
