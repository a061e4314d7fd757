/*
 * CPU oracle for the W8A8 quantised-FFN operators.  TEST INFRASTRUCTURE ONLY:
 * see w8a8_oracle.h for what this is, who may call it, and its parity status
 * (PARITY UNPINNED against reference outputs: the reference has no golden
 * vectors and cannot be built without the Ascend toolchain).
 *
 * Build with:  gcc -O2 -fopenmp -ffp-contract=off -fno-fast-math -mfma -mf16c
 * so that no multiply/add pair is contracted behind the source's back; every
 * fused multiply-add below is an explicit fmaf().
 *
 * Reference paths are relative to the reference project root; the common
 * prefix operators/<op>/csrc/ops/<dir>/ is abbreviated:
 *   DQ   = operators/dynamicquant/csrc/ops/dynamic_quant
 *   ARDQ = operators/addrmsnormdynamicquant/csrc/ops/add_rms_norm_dynamic_quant
 *   QM   = operators/quantmatmul/csrc/ops/quant_matmul
 *   GMSQ = operators/groupedmatmulswigluquant/csrc/ops/grouped_matmul_swiglu_quant
 *   GMM  = operators/groupedmatmul/csrc/ops/grouped_matmul
 *   MFR  = operators/moefinalizerouting/csrc/ops/moe_finalize_routing
 *   MRR  = operators/moererouting/csrc/ops/moe_re_routing
 */
#include "w8a8_oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

/* ------------------------------------------------------------------------ */
/* bit-level conversions                                                     */
/* ------------------------------------------------------------------------ */
static inline uint32_t f2u(float f)
{
    uint32_t u;
    memcpy(&u, &f, 4);
    return u;
}
static inline float u2f(uint32_t u)
{
    float f;
    memcpy(&f, &u, 4);
    return f;
}

float oracle_bf16_to_f32(uint16_t h) { return u2f((uint32_t)h << 16); }

/* fp32 -> bf16, round to nearest even; NaN stays NaN (quiet). */
uint16_t oracle_f32_to_bf16(float f)
{
    uint32_t u = f2u(f);
    if ((u & 0x7fffffffu) > 0x7f800000u) {
        return (uint16_t)((u >> 16) | 0x0040u);
    }
    uint32_t lsb = (u >> 16) & 1u;
    u += 0x7fffu + lsb;
    return (uint16_t)(u >> 16);
}

float oracle_f16_to_f32(uint16_t h)
{
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1fu;
    uint32_t man = h & 0x3ffu;
    if (exp == 0x1fu) {
        return u2f(sign | 0x7f800000u | (man << 13));
    }
    if (exp == 0) {
        /* subnormal: man * 2^-24 (exact in fp32) */
        float v = (float)man * 5.9604644775390625e-8f;
        return (sign != 0) ? -v : v;
    }
    return u2f(sign | ((exp + 112u) << 23) | (man << 13));
}

/* fp32 -> fp16, round to nearest even, IEEE overflow to inf, gradual underflow. */
uint16_t oracle_f32_to_f16(float f)
{
    uint32_t u = f2u(f);
    uint16_t sign = (uint16_t)((u >> 16) & 0x8000u);
    uint32_t a = u & 0x7fffffffu;
    if (a > 0x7f800000u) {
        return (uint16_t)(sign | 0x7e00u);
    }
    if (a >= 0x477ff000u) {
        /* >= 65520 rounds to infinity */
        return (uint16_t)(sign | 0x7c00u);
    }
    if (a < 0x38800000u) {
        /* below the smallest normal half (2^-14): the result is a multiple of
         * 2^-24; 2^-25 and anything smaller rounds (ties to even) to zero */
        if (a <= 0x33000000u) {
            return sign;
        }
        /* v * 2^24 is exact; nearbyint in the default rounding mode is RNE.
         * q == 1024 encodes the smallest normal, as it should. */
        float q = nearbyintf(u2f(a) * 16777216.0f);
        return (uint16_t)(sign | (uint16_t)q);
    }
    uint32_t lsb = (a >> 13) & 1u;
    a += 0xfffu + lsb;
    return (uint16_t)(sign | (uint16_t)((a - 0x38000000u) >> 13));
}

/* fp16 -> int8: round to nearest even, saturate, NaN -> 0.
 * (CAST_RINT half -> int8, e.g. DQ/op_kernel/dynamic_quant_kernel.cpp:282) */
static inline int8_t f16_to_i8(uint16_t h)
{
    float v = oracle_f16_to_f32(h);
    if (v != v) {
        return 0;
    }
    float r = nearbyintf(v);
    if (r > 127.0f) {
        return 127;
    }
    if (r < -128.0f) {
        return -128;
    }
    return (int8_t)r;
}

/* The narrowing every quantising kernel performs (AS_WRITTEN): fp32 -> fp16
 * with CAST_RINT, then fp16 -> int8 with CAST_RINT
 * (DQ/op_kernel/dynamic_quant_kernel.cpp:279-282,
 *  ARDQ/op_kernel/add_rms_norm_dynamic_quant_kernel.cpp:312-314,
 *  GMSQ/op_kernel/gmsq_vec_kernel.cpp:256-257).  DIRECT rounds fp32 -> int8
 * once. */
int8_t oracle_narrow_i8(float v, int round_mode)
{
    if (round_mode == W8A8_ROUND_AS_WRITTEN) {
        return f16_to_i8(oracle_f32_to_f16(v));
    }
    if (v != v) {
        return 0;
    }
    float r = nearbyintf(v);
    if (r > 127.0f) {
        return 127;
    }
    if (r < -128.0f) {
        return -128;
    }
    return (int8_t)r;
}

static inline float load_as_f32(const void* p, int64_t i, int dtype)
{
    switch (dtype) {
    case W8A8_DT_F16:
        return oracle_f16_to_f32(((const uint16_t*)p)[i]);
    case W8A8_DT_BF16:
        return oracle_bf16_to_f32(((const uint16_t*)p)[i]);
    default:
        return ((const float*)p)[i];
    }
}

static inline void store_from_f32(void* p, int64_t i, int dtype, float v)
{
    switch (dtype) {
    case W8A8_DT_F16:
        ((uint16_t*)p)[i] = oracle_f32_to_f16(v);
        break;
    case W8A8_DT_BF16:
        ((uint16_t*)p)[i] = oracle_f32_to_bf16(v);
        break;
    default:
        ((float*)p)[i] = v;
        break;
    }
}

/* |a| as an unsigned bit pattern.  Ordering these patterns as integers orders
 * finite magnitudes, puts inf above every finite value and NaN above inf, so
 * an integer max is a NaN-propagating absolute maximum (what torch's amax in
 * the benchmark's golden does). */
static inline uint32_t abs_bits(float a) { return f2u(a) & 0x7fffffffu; }

int oracle_num_threads(void)
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* ------------------------------------------------------------------------ */
/* DynamicQuant                                                              */
/* DQ/op_kernel/dynamic_quant_kernel.cpp:15-26 (math), :240 (clamp 1e-12),   */
/* :249 (scale = amax * (1/127)), :256-257 (inv = Reciprocal(amax) * 127),   */
/* :260-276 (y = x * inv), :279-282 (two-step narrowing).                    */
/* ------------------------------------------------------------------------ */
int oracle_dynamic_quant(const void* x, int8_t* y, float* scale, int64_t M, int64_t N, int dtype,
                         int round_mode)
{
    if (dtype != W8A8_DT_F16 && dtype != W8A8_DT_BF16) {
        return -1;
    }
    if (M < 0 || N <= 0) {
        return -1;
    }
    const float inv127 = 1.0f / 127.0f;
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < M; ++r) {
        uint32_t mb = 0;
        for (int64_t j = 0; j < N; ++j) {
            uint32_t b = abs_bits(load_as_f32(x, r * N + j, dtype));
            if (b > mb) {
                mb = b;
            }
        }
        float amax = u2f(mb);
        /* Maxs(amax, 1e-12): a NaN maximum stays NaN */
        if (amax < 1e-12f) {
            amax = 1e-12f;
        }
        scale[r] = amax * inv127;
        float inv = (1.0f / amax) * 127.0f;
        for (int64_t j = 0; j < N; ++j) {
            float v = load_as_f32(x, r * N + j, dtype) * inv;
            y[r * N + j] = oracle_narrow_i8(v, round_mode);
        }
    }
    return 0;
}

/* ------------------------------------------------------------------------ */
/* AddRmsNormDynamicQuant                                                    */
/* ARDQ/op_kernel/add_rms_norm_dynamic_quant_kernel.cpp:15-30 (algebra),     */
/* :232-247 (fp32 add), :251-265 (xOut rounded to T only for the store),     */
/* :268-270 (z = xOut*gamma), :275-282 (sum x^2, max|z|, *invN, +eps, sqrt), */
/* :286-298 (rstd, m, clamp, scale, k), :308-314 (y = narrow(z*k)).          */
/*                                                                           */
/* The order in which the Ascend vector unit adds the squares cannot be      */
/* known here.  W8A8_SUM_CANONICAL is this project's own fixed order, the    */
/* one its CUDA kernel uses: 256 lanes; lane t owns the 8-element chunks     */
/* c = t, t+256, ... and folds their elements in order with fmaf(v,v,acc);   */
/* lanes combine inside each group of 32 by a butterfly (xor 16,8,4,2,1) and */
/* the eight group sums are added left to right.  W8A8_SUM_FP64 accumulates  */
/* sequentially in double and is used to state the tolerance.                */
/* ------------------------------------------------------------------------ */
static float sumsq_canonical(const float* v, int64_t N)
{
    float lane[256];
    for (int t = 0; t < 256; ++t) {
        lane[t] = 0.0f;
    }
    int64_t chunks = (N + 7) / 8;
    for (int64_t c = 0; c < chunks; ++c) {
        int t = (int)(c & 255);
        int64_t e0 = c * 8;
        int64_t e1 = e0 + 8 < N ? e0 + 8 : N;
        float acc = lane[t];
        for (int64_t e = e0; e < e1; ++e) {
            acc = fmaf(v[e], v[e], acc);
        }
        lane[t] = acc;
    }
    float total = 0.0f;
    for (int w = 0; w < 8; ++w) {
        float a[32];
        float b[32];
        for (int l = 0; l < 32; ++l) {
            a[l] = lane[w * 32 + l];
        }
        for (int off = 16; off >= 1; off >>= 1) {
            for (int l = 0; l < 32; ++l) {
                b[l] = a[l] + a[l ^ off];
            }
            for (int l = 0; l < 32; ++l) {
                a[l] = b[l];
            }
        }
        total = (w == 0) ? a[0] : total + a[0];
    }
    return total;
}

int oracle_add_rms_norm_dynamic_quant(const void* x1, const void* x2, const void* gamma, int8_t* y,
                                      void* x_out, float* scale_out, int64_t rows, int64_t N,
                                      float eps, int dtype, int round_mode, int sum_order)
{
    if (dtype != W8A8_DT_F16 && dtype != W8A8_DT_BF16) {
        return -1;
    }
    if (rows < 0 || N <= 0 || N > 16384) {
        return -1; /* ARDQ/op_plugin/add_rms_norm_dynamic_quant_plugin.cpp:82 */
    }
    const float invN = 1.0f / (float)N;
    const float inv127 = 1.0f / 127.0f;
#pragma omp parallel
    {
        float* xo = (float*)malloc(sizeof(float) * (size_t)N);
        float* z = (float*)malloc(sizeof(float) * (size_t)N);
#pragma omp for schedule(static)
        for (int64_t r = 0; r < rows; ++r) {
            uint32_t mb = 0;
            for (int64_t j = 0; j < N; ++j) {
                float a = load_as_f32(x1, r * N + j, dtype);
                float b = load_as_f32(x2, r * N + j, dtype);
                float s = a + b;
                xo[j] = s;
                store_from_f32(x_out, r * N + j, dtype, s);
                float zz = s * load_as_f32(gamma, j, dtype);
                z[j] = zz;
                uint32_t ab = abs_bits(zz);
                if (ab > mb) {
                    mb = ab;
                }
            }
            float sum;
            if (sum_order == W8A8_SUM_FP64) {
                double acc = 0.0;
                for (int64_t j = 0; j < N; ++j) {
                    acc += (double)xo[j] * (double)xo[j];
                }
                sum = (float)acc;
            } else {
                sum = sumsq_canonical(xo, N);
            }
            float mean = sum * invN;
            float rms = sqrtf(mean + eps);
            float max_abs = u2f(mb);
            float rstd = 1.0f / rms;
            float m = max_abs * rstd;
            float sm = (m < 1e-12f) ? 1e-12f : m;
            float sc = sm * inv127;
            float k = rstd / sc;
            scale_out[r] = sc;
            for (int64_t j = 0; j < N; ++j) {
                y[r * N + j] = oracle_narrow_i8(z[j] * k, round_mode);
            }
        }
        free(xo);
        free(z);
    }
    return 0;
}

/* ------------------------------------------------------------------------ */
/* int8 x int8 -> int32 row product (exact).  The reference delegates this   */
/* to the Ascend Matmul library (QM/op_kernel/quant_matmul_cube_kernel.cpp:  */
/* 119-173, GMSQ/op_kernel/gmsq_cube_kernel.cpp:48-130); an integer triple   */
/* loop is the same function.                                                */
/* ------------------------------------------------------------------------ */
static void i8_row_times_matrix(const int8_t* a, const int8_t* b, int32_t* acc, int64_t K,
                                int64_t N, int64_t ldb, int transposed)
{
    if (!transposed) {
        /* b is [K, N] with row pitch ldb */
        for (int64_t j = 0; j < N; ++j) {
            acc[j] = 0;
        }
        for (int64_t k = 0; k < K; ++k) {
            int32_t av = a[k];
            if (av == 0) {
                continue;
            }
            const int8_t* br = b + k * ldb;
            for (int64_t j = 0; j < N; ++j) {
                acc[j] += av * (int32_t)br[j];
            }
        }
    } else {
        /* b is [N, K] with row pitch ldb */
        for (int64_t j = 0; j < N; ++j) {
            const int8_t* br = b + j * ldb;
            int32_t s = 0;
            for (int64_t k = 0; k < K; ++k) {
                s += (int32_t)a[k] * (int32_t)br[k];
            }
            acc[j] = s;
        }
    }
}

/* ------------------------------------------------------------------------ */
/* QuantMatmul                                                               */
/* QM/op_kernel/quant_matmul_epilogue_kernel.cpp:15-22 (golden semantics),   */
/* :113-121 (flag decoding), :247-251 (pertoken index, modulo M when the     */
/* rows cover several batches), :261 (int32 -> fp32), :265-301 (int32 bias   */
/* added AFTER widening, scale, offset, pertoken, float bias, in this        */
/* order), :305 (RINT cast to fp16/bf16).                                    */
/* ------------------------------------------------------------------------ */
static float qm_vec_elem(const void* p, int64_t i, int kind)
{
    switch (kind) {
    case W8A8_QM_BIAS_I32:
        return (float)((const int32_t*)p)[i];
    case W8A8_QM_BIAS_F16:
        return oracle_f16_to_f32(((const uint16_t*)p)[i]);
    case W8A8_QM_BIAS_BF16:
        return oracle_bf16_to_f32(((const uint16_t*)p)[i]);
    default:
        return ((const float*)p)[i];
    }
}

int oracle_quant_matmul(const int8_t* x1, const int8_t* x2, const void* scale, const float* offset,
                        const float* pertoken, const void* bias, void* out, int64_t batch,
                        int64_t M, int64_t N, int64_t K, int64_t flags, int out_dtype,
                        int x2_transposed, int32_t* acc_out)
{
    if (batch <= 0 || M <= 0 || N <= 0 || K <= 0) {
        return -1;
    }
    if (out_dtype != W8A8_DT_F16 && out_dtype != W8A8_DT_BF16) {
        return -1;
    }
    const int scale_perchan = (flags & W8A8_QM_SCALE_PERCHAN) != 0;
    const int scale_bf16 = (flags & W8A8_QM_SCALE_BF16) != 0;
    const int has_offset = (flags & W8A8_QM_HAS_OFFSET) != 0;
    const int offset_perchan = (flags & W8A8_QM_OFFSET_PERCHAN) != 0;
    const int has_pt = (flags & W8A8_QM_HAS_PT) != 0;
    const int bias_kind = (int)((flags & W8A8_QM_BIAS_MASK) >> W8A8_QM_BIAS_SHIFT);
    const int bias_perchan = (flags & W8A8_QM_BIAS_PERCHAN) != 0;
    if (bias_kind > W8A8_QM_BIAS_F32) {
        return -1;
    }
    const int64_t rows = batch * M;
#pragma omp parallel
    {
        int32_t* acc = (int32_t*)malloc(sizeof(int32_t) * (size_t)N);
#pragma omp for schedule(dynamic, 4)
        for (int64_t r = 0; r < rows; ++r) {
            const int64_t b = r / M;
            i8_row_times_matrix(x1 + r * K, x2 + b * K * N, acc, K, N, x2_transposed ? K : N,
                                x2_transposed);
            if (acc_out != NULL) {
                memcpy(acc_out + r * N, acc, sizeof(int32_t) * (size_t)N);
            }
            /* pertoken[m]: the flag says "index modulo M"; with the plugin's
             * layouts r % M is the token index in both cases */
            float pt = 1.0f;
            if (has_pt) {
                pt = pertoken[(flags & W8A8_QM_PT_MOD_M) ? (r % M) : r];
            }
            for (int64_t j = 0; j < N; ++j) {
                float v = (float)acc[j];
                if (bias_kind == W8A8_QM_BIAS_I32) {
                    v = v + qm_vec_elem(bias, bias_perchan ? j : 0, bias_kind);
                }
                float sc = scale_bf16
                               ? oracle_bf16_to_f32(((const uint16_t*)scale)[scale_perchan ? j : 0])
                               : ((const float*)scale)[scale_perchan ? j : 0];
                v = v * sc;
                if (has_offset) {
                    v = v + offset[offset_perchan ? j : 0];
                }
                if (has_pt) {
                    v = v * pt;
                }
                if (bias_kind >= W8A8_QM_BIAS_F16) {
                    v = v + qm_vec_elem(bias, bias_perchan ? j : 0, bias_kind);
                }
                store_from_f32(out, r * N + j, out_dtype, v);
            }
        }
        free(acc);
    }
    return 0;
}

/* ------------------------------------------------------------------------ */
/* exp and silu.                                                             */
/* GMSQ/op_kernel/gmsq_vec_kernel.cpp:213-218: silu(l) = l / (1 + exp(-l)),  */
/* evaluated as Muls(-1) -> Exp -> Adds(1) -> Div, all fp32.  The accuracy   */
/* of the Ascend vector Exp is not documented, so the oracle fixes its own   */
/* fp32 exp, built only from IEEE mul/add/fma so that the CUDA kernel can    */
/* evaluate the identical sequence: Cody-Waite reduction by ln2 in two       */
/* pieces, a degree-5 polynomial in Horner form (the classic single          */
/* precision coefficients published with the Cephes library), and a two-step */
/* power-of-two scaling that is exact outside the subnormal range.           */
/* ------------------------------------------------------------------------ */
float oracle_expf(float x)
{
    if (x != x) {
        return x;
    }
    if (x > 89.0f) {
        x = 89.0f;
    }
    if (x < -104.0f) {
        x = -104.0f;
    }
    float n = nearbyintf(x * 1.44269504088896341f);
    float r = fmaf(n, -0.693359375f, x);
    r = fmaf(n, 2.12194440e-4f, r);
    float p = 1.9875691500e-4f;
    p = fmaf(p, r, 1.3981999507e-3f);
    p = fmaf(p, r, 8.3334519073e-3f);
    p = fmaf(p, r, 4.1665795894e-2f);
    p = fmaf(p, r, 1.6666665459e-1f);
    p = fmaf(p, r, 5.0000001201e-1f);
    float r2 = r * r;
    float e = fmaf(p, r2, r);
    e = e + 1.0f;
    int ni = (int)n; /* |n| <= 151 */
    int n1 = ni >> 1;
    int n2 = ni - n1;
    float s1 = u2f((uint32_t)(n1 + 127) << 23);
    float s2 = u2f((uint32_t)(n2 + 127) << 23);
    return (e * s1) * s2;
}

float oracle_silu(float l, int exp_kind)
{
    float t = l * -1.0f;
    float e = (exp_kind == W8A8_EXP_LIBM) ? expf(t) : oracle_expf(t);
    e = e + 1.0f;
    return l / e;
}

/* ------------------------------------------------------------------------ */
/* GroupedMatmulSwigluQuant                                                  */
/* GMSQ/op_kernel/gmsq_vec_kernel.cpp:15-20 (math), :48-49 (FLT_MIN clamp,   */
/* 1/127 constant), :160-167 (expert of a row from the cumulative list),     */
/* :207-212 (dequant: (float(acc) * xScale[i]) * wScale[g, j], per-token     */
/* first), :213-218 (silu on the LEFT half, times the right half), :223-235  */
/* (row magnitude, then !(amax > FLT_MIN) -> FLT_MIN), :236 (y_scale =       */
/* amax * (1/127)), :240 (inv = 127 / amax), :253-257 (clamp to [-128,127],  */
/* two-step narrowing).                                                      */
/*                                                                           */
/* Choices where the Ascend instruction semantics are not documented: the    */
/* row magnitude ignores NaN activations (fmaxf), and a NaN activation       */
/* narrows to 0 (the reference states that for its int8 cast at             */
/* DQ/op_kernel/dynamic_quant_kernel.cpp:22-26).                             */
/* ------------------------------------------------------------------------ */
static int check_group_list(const int64_t* gl, int64_t E, int64_t M)
{
    int64_t prev = 0;
    for (int64_t g = 0; g < E; ++g) {
        if (gl[g] < prev || gl[g] > M) {
            return -1;
        }
        prev = gl[g];
    }
    return (prev == M) ? 0 : -1;
}

int oracle_grouped_matmul_swiglu_quant(const int8_t* x, const int8_t* w, const float* w_scale,
                                       const float* x_scale, const int64_t* group_list, int8_t* y,
                                       float* y_scale, int64_t M, int64_t K, int64_t N, int64_t E,
                                       int w_transposed, int round_mode, int exp_kind,
                                       float* act_out)
{
    if (M < 0 || K <= 0 || N <= 0 || (N & 1) || E <= 0) {
        return -1;
    }
    if (check_group_list(group_list, E, M) != 0) {
        return -1;
    }
    const int64_t H = N / 2;
    const float tiny = 1.1754944e-38f;
    const float inv127 = 1.0f / 127.0f;
    /* expert of every row */
    int32_t* row_g = (int32_t*)malloc(sizeof(int32_t) * (size_t)(M > 0 ? M : 1));
    {
        int64_t g = 0;
        for (int64_t r = 0; r < M; ++r) {
            while (g < E && r >= group_list[g]) {
                ++g;
            }
            row_g[r] = (int32_t)(g < E ? g : E - 1);
        }
    }
#pragma omp parallel
    {
        int32_t* acc = (int32_t*)malloc(sizeof(int32_t) * (size_t)N);
        float* act = (float*)malloc(sizeof(float) * (size_t)H);
#pragma omp for schedule(dynamic, 4)
        for (int64_t r = 0; r < M; ++r) {
            const int64_t g = row_g[r];
            i8_row_times_matrix(x + r * K, w + g * K * N, acc, K, N, w_transposed ? K : N,
                                w_transposed);
            const float xs = x_scale[r];
            const float* ws = w_scale + g * N;
            float amax = 0.0f;
            for (int64_t j = 0; j < H; ++j) {
                float l = ((float)acc[j] * xs) * ws[j];
                float u = ((float)acc[H + j] * xs) * ws[H + j];
                float a = oracle_silu(l, exp_kind) * u;
                act[j] = a;
                amax = fmaxf(amax, fabsf(a));
            }
            if (act_out != NULL) {
                memcpy(act_out + r * H, act, sizeof(float) * (size_t)H);
            }
            if (!(amax > tiny)) {
                amax = tiny;
            }
            y_scale[r] = amax * inv127;
            const float inv = 127.0f / amax;
            for (int64_t j = 0; j < H; ++j) {
                float v = act[j] * inv;
                if (v == v) {
                    if (v > 127.0f) {
                        v = 127.0f;
                    }
                    if (v < -128.0f) {
                        v = -128.0f;
                    }
                }
                y[r * H + j] = oracle_narrow_i8(v, round_mode);
            }
        }
        free(acc);
        free(act);
    }
    free(row_g);
    return 0;
}

/* ------------------------------------------------------------------------ */
/* GroupedMatmul                                                             */
/* GMM/op_kernel/grouped_matmul_kernel.cpp:15-16 (math: y[rows_g] =          */
/* x[rows_g] @ weight[g] (+ bias[g])), :123-150 (per task operands; the      */
/* library accumulates in fp32 and the result takes x's dtype),              */
/* GMM/op_kernel/grouped_matmul_launch.h:55-63 (weight [E,K,N] or [E,N,K]).  */
/* The library's fp32 accumulation order is unknown: the float path here     */
/* adds in ascending k and is compared with a tolerance.                     */
/*                                                                           */
/* dtype == W8A8_DT_I8 is this project's extension for the quantised down    */
/* projection (the reference operator has no int8 path): int32 accumulate,   */
/* then (float(acc) * w_scale[g, n]) * x_scale[m] -- the QuantMatmul order   */
/* (QM/op_kernel/quant_matmul_epilogue_kernel.cpp:274-293) -- optional fp32- */
/* widened bias added last, RNE to out_dtype.                                */
/* ------------------------------------------------------------------------ */
int oracle_grouped_matmul(const void* x, const void* w, const void* bias, void* y,
                          const float* x_scale, const float* w_scale, const int64_t* group_list,
                          int64_t M, int64_t N, int64_t K, int64_t E, int dtype, int bias_dtype,
                          int out_dtype, int w_transposed)
{
    if (M < 0 || K <= 0 || N <= 0 || E <= 0) {
        return -1;
    }
    if (check_group_list(group_list, E, M) != 0) {
        return -1;
    }
    if (dtype == W8A8_DT_I8 && (x_scale == NULL || w_scale == NULL)) {
        return -1;
    }
    int32_t* row_g = (int32_t*)malloc(sizeof(int32_t) * (size_t)(M > 0 ? M : 1));
    {
        int64_t g = 0;
        for (int64_t r = 0; r < M; ++r) {
            while (g < E && r >= group_list[g]) {
                ++g;
            }
            row_g[r] = (int32_t)(g < E ? g : E - 1);
        }
    }
#pragma omp parallel
    {
        int32_t* acc = (int32_t*)malloc(sizeof(int32_t) * (size_t)N);
        float* facc = (float*)malloc(sizeof(float) * (size_t)N);
        float* xrow = (float*)malloc(sizeof(float) * (size_t)K);
#pragma omp for schedule(dynamic, 4)
        for (int64_t r = 0; r < M; ++r) {
            const int64_t g = row_g[r];
            if (dtype == W8A8_DT_I8) {
                i8_row_times_matrix((const int8_t*)x + r * K, (const int8_t*)w + g * K * N, acc, K,
                                    N, w_transposed ? K : N, w_transposed);
                const float xs = x_scale[r];
                for (int64_t j = 0; j < N; ++j) {
                    float v = ((float)acc[j] * w_scale[g * N + j]) * xs;
                    if (bias != NULL) {
                        v = v + load_as_f32(bias, g * N + j, bias_dtype);
                    }
                    store_from_f32(y, r * N + j, out_dtype, v);
                }
            } else {
                for (int64_t k = 0; k < K; ++k) {
                    xrow[k] = load_as_f32(x, r * K + k, dtype);
                }
                for (int64_t j = 0; j < N; ++j) {
                    facc[j] = 0.0f;
                }
                if (!w_transposed) {
                    for (int64_t k = 0; k < K; ++k) {
                        const float a = xrow[k];
                        for (int64_t j = 0; j < N; ++j) {
                            facc[j] = fmaf(a, load_as_f32(w, (g * K + k) * N + j, dtype), facc[j]);
                        }
                    }
                } else {
                    for (int64_t j = 0; j < N; ++j) {
                        float s = 0.0f;
                        for (int64_t k = 0; k < K; ++k) {
                            s = fmaf(xrow[k], load_as_f32(w, (g * N + j) * K + k, dtype), s);
                        }
                        facc[j] = s;
                    }
                }
                for (int64_t j = 0; j < N; ++j) {
                    float v = facc[j];
                    if (bias != NULL) {
                        v = v + load_as_f32(bias, g * N + j, bias_dtype);
                    }
                    store_from_f32(y, r * N + j, dtype, v);
                }
            }
        }
        free(acc);
        free(facc);
        free(xrow);
    }
    free(row_g);
    return 0;
}

/* ------------------------------------------------------------------------ */
/* Expert-parallel bookkeeping.                                              */
/*                                                                           */
/* oracle_route_count: stable counting sort of the T*topk (token, k) pairs   */
/* by expert.  expanded_pos[i*topk + k] is the row that pair occupies in the */
/* expert-major expanded matrix; cumsum is the group list the grouped        */
/* matmuls consume.  Within an expert, pairs keep (token, k) lexicographic   */
/* order, which is the order a rank-major all-to-all followed by the         */
/* MoeReRouting permutation produces                                         */
/* (MRR/op_kernel/moe_re_routing_kernel.cpp:15-24).                          */
/* ------------------------------------------------------------------------ */
int oracle_route_count(const int32_t* expert_idx, int64_t T, int64_t topk, int64_t E,
                       int64_t* count_per_expert, int64_t* cumsum, int64_t* expanded_pos)
{
    if (T < 0 || topk <= 0 || E <= 0) {
        return -1;
    }
    for (int64_t e = 0; e < E; ++e) {
        count_per_expert[e] = 0;
    }
    for (int64_t i = 0; i < T * topk; ++i) {
        int32_t e = expert_idx[i];
        if (e < 0 || e >= E) {
            return -1;
        }
        count_per_expert[e]++;
    }
    int64_t run = 0;
    int64_t* next = (int64_t*)malloc(sizeof(int64_t) * (size_t)E);
    for (int64_t e = 0; e < E; ++e) {
        next[e] = run;
        run += count_per_expert[e];
        cumsum[e] = run;
    }
    for (int64_t i = 0; i < T * topk; ++i) {
        expanded_pos[i] = next[expert_idx[i]]++;
    }
    free(next);
    return 0;
}

int oracle_gather_rows(const void* src, void* dst, const int64_t* src_row, int64_t rows,
                       int64_t row_bytes)
{
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r) {
        memcpy((char*)dst + r * row_bytes, (const char*)src + src_row[r] * row_bytes,
               (size_t)row_bytes);
    }
    return 0;
}

/* Combine: out[i, c] = sum_k probs[i, k] * rows[p(i, k), c], fp32, ascending
 * k, RNE narrowing (MFR/op_kernel/moe_finalize_routing_kernel.cpp:15-25 with
 * no skip and no bias; p(i,k) row-arranged as in drop_pad_mode 2/3).  A
 * position outside [0, rows) contributes nothing. */
int oracle_combine(const void* rows, const float* probs, const int64_t* expanded_pos, void* out,
                   int64_t T, int64_t topk, int64_t H, int dtype)
{
    if (dtype != W8A8_DT_F16 && dtype != W8A8_DT_BF16 && dtype != W8A8_DT_F32) {
        return -1;
    }
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < T; ++i) {
        for (int64_t c = 0; c < H; ++c) {
            float acc = 0.0f;
            for (int64_t k = 0; k < topk; ++k) {
                int64_t p = expanded_pos[i * topk + k];
                if (p < 0) {
                    continue;
                }
                float v = load_as_f32(rows, p * H + c, dtype);
                acc = acc + probs[i * topk + k] * v;
            }
            store_from_f32(out, i * H + c, dtype, acc);
        }
    }
    return 0;
}

/* ------------------------------------------------------------------------ */
/* MoeReRouting                                                              */
/* MRR/op_kernel/moe_re_routing_kernel.cpp:15-24 (semantics), same text in   */
/* MRR/op_kernel/moe_re_routing_launch.h:15-21:                              */
/*   srcStart(i,j) = sum_{i'<i} rowSum(i') + sum_{j'<j} cnt[i][j']           */
/*   dstStart(i,j) = sum_{j'<j} colSum(j') + sum_{i'<i} cnt[i'][j]           */
/*   out[dstStart+k] = in[srcStart+k], idx[dstStart+k] = srcStart+k,         */
/*   expert_token_num[j] = colSum(j) (count mode; the plugin ignores         */
/*   expert_token_num_type, MRR/op_plugin/moe_re_routing_plugin.cpp:75).     */
/* ------------------------------------------------------------------------ */
int oracle_moe_re_routing(const void* tokens, const int64_t* counts, const float* scales, void* out_tokens,
                          float* out_scales, int32_t* out_idx, int64_t* expert_token_num, int64_t A,
                          int64_t row_bytes, int64_t N, int64_t E)
{
    if (A < 0 || row_bytes <= 0 || N <= 0 || E <= 0) {
        return -1;
    }
    int64_t total = 0;
    for (int64_t i = 0; i < N * E; ++i) {
        if (counts[i] < 0) {
            return -1;
        }
        total += counts[i];
    }
    if (total > A) {
        return -1;
    }
    int64_t col_start = 0;
    for (int64_t j = 0; j < E; ++j) {
        int64_t col_sum = 0;
        int64_t row_start = 0;
        for (int64_t i = 0; i < N; ++i) {
            int64_t before = 0; /* sum_{j'<j} cnt[i][j'] */
            for (int64_t jj = 0; jj < j; ++jj) {
                before += counts[i * E + jj];
            }
            const int64_t src = row_start + before;
            const int64_t dst = col_start + col_sum;
            const int64_t c = counts[i * E + j];
#pragma omp parallel for schedule(static) if (c * row_bytes > (1 << 16))
            for (int64_t k = 0; k < c; ++k) {
                memcpy((char*)out_tokens + (dst + k) * row_bytes, (const char*)tokens + (src + k) * row_bytes,
                       (size_t)row_bytes);
                if (scales != NULL && out_scales != NULL) {
                    out_scales[dst + k] = scales[src + k];
                }
                out_idx[dst + k] = (int32_t)(src + k);
            }
            col_sum += c;
            int64_t row_sum = 0;
            for (int64_t jj = 0; jj < E; ++jj) {
                row_sum += counts[i * E + jj];
            }
            row_start += row_sum;
        }
        expert_token_num[j] = col_sum;
        col_start += col_sum;
    }
    return 0;
}

/* ------------------------------------------------------------------------ */
/* MoeFinalizeRouting                                                        */
/* MFR/op_kernel/moe_finalize_routing_kernel.cpp:15-25 (formula), :133-181   */
/* (one term: fp32(row) [+ fp32(bias[eid])], then * fp32(scale), then added   */
/* to the accumulator), :231-245 (accumulator starts as fp32(skip1) and       */
/* fp32(skip2) is added to it), :432-437 (round-to-nearest-even store).       */
/*   p(i,k) = esdr[k*R + i] (drop_pad_mode 0/1) or esdr[i*K + k] (2/3);       */
/*   p outside [0, num_dst) drops the whole term; eid outside [0, E) drops    */
/*   only the bias; scales / expert are indexed [i*K + k] in every mode.      */
/* ------------------------------------------------------------------------ */
int oracle_moe_finalize_routing(const void* rows, const int32_t* esdr, const void* skip1, const void* skip2,
                                const void* bias, const void* scales, const int32_t* expert, void* out,
                                int64_t R, int64_t H, int64_t K, int64_t E, int64_t num_dst, int drop_pad_mode,
                                int dtype, int scale_dtype)
{
    if (dtype != W8A8_DT_F16 && dtype != W8A8_DT_BF16 && dtype != W8A8_DT_F32) {
        return -1;
    }
    if (scales != NULL && scale_dtype != W8A8_DT_F16 && scale_dtype != W8A8_DT_BF16 && scale_dtype != W8A8_DT_F32) {
        return -1;
    }
    if (R < 0 || H <= 0 || K <= 0 || num_dst < 0) {
        return -1;
    }
    const int col_mode = (drop_pad_mode <= 1);
    const int has_bias = (bias != NULL && expert != NULL);
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < R; ++i) {
        for (int64_t c = 0; c < H; ++c) {
            float acc = (skip1 != NULL) ? load_as_f32(skip1, i * H + c, dtype) : 0.0f;
            if (skip2 != NULL) {
                acc = acc + load_as_f32(skip2, i * H + c, dtype);
            }
            for (int64_t k = 0; k < K; ++k) {
                const int64_t p = esdr[col_mode ? (k * R + i) : (i * K + k)];
                if (p < 0 || p >= num_dst) {
                    continue;
                }
                float term = load_as_f32(rows, p * H + c, dtype);
                if (has_bias) {
                    const int64_t eid = expert[i * K + k];
                    if (eid >= 0 && eid < E) {
                        term = term + load_as_f32(bias, eid * H + c, dtype);
                    }
                }
                if (scales != NULL) {
                    term = term * load_as_f32(scales, i * K + k, scale_dtype);
                }
                acc = acc + term;
            }
            store_from_f32(out, i * H + c, dtype, acc);
        }
    }
    return 0;
}

/* ------------------------------------------------------------------------ */
/* MoeGatingTopKSoftmax                                                      */
/* MGT/op_kernel/moe_gating_kernel.cpp:14-21 (formula), :305-339 (max, x-max, */
/* exp, sum), :344-368 (descending sort with indices), :390-392 (divide the   */
/* selected values by the row sum, round to the input type).  The reference   */
/* leaves the summation order and the exp implementation to its hardware;     */
/* here the sum runs over 32 lanes (lane t adds elements t, t+32, ... in      */
/* ascending order, then a butterfly over distances 16, 8, 4, 2, 1) and exp   */
/* is oracle_expf, both shared with the CUDA kernel.  Equal values: lower     */
/* column first.                                                              */
/* ------------------------------------------------------------------------ */
int oracle_moe_gating_top_k_softmax(const void* x, const uint8_t* finished, void* y, int32_t* expert_idx,
                                    int32_t* row_idx, int64_t rows, int64_t inner, int64_t k, int dtype)
{
    if (dtype != W8A8_DT_F16 && dtype != W8A8_DT_BF16 && dtype != W8A8_DT_F32) {
        return -1;
    }
    if (rows < 0 || inner <= 0 || k <= 0 || k > inner) {
        return -1;
    }
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r) {
        float* e = (float*)malloc((size_t)inner * sizeof(float));
        float m = -INFINITY;
        for (int64_t c = 0; c < inner; ++c) {
            e[c] = load_as_f32(x, r * inner + c, dtype);
            m = fmaxf(m, e[c]);
        }
        float lane[32];
        for (int t = 0; t < 32; ++t) {
            lane[t] = 0.0f;
        }
        for (int64_t c = 0; c < inner; ++c) {
            e[c] = oracle_expf(e[c] - m);
            lane[c & 31] = lane[c & 31] + e[c];
        }
        for (int off = 16; off > 0; off >>= 1) {
            float next[32];
            for (int t = 0; t < 32; ++t) {
                next[t] = lane[t] + lane[t ^ off];
            }
            memcpy(lane, next, sizeof(lane));
        }
        const float sum = lane[0];
        for (int64_t j = 0; j < k; ++j) {
            int64_t best = -1;
            for (int64_t c = 0; c < inner; ++c) {
                if (e[c] >= 0.0f && (best < 0 || e[c] > e[best])) {
                    best = c;
                }
            }
            const float val = (best >= 0) ? e[best] : NAN;
            store_from_f32(y, r * k + j, dtype, val / sum);
            expert_idx[r * k + j] = (finished != NULL && finished[r]) ? (int32_t)inner : (int32_t)best;
            row_idx[r * k + j] = (int32_t)(j * rows + r);
            if (best >= 0) {
                e[best] = -1.0f;
            }
        }
        free(e);
    }
    return 0;
}

/* ------------------------------------------------------------------------ */
/* DequantSwigluQuant                                                        */
/* DQSQ/op_kernel/dqsq_kernel.cpp, in the order its vector instructions run: */
/* weight_scale (:335-347), quant_scale on the half that is not the gate     */
/* input (:349-363), activation_scale on both halves (:386-410), the gate    */
/* out = (a*b) / (1 + exp(gate * -1)) (:415-428), row maximum with           */
/* not-greater-than-zero read as 0 (:489-495), s = max(m*(1/127), 1e-12)     */
/* (:496-499), out / s in the batched short-row layout (:482) and            */
/* out * (1/s) otherwise (:500-504): here the division is used when the      */
/* half-row padded to 32 bytes of the input type is at most 1984 elements    */
/* (:97), the reciprocal for longer rows; clamp to [-128, 127] (:509-510),   */
/* fp32 -> fp16 -> int8 (:516-524).  A NaN activation quantises to 0.        */
/* ------------------------------------------------------------------------ */
int oracle_dequant_swiglu_quant(const void* x, const float* weight_scale, const float* activation_scale,
                                const float* quant_scale, int8_t* y, float* scale, int64_t M, int64_t H,
                                int x_dtype, int activate_left, int round_mode, float* out_f32)
{
    const int is_i32 = (x_dtype == W8A8_DT_I32);
    if (!is_i32 && x_dtype != W8A8_DT_F16 && x_dtype != W8A8_DT_BF16) {
        return -1;
    }
    if (M < 0 || H <= 0 || is_i32 != (weight_scale != NULL) || is_i32 != (activation_scale != NULL)) {
        return -1;
    }
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < M; ++r) {
        float* out = (float*)malloc((size_t)H * sizeof(float));
        float m = 0.0f;
        for (int64_t j = 0; j < H; ++j) {
            float a, b;
            if (is_i32) {
                a = (float)((const int32_t*)x)[r * 2 * H + j] * weight_scale[j];
                b = (float)((const int32_t*)x)[r * 2 * H + H + j] * weight_scale[H + j];
            } else {
                a = load_as_f32(x, r * 2 * H + j, x_dtype);
                b = load_as_f32(x, r * 2 * H + H + j, x_dtype);
            }
            if (quant_scale != NULL) {
                if (activate_left) {
                    b = b * quant_scale[j];
                } else {
                    a = a * quant_scale[j];
                }
            }
            if (is_i32) {
                a = a * activation_scale[r];
                b = b * activation_scale[r];
            }
            const float gate = activate_left ? a : b;
            const float den = oracle_expf(gate * -1.0f) + 1.0f;
            out[j] = (a * b) / den;
            m = fmaxf(m, fabsf(out[j]));
            if (out_f32 != NULL) {
                out_f32[r * H + j] = out[j];
            }
        }
        float s = m * (1.0f / 127.0f);
        if (s < 1e-12f) {
            s = 1e-12f;
        }
        scale[r] = s;
        const int64_t pad = is_i32 ? 8 : 16;
        const int divide = ((H + pad - 1) / pad * pad <= 1984);
        const float inv = 1.0f / s;
        for (int64_t j = 0; j < H; ++j) {
            float q = divide ? out[j] / s : out[j] * inv;
            if (q != q) {
                y[r * H + j] = 0;
                continue;
            }
            q = fmaxf(fminf(q, 127.0f), -128.0f);
            y[r * H + j] = oracle_narrow_i8(q, round_mode);
        }
        free(out);
    }
    return 0;
}
