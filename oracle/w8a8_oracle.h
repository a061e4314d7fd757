/*
 * CPU oracle for the W8A8 quantised-FFN operators.  TEST INFRASTRUCTURE ONLY.
 *
 * This is a scalar C restatement of the arithmetic of five operators of
 * ai-jiaqian/cannbench-operator-solutions, written from the formulas in the
 * reference kernels (file:line given on every function; paths are relative to
 * the reference project root).  It exists to check the CUDA library and to be
 * timed as the CPU baseline.  Nothing in the product library links, loads or
 * calls it; only tests, the smoke check and the benchmark's CPU legs do.
 *
 * Parity status: the reference ships no golden vectors and no tests, and its
 * kernels only compile with the Ascend toolchain, so this oracle is pinned
 * only by (a) the formulas in the reference sources and (b) the hand-derived
 * known-answer cases in tests/golden/.  PARITY UNPINNED against reference
 * outputs.
 *
 * Rounding modes
 *   W8A8_ROUND_AS_WRITTEN  fp32 -> fp16 (RNE) -> int8 (RNE, saturating): the
 *                          two-step narrowing every reference kernel performs.
 *   W8A8_ROUND_DIRECT      fp32 -> int8 (RNE, saturating) in one step.
 */
#ifndef W8A8_ORACLE_H
#define W8A8_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define W8A8_DT_F16 0
#define W8A8_DT_BF16 1
#define W8A8_DT_F32 2
#define W8A8_DT_I8 3
#define W8A8_DT_I32 4

#define W8A8_ROUND_AS_WRITTEN 0
#define W8A8_ROUND_DIRECT 1

/* sum-of-squares order for add_rms_norm_dynamic_quant */
#define W8A8_SUM_CANONICAL 0 /* the 256-lane order the CUDA kernel uses  */
#define W8A8_SUM_FP64 1      /* sequential double accumulation (tolerance) */

/* exp() used inside silu */
#define W8A8_EXP_CANONICAL 0 /* w8a8_expf below, shared with the CUDA code */
#define W8A8_EXP_LIBM 1      /* libm expf (tolerance reporting)            */

/* quant_matmul epilogue flag word: same bit layout as the reference's QM_F_*
 * (operators/quantmatmul/csrc/ops/quant_matmul/op_kernel/quant_matmul_launch.h:39-53) */
#define W8A8_QM_SCALE_PERCHAN (1LL << 0)
#define W8A8_QM_SCALE_BF16 (1LL << 1)
#define W8A8_QM_HAS_OFFSET (1LL << 2)
#define W8A8_QM_OFFSET_PERCHAN (1LL << 3)
#define W8A8_QM_HAS_PT (1LL << 4)
#define W8A8_QM_BIAS_SHIFT 5
#define W8A8_QM_BIAS_MASK (7LL << W8A8_QM_BIAS_SHIFT)
#define W8A8_QM_BIAS_PERCHAN (1LL << 8)
#define W8A8_QM_PT_MOD_M (1LL << 9)
#define W8A8_QM_BIAS_NONE 0
#define W8A8_QM_BIAS_I32 1
#define W8A8_QM_BIAS_F16 2
#define W8A8_QM_BIAS_BF16 3
#define W8A8_QM_BIAS_F32 4

/* scalar helpers (exported so tests can pin them) */
float oracle_bf16_to_f32(uint16_t h);
float oracle_f16_to_f32(uint16_t h);
uint16_t oracle_f32_to_bf16(float f);
uint16_t oracle_f32_to_f16(float f);
int8_t oracle_narrow_i8(float v, int round_mode);
float oracle_expf(float x);
float oracle_silu(float l, int exp_kind);

int oracle_dynamic_quant(const void* x, int8_t* y, float* scale, int64_t M, int64_t N, int dtype,
                         int round_mode);

int oracle_add_rms_norm_dynamic_quant(const void* x1, const void* x2, const void* gamma, int8_t* y,
                                      void* x_out, float* scale_out, int64_t rows, int64_t N,
                                      float eps, int dtype, int round_mode, int sum_order);

/* acc_out (optional) receives the raw int32 product [batch*M, N]. */
int oracle_quant_matmul(const int8_t* x1, const int8_t* x2, const void* scale, const float* offset,
                        const float* pertoken, const void* bias, void* out, int64_t batch,
                        int64_t M, int64_t N, int64_t K, int64_t flags, int out_dtype,
                        int x2_transposed, int32_t* acc_out);

/* act_out (optional) receives the fp32 SwiGLU activations [M, N/2]. */
int oracle_grouped_matmul_swiglu_quant(const int8_t* x, const int8_t* w, const float* w_scale,
                                       const float* x_scale, const int64_t* group_list, int8_t* y,
                                       float* y_scale, int64_t M, int64_t K, int64_t N, int64_t E,
                                       int w_transposed, int round_mode, int exp_kind,
                                       float* act_out);

/* dtype = F16/BF16/F32: the reference's float path.  dtype = I8: int8 x/w with
 * fp32 x_scale[M], w_scale[E,N] and out_dtype (F16/BF16) output.           */
int oracle_grouped_matmul(const void* x, const void* w, const void* bias, void* y,
                          const float* x_scale, const float* w_scale, const int64_t* group_list,
                          int64_t M, int64_t N, int64_t K, int64_t E, int dtype, int bias_dtype,
                          int out_dtype, int w_transposed);

/* Expert-parallel bookkeeping and the combine arithmetic. */
int oracle_route_count(const int32_t* expert_idx, int64_t T, int64_t topk, int64_t E,
                       int64_t* count_per_expert, int64_t* cumsum, int64_t* expanded_pos);
int oracle_gather_rows(const void* src, void* dst, const int64_t* src_row, int64_t rows,
                       int64_t row_bytes);
int oracle_combine(const void* rows, const float* probs, const int64_t* expanded_pos, void* out,
                   int64_t T, int64_t topk, int64_t H, int dtype);

/* MoeReRouting: regroup a rank-major / expert-minor token buffer (what an all-to-all delivers) into expert-major
 * order.  counts[i*E + j] = rows received from rank i for local expert j.  row_bytes is the byte length of a token
 * row; scales / out_scales may be NULL. */
int oracle_moe_re_routing(const void* tokens, const int64_t* counts, const float* scales, void* out_tokens,
                          float* out_scales, int32_t* out_idx, int64_t* expert_token_num, int64_t A,
                          int64_t row_bytes, int64_t N, int64_t E);

/* MoeFinalizeRouting: out[i] = skip1[i] + skip2[i] + sum_k scales[i,k] * (rows[p(i,k)] + bias[expert[i,k]]),
 * fp32, ascending k, RNE store.  Every optional operand may be NULL (bias needs expert). */
int oracle_moe_finalize_routing(const void* rows, const int32_t* esdr, const void* skip1, const void* skip2,
                                const void* bias, const void* scales, const int32_t* expert, void* out,
                                int64_t R, int64_t H, int64_t K, int64_t E, int64_t num_dst, int drop_pad_mode,
                                int dtype, int scale_dtype);

/* MoeGatingTopKSoftmax: softmax over the last dimension, the k largest probabilities (lower column first among
 * equals), their columns (inner for finished rows) and row_idx = j * rows + r. */
int oracle_moe_gating_top_k_softmax(const void* x, const uint8_t* finished, void* y, int32_t* expert_idx,
                                    int32_t* row_idx, int64_t rows, int64_t inner, int64_t k, int dtype);

/* DequantSwigluQuant: x [M, 2H] int32 (with weight_scale [2H], activation_scale [M]) or F16 / BF16;
 * out_f32 (optional) receives the fp32 activations before quantisation. */
int oracle_dequant_swiglu_quant(const void* x, const float* weight_scale, const float* activation_scale,
                                const float* quant_scale, int8_t* y, float* scale, int64_t M, int64_t H,
                                int x_dtype, int activate_left, int round_mode, float* out_f32);

int oracle_num_threads(void);

#ifdef __cplusplus
}
#endif
#endif
