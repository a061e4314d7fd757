/*
 * libw8a8ffn -- C ABI of the B200 (sm_100a) W8A8 quantised-FFN operators.
 *
 * Every entry point is the CUDA counterpart of one launcher (or launcher
 * pair) of the Ascend operator catalog ai-jiaqian/cannbench-operator-solutions;
 * the comment on each declaration names the reference interface it replaces
 * (paths relative to that project's root).  The Ascend tiling arguments
 * (numBlocks, rowsPerCore, ...) have no meaning here and are dropped: tiling
 * is internal.
 *
 * Conventions
 *   - All pointers are DEVICE pointers unless the parameter says "host".
 *   - The caller owns every buffer, including workspaces, whose size comes
 *     from the matching *_workspace_size() query.  The library allocates
 *     nothing and keeps no mutable global state besides cached function
 *     attributes, the kernel-shape override of w8a8_set_gemm_shape() and the
 *     one deliberate exception: the device scratch built into the library
 *     image that w8a8_grouped_matmul_swiglu_quant_static() works in.
 *   - Work is enqueued on `stream` (a cudaStream_t passed as void*; NULL is
 *     the legacy default stream) and the call returns without synchronising.
 *   - Return value: W8A8_OK or a negative W8A8_ERR_* code.  Nothing throws.
 *     A call with zero rows is a successful no-op, as in the reference
 *     plugins.
 *   - dtype codes: W8A8_DT_F16 / W8A8_DT_BF16 / W8A8_DT_F32 / W8A8_DT_I8 / W8A8_DT_I32.
 *   - Row-major, densely packed tensors.  Rows that are 16-byte aligned
 *     take the vectorised kernels; anything else takes a slower generic path
 *     with identical results.
 */
#ifndef W8A8FFN_H
#define W8A8FFN_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define W8A8_OK 0
#define W8A8_ERR_INVALID (-1)     /* bad shape, dtype, flag or null pointer          */
#define W8A8_ERR_ALIGN (-2)       /* a pointer or pitch misses a required alignment   */
#define W8A8_ERR_GROUP_LIST (-3)  /* group list not a non-decreasing cumsum ending at M */
#define W8A8_ERR_WORKSPACE (-4)   /* workspace missing or too small                   */
#define W8A8_ERR_CUDA (-5)        /* a CUDA runtime / driver call failed              */
#define W8A8_ERR_UNSUPPORTED (-6) /* valid in the reference, not implemented here     */
#define W8A8_ERR_LIMIT (-7)       /* problem larger than a fixed built-in capacity     */

#define W8A8_DT_F16 0
#define W8A8_DT_BF16 1
#define W8A8_DT_F32 2
#define W8A8_DT_I8 3
#define W8A8_DT_I32 4

/* `flags` of the quantising operators */
#define W8A8_F_ROUND_DIRECT 1 /* fp32 -> int8 in one rounding instead of the
                                 reference's fp32 -> fp16 -> int8 */

/* grouped_matmul_swiglu_quant only: run one of its two stages, which the
 * reference exposes as two launchers (launch_gmsq_cube, launch_gmsq_vec).
 * Neither bit set = both stages.  The workspace carries the activations and
 * row maxima from the first stage to the second. */
#define W8A8_F_STAGE_MATMUL 2  /* plan + tensor-core matmul + fused dequant/SwiGLU/row-max */
#define W8A8_F_STAGE_REQUANT 4 /* per-row requantisation of the stored activations        */

/* weight layout of the matmuls */
#define W8A8_W_KN 0 /* [.., K, N], N contiguous: the reference's layout       */
#define W8A8_W_NK 1 /* [.., N, K], K contiguous: transpose_weight=True layout */

/* quant_matmul epilogue flag word; identical bit layout to the reference's
 * QM_F_* (operators/quantmatmul/csrc/ops/quant_matmul/op_kernel/quant_matmul_launch.h:39-53) */
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

/* Library identification and error text. */
int w8a8_version(void);

/* Kernels this library has launched so far in this process (every entry point counts its own launches; memsets
 * and copies are not kernels).  Difference two readings to count the launches of a region. */
int64_t w8a8_kernel_launch_count(void);
const char* w8a8_status_string(int status);

/*
 * DynamicQuant: per-row absmax int8 quantisation of x[M, N] (fp16 / bf16).
 *   scale[m] = max(amax_m, 1e-12) * (1/127);  y = narrow(x * ((1/amax_m) * 127))
 * Replaces launch_dynamic_quant_half / launch_dynamic_quant_bfloat16
 * (operators/dynamicquant/csrc/ops/dynamic_quant/op_kernel/dynamic_quant_launch.h:29-41).
 */
int w8a8_dynamic_quant(const void* x, int8_t* y, float* scale, int64_t M, int64_t N, int dtype,
                       int flags, void* stream);

/*
 * AddRmsNormDynamicQuant: x_out = x1 + x2 (rounded to dtype on store),
 * RMSNorm * gamma, per-row absmax int8 quantisation.  N <= 16384.
 * Replaces launch_ardq_half / launch_ardq_bf16
 * (operators/addrmsnormdynamicquant/csrc/ops/add_rms_norm_dynamic_quant/op_kernel/add_rms_norm_dynamic_quant_launch.h:32-41).
 */
int w8a8_add_rms_norm_dynamic_quant(const void* x1, const void* x2, const void* gamma, int8_t* y,
                                    void* x_out, float* scale_out, int64_t rows, int64_t N,
                                    float epsilon, int dtype, int flags, void* stream);

/*
 * QuantMatmul: out[b] = epilogue(x1[b] @ x2[b]), int8 x int8 -> int32 on the
 * tensor cores with the dequant chain fused into the epilogue (no int32
 * workspace):  ((float(acc) + i32bias) * scale + offset) * pertoken + fbias,
 * rounded to out_dtype (F16 or BF16).
 * Replaces the pair qm_launch_cube_i32 + qm_launch_epilogue_{f16,bf16} and the
 * tiling helper qm_calc_cube_tiling
 * (operators/quantmatmul/csrc/ops/quant_matmul/op_kernel/quant_matmul_launch.h:80-99).
 *   x1 int8 [batch, M, K]; x2 int8 [batch, K, N] (W8A8_W_KN) or [batch, N, K]
 *   (W8A8_W_NK); scale fp32|bf16 [1|N]; offset fp32 [1|N] or NULL; pertoken
 *   fp32 [M] or NULL; bias per flags or NULL, optionally batched [batch, N]
 *   (bias_batch_stride = N elements, else 0).
 * K and N must be multiples of 16.
 */
int w8a8_quant_matmul(const int8_t* x1, const int8_t* x2, const void* scale, const float* offset,
                      const float* pertoken, const void* bias, void* out, int64_t batch, int64_t M,
                      int64_t N, int64_t K, int64_t flags, int out_dtype, int x2_layout,
                      int64_t bias_batch_stride, void* stream);

/*
 * The bare tensor-core stage: c[b] = x1[b] @ x2[b] as exact int32 (no
 * epilogue).  Counterpart of qm_launch_cube_i32
 * (operators/quantmatmul/csrc/ops/quant_matmul/op_kernel/quant_matmul_launch.h:88-90)
 * and launch_gmsq_cube; the fused operators never materialise this matrix,
 * the entry point exists for callers that want the raw accumulators.
 */
int w8a8_matmul_i8_i32(const int8_t* x1, const int8_t* x2, int32_t* c, int64_t batch, int64_t M, int64_t N,
                       int64_t K, int x2_layout, void* stream);

/*
 * GroupedMatmulSwigluQuant: per expert g (rows [cumsum[g-1], cumsum[g])):
 *   acc = x[rows_g] @ w[g]; l = (float(acc[:, :N/2]) * x_scale) * w_scale[g, :N/2];
 *   u likewise for the right half; act = silu(l) * u;
 *   y_scale = max(FLT_MIN, max|act|) * (1/127); y = narrow(clamp(act * (127/amax)))
 * Replaces launch_gmsq_cube + launch_gmsq_vec and the gmsq_calc_* queries
 * (operators/groupedmatmulswigluquant/csrc/ops/grouped_matmul_swiglu_quant/op_kernel/gmsq_launch.h:48-82).
 * The reference carries at most 64 group ends by value; here `group_list` is
 * an int64 cumulative list of length E in host memory (validated, then passed
 * by value, E <= 1024) or in device memory (list_on_device = 1; validated on
 * the device: an invalid list leaves y untouched and sets a flag readable
 * with w8a8_workspace_error()).  list_on_device = 2 is a device list that may
 * end below M: M is then an upper bound (the buffers' row capacity) and rows
 * past the list's last entry are neither read nor written, which lets a
 * caller that only knows the row count on the device launch without a
 * readback.
 *   x int8 [M, K]; w int8 [E, K, N] (W8A8_W_KN) or [E, N, K] (W8A8_W_NK);
 *   w_scale fp32 [E, N]; x_scale fp32 [M]; y int8 [M, N/2]; y_scale fp32 [M].
 * K a multiple of 16, N a multiple of 32.
 */
size_t w8a8_grouped_matmul_swiglu_quant_workspace_size(int64_t M, int64_t K, int64_t N, int64_t E);
int w8a8_grouped_matmul_swiglu_quant(const int8_t* x, const int8_t* w, const float* w_scale,
                                     const float* x_scale, int8_t* y, float* y_scale, int64_t M,
                                     int64_t K, int64_t N, int64_t E, const int64_t* group_list,
                                     int list_on_device, int w_layout, int flags, void* workspace,
                                     size_t workspace_bytes, void* stream);

/*
 * GroupedMatmulSwigluQuant for callers that cannot hand the library a workspace.
 * (No counterpart in the reference: its plugin always allocates the matmul
 * intermediate itself.)
 *
 * Some callers have no way to obtain device memory at the point where they run
 * the operator: code inside a region being captured into a CUDA graph (an
 * allocation there is an error), a serving loop whose memory was handed out
 * once at start-up and whose latency budget cannot absorb the device-wide
 * synchronisation an allocation may cause, or a host that embeds the library
 * behind an interface with no allocator to call back into.  For them this entry
 * point does the same work as w8a8_grouped_matmul_swiglu_quant with the same
 * arguments minus the workspace, using W8A8_STATIC_SCRATCH_BYTES of device
 * memory that are part of the library image.  It calls no allocation routine.
 *
 * Limit: w8a8_grouped_matmul_swiglu_quant_workspace_size(M, K, N, E) must not
 * exceed W8A8_STATIC_SCRATCH_BYTES (for example 1024 rows at N = 4096, or 2048
 * rows at N = 2048, with up to a few hundred experts); larger problems return
 * W8A8_ERR_LIMIT and do nothing.  Every GPU that loads the library holds those
 * bytes until the process exits.
 *
 * The first call on each device looks up the address of the built-in memory
 * (cudaGetSymbolAddress, with that device current).  Make that first call
 * outside any stream capture.
 *
 * All calls on a device share the one scratch area.  A call overwrites what the
 * previous one left and clears what it needs cleared, so back-to-back calls on
 * one stream are fine; two calls whose kernels can overlap on the GPU (different
 * streams without an ordering between them, or several host threads) race on it
 * and give wrong results.  Use the workspace variant for concurrent calls.
 *
 * With a device group list (list_on_device 1 or 2) the list is validated on the
 * GPU and a bad list is reported through an error word, as in the workspace
 * variant; here that word sits in the built-in scratch, so read it with
 * w8a8_static_scratch_error(stream) (synchronises the stream; 0 = none,
 * 1 = invalid device group list and y left untouched, 2 = a pipeline wait ran
 * out).  Host group lists are validated before anything is launched.
 */
#define W8A8_STATIC_SCRATCH_BYTES ((8 << 20) + (64 << 10))
int w8a8_static_scratch_error(void* stream);
int w8a8_grouped_matmul_swiglu_quant_static(const int8_t* x, const int8_t* w, const float* w_scale,
                                            const float* x_scale, int8_t* y, float* y_scale, int64_t M,
                                            int64_t K, int64_t N, int64_t E, const int64_t* group_list,
                                            int list_on_device, int w_layout, int flags, void* stream);

/*
 * GroupedMatmul: y[rows_g] = x[rows_g] @ w[g] (+ bias[g]).
 * Replaces launch_gmm and calc_gmm_workspace_size
 * (operators/groupedmatmul/csrc/ops/grouped_matmul/op_kernel/grouped_matmul_launch.h:50-71).
 *   dtype F16 / BF16: the reference's float path, fp32 accumulate, output in
 *   dtype (x_scale, w_scale NULL).
 *   dtype F32 (the reference's GMM_DT_FLOAT): both operands are split into
 *   three bf16 pieces each and the six leading piece products are accumulated
 *   in fp32 on the bf16 tensor path (what is dropped is below 2^-24 of
 *   |x||w|); output and bias F32; needs the larger workspace of
 *   w8a8_grouped_matmul_f32_workspace_size (room for the split operands).
 *   dtype I8: the quantised down projection the reference operator lacks:
 *   int32 accumulate, (float(acc) * w_scale[g, n]) * x_scale[m] (+ bias),
 *   rounded to out_dtype.
 * group_list as for grouped_matmul_swiglu_quant.
 */
size_t w8a8_grouped_matmul_workspace_size(int64_t M, int64_t N, int64_t K, int64_t E);
size_t w8a8_grouped_matmul_f32_workspace_size(int64_t M, int64_t N, int64_t K, int64_t E);
int w8a8_grouped_matmul(const void* x, const void* w, const void* bias, void* y,
                        const float* x_scale, const float* w_scale, int64_t M, int64_t N, int64_t K,
                        int64_t E, const int64_t* group_list, int list_on_device, int dtype,
                        int bias_dtype, int out_dtype, int w_layout, void* workspace,
                        size_t workspace_bytes, void* stream);

/*
 * Test and tuning hook (no reference counterpart): forces the tensor-core kernel shape for every later matmul
 * call of the process.  0 = the library's own choice (the default), 1 = one CTA per 128-row tile, 2 = CTA pairs
 * (cta_group::2) on 256-row tiles, 3 = grouped problems as pairs on whole 256-row blocks plus single CTAs on the
 * leftovers (dense problems ignore 3).  Every shape gives identical results.  Returns the previous setting, or
 * W8A8_ERR_INVALID.
 */
int w8a8_set_gemm_shape(int shape);

/* Test and tuning hook (no reference counterpart): grouped_matmul_swiglu_quant requantises in a second kernel over
 * the stored activations (on = 0, the default) or inside the matmul kernels (on = 1): the CTAs that compute the
 * column tiles of a row block each quantise a share of its rows one tile later, once all column tiles have been
 * counted.  Identical results and, measured, the same time to within 2 % and the same DRAM traffic; the fused form
 * has one launch less, but its CTAs wait for one another (bounded; error word 2), which assumes that
 * the CTAs of the launch are resident together.  Used only when N / 2 spans at most half as many 128-column tiles
 * as the GPU has SMs; otherwise the call runs the second kernel.  Returns the previous setting. */
int w8a8_set_gmsq_fused_requant(int on);

/* Test and tuning hook (no reference counterpart): how many warps of the grouped_matmul_swiglu_quant kernels run the
 * dequant / SwiGLU / row-max epilogue, 8 or 16 (default 16).  Identical results.  Returns the previous setting, or
 * W8A8_ERR_INVALID. */
int w8a8_set_gmsq_epilogue_warps(int warps);


/* Reads (synchronously, on `stream`) the device-side error word a grouped
 * call left in its workspace: 0 = none, 1 = invalid device group list,
 * 2 = a pipeline wait ran out. */
int w8a8_workspace_error(const void* workspace, void* stream);

/* The same report for the matmuls that take no workspace (w8a8_quant_matmul, w8a8_matmul_i8_i32): reads
 * (synchronously, on `stream`) and clears the current device's error word, 0 = none, 2 = a pipeline wait ran out
 * since the last read (the output of that call is incomplete). */
int w8a8_pipeline_error(void* stream);

/*
 * Expert-parallel helpers (the layout contract of MoeReRouting and the
 * arithmetic of MoeFinalizeRouting, which the reference keeps in separate
 * operators: operators/moererouting/csrc/ops/moe_re_routing/op_kernel/moe_re_routing_launch.h:15-21,
 * operators/moefinalizerouting/csrc/ops/moe_finalize_routing/op_kernel/moe_finalize_routing_kernel.cpp:15-25).
 *
 * w8a8_route_plan: stable counting sort of the T*topk (token, k) pairs by
 * expert.  Writes count[E], the inclusive cumsum[E] (the group list) and
 * expanded_pos[T*topk] (row of each pair in expert-major order), all int64.
 * workspace: w8a8_route_plan_workspace_size(T, topk, E) bytes.
 */
size_t w8a8_route_plan_workspace_size(int64_t T, int64_t topk, int64_t E);
int w8a8_route_plan(const int32_t* expert_idx, int64_t T, int64_t topk, int64_t E, int64_t* count,
                    int64_t* cumsum, int64_t* expanded_pos, void* workspace,
                    size_t workspace_bytes, void* stream);

/* dst[pos[i*topk+k]] = src[i] for row payloads of row_bytes (int8 tokens) and
 * dst_scale likewise for the fp32 per-token scales (may be NULL). */
int w8a8_scatter_rows(const void* src, const float* src_scale, void* dst, float* dst_scale,
                      const int64_t* expanded_pos, int64_t T, int64_t topk, int64_t row_bytes,
                      void* stream);

/* dst[d] = src[index[d]] for rows of row_bytes (and dst_scale[d] = src_scale[index[d]] when both scale
 * pointers are given); a negative index leaves the row untouched.  This is the data movement of
 * MoeReRouting (rank-major -> expert-major after an all-to-all) with the permutation supplied by the
 * caller (operators/moererouting/csrc/ops/moe_re_routing/op_kernel/moe_re_routing_kernel.cpp:15-24). */
int w8a8_permute_rows(const void* src, const float* src_scale, void* dst, float* dst_scale,
                      const int64_t* index, int64_t rows, int64_t row_bytes, void* stream);

/*
 * MoeReRouting with the (N ranks x E local experts) count matrix in device memory: no host readback, the cell
 * tables are built by one small kernel, then rows move as in w8a8_permute_rows.
 *   srcStart(i,j) = sum_{i'<i} rowSum(i') + sum_{j'<j} cnt[i][j'];  dstStart(i,j) = sum_{j'<j} colSum(j') +
 *   sum_{i'<i} cnt[i'][j];  out[dstStart+k] = in[srcStart+k], out_idx[dstStart+k] = srcStart+k,
 *   expert_token_num[j] = colSum(j) in the counts' own integer type.
 * Replaces launch_moe_rr_{h,bf,i8}_{i32,i64}
 * (operators/moererouting/csrc/ops/moe_re_routing/op_kernel/moe_re_routing_launch.h:44-74); the token type only
 * enters as row_bytes = H * element size, count_bytes is 4 (int32) or 8 (int64).  scales / out_scales are optional
 * (fp32 [A]).  Rows past the routed total are left untouched.  A negative count or a total above A copies nothing
 * and sets the workspace error word (w8a8_workspace_error() returns 1).
 */
size_t w8a8_moe_re_routing_workspace_size(int64_t A, int64_t N, int64_t E);
int w8a8_moe_re_routing(const void* tokens, const void* counts, const float* scales, void* out_tokens,
                        float* out_scales, int32_t* out_idx, void* expert_token_num, int64_t A,
                        int64_t row_bytes, int64_t N, int64_t E, int count_bytes, void* workspace,
                        size_t workspace_bytes, void* stream);

/*
 * Fused dispatch (no reference counterpart: the reference is single-device).  Instead of packing rows, running
 * an all-to-all and regrouping the result, every quantised token row is stored directly at the row it occupies in
 * the expert-major buffer of the rank that owns its expert -- a peer pointer when that rank is another GPU
 * (plain stores over NVLink).  Per expert e: row_dst[e] / scale_dst[e] are the addresses of the first row / scale
 * this rank may write for e in the owner's buffers, my_base[e] the position of this rank's first (token, k) pair
 * for e in its own expert-major order (the exclusive cumsum of w8a8_route_plan's count).  The caller synchronises
 * the ranks before the owners read.
 */
int w8a8_dispatch_rows(const void* src, const float* src_scale, const int32_t* expert_idx,
                       const int64_t* expanded_pos, const uint64_t* row_dst, const uint64_t* scale_dst,
                       const int64_t* my_base, int64_t T, int64_t topk, int64_t row_bytes, void* stream);

/*
 * Address tables of the fused expert-parallel transport, computed on the device from the all-gathered count
 * matrix counts[P, E] (rows rank i routes to global expert e; expert e lives on rank e / (E / P)), so that a step
 * needs no host readback.  peer_base[P] are the ranks' buffer addresses as this rank sees them; off_x / off_s /
 * off_back the byte offsets of the int8 rows, the fp32 scales and the 16-bit return rows inside each buffer.
 * Outputs: row_dst[E], scale_dst[E], my_base[E] for w8a8_dispatch_rows; group_list[E / P] (cumulative rows of this
 * rank's experts, a device list for the grouped matmuls with list_on_device = 2); seg_first[(E / P) * P + 1] and
 * seg_ptr[(E / P) * P] for w8a8_expand_row_pointers; status[0] is set to 1 when some rank would receive more than
 * cap_rows rows (sticky: this call never clears it, the caller does after reading it).  P <= 64, E <= 1024, P * E <= 2048 (W8A8_ERR_LIMIT beyond).  No reference counterpart.
 */
int w8a8_ep_tables(const int64_t* counts, int64_t P, int64_t E, int64_t rank, const uint64_t* peer_base,
                   uint64_t off_x, uint64_t off_s, uint64_t off_back, int64_t row_bytes, int64_t back_row_bytes,
                   int64_t cap_rows, uint64_t* row_dst, uint64_t* scale_dst, int64_t* my_base,
                   int64_t* group_list, int64_t* seg_first, uint64_t* seg_ptr, int32_t* status, void* stream);

/* out[r] = seg_ptr[s] + (r - seg_first[s]) * row_bytes for the segment s containing row r (seg_first has
 * nseg + 1 non-decreasing entries): turns a (source rank, expert) segment table into one destination address per
 * row for w8a8_grouped_matmul_to_rows. */
int w8a8_expand_row_pointers(const int64_t* seg_first, const uint64_t* seg_ptr, int64_t nseg, int64_t rows,
                             int64_t row_bytes, uint64_t* out, void* stream);

/*
 * GroupedMatmul whose epilogue is the combine transport: identical to w8a8_grouped_matmul except that output row
 * r is stored at out_row_ptrs[r] (N contiguous elements, 16-byte aligned), which may lie in another GPU's memory.
 * The down projection then needs neither an un-permute pass nor an all-to-all: each row lands where its home
 * rank's w8a8_combine will read it.
 */
int w8a8_grouped_matmul_to_rows(const void* x, const void* w, const void* bias, const uint64_t* out_row_ptrs,
                                const float* x_scale, const float* w_scale, int64_t M, int64_t N, int64_t K,
                                int64_t E, const int64_t* group_list, int list_on_device, int dtype,
                                int bias_dtype, int out_dtype, int w_layout, void* workspace,
                                size_t workspace_bytes, void* stream);

/* out[i, :] = sum_k probs[i, k] * rows[pos[i*topk+k], :], fp32, ascending k,
 * rounded to dtype (F16 / BF16).  A negative position contributes nothing. */
int w8a8_combine(const void* rows, const float* probs, const int64_t* expanded_pos, void* out,
                 int64_t T, int64_t topk, int64_t H, int dtype, void* stream);

/*
 * MoeFinalizeRouting: out[i, :] = skip1[i, :] + skip2[i, :] + sum_k scales[i, k] * (rows[p(i, k), :] +
 * bias[expert_for_source_row[i, k], :]) with p(i, k) = src_to_dst_row[k * num_rows + i] for drop_pad_mode 0 / 1 and
 * src_to_dst_row[i * K + k] for 2 / 3.  fp32 throughout, ascending k, each term formed as (row + bias) * scale and
 * then added (no fused multiply-add), round-to-nearest-even store.  p outside [0, num_dst) drops the term, an
 * expert id outside [0, E) drops only its bias.  skip1, skip2, bias (needs expert_for_source_row) and scales are
 * optional; without scales K is 1.  rows / skips / bias / out share `dtype` (F16, BF16 or F32), scales have
 * `scale_dtype`.  Replaces the nine launch_mfr_<rows type>_<scale type> launchers
 * (operators/moefinalizerouting/csrc/ops/moe_finalize_routing/op_kernel/moe_finalize_routing_launch.h; formula in
 * moe_finalize_routing_kernel.cpp:15-25).  K above 128 is accepted for F32 rows only (W8A8_ERR_LIMIT otherwise).
 */
int w8a8_moe_finalize_routing(const void* rows, const int32_t* src_to_dst_row, const void* skip1,
                              const void* skip2, const void* bias, const void* scales,
                              const int32_t* expert_for_source_row, void* out, int64_t num_rows, int64_t H,
                              int64_t K, int64_t E, int64_t num_dst, int drop_pad_mode, int dtype,
                              int scale_dtype, void* stream);

/*
 * MoeGatingTopKSoftmax: p = softmax(x, last dim) in fp32; y[r, j] = the j-th largest p of row r (rounded to x's
 * type), expert_idx[r, j] its column (equal values: lower column first), row_idx[r, j] = j * rows + r.  A row
 * with finished[r] != 0 reports `inner` as every expert index; y and row_idx are unaffected.  `finished` is
 * optional (one byte per row, torch bool).  x: F16 / BF16 / F32 [rows, inner], 0 < k <= inner <=
 * W8A8_GATING_MAX_EXPERTS (W8A8_ERR_LIMIT beyond; the row is held in one warp's registers).
 * Replaces launch_moe_gating_kernel_{float,half,bfloat16}
 * (operators/moegatingtopksoftmax/csrc/ops/moe_gating_top_k_softmax/op_kernel/moe_gating_launch.h; formula in
 * moe_gating_kernel.cpp:14-21).
 */
#define W8A8_GATING_MAX_EXPERTS 1024
int w8a8_moe_gating_top_k_softmax(const void* x, const uint8_t* finished, void* y, int32_t* expert_idx,
                                  int32_t* row_idx, int64_t rows, int64_t inner, int64_t k, int dtype,
                                  void* stream);

/*
 * DequantSwigluQuant: x [M, 2H] int32 (a matmul accumulator; needs weight_scale fp32 [2H] and activation_scale
 * fp32 [M]) or F16 / BF16 (both scales must be NULL); A = x[:, :H], B = x[:, H:] after dequantisation
 * d = (float(x) * weight_scale) * activation_scale[row].  activate_left == 0: out = silu(B) * A, otherwise
 * out = silu(A) * B, evaluated as (A * B) / (1 + exp(-gate)); the optional quant_scale fp32 [H] multiplies the
 * half that is not the gate input; s = max(max|out| / 127, 1e-12); y = narrow(clamp(out / s, -128, 127)) int8
 * [M, H], scale fp32 [M]; rows whose padded half is longer than 1984 elements use out * (1 / s), as the
 * reference's long-row layout does.  flags: W8A8_F_ROUND_DIRECT.
 * Replaces launch_dqsq_{int32,half,bfloat16}
 * (operators/dequantswigluquant/csrc/ops/dequant_swiglu_quant/op_kernel/dqsq_launch.h; formula in
 * dqsq_kernel.cpp:14-28).
 */
int w8a8_dequant_swiglu_quant(const void* x, const float* weight_scale, const float* activation_scale,
                              const float* quant_scale, int8_t* y, float* scale, int64_t M, int64_t H,
                              int x_dtype, int activate_left, int flags, void* stream);

/*
 * GroupedMatmulSwigluQuant for rows that start, and results that end, in pinned HOST memory (no reference
 * counterpart: its plugin takes device tensors only).  Host C++ that cuts the rows into chunks of chunk_rows and keeps
 * a copy-in stream, the caller's stream and a copy-out stream busy at once over double-buffered device staging, each
 * chunk being one w8a8_grouped_matmul_swiglu_quant call with the chunk's own group list; the call then costs about
 * as long as the slower copy direction instead of copy + compute + copy, and the results equal one call over all
 * rows bit for bit.  Weights and their scales stay on the device.  device_mem: w8a8_gmsq_host_pipe_device_bytes()
 * bytes of device memory the caller owns (staging + workspace).  create makes two streams and a few events;
 * run enqueues everything and returns (the results are complete when `stream` has caught up); one run at a time per
 * pipe.  flags: W8A8_F_ROUND_DIRECT.
 */
typedef struct W8A8HostPipe W8A8HostPipe;
size_t w8a8_gmsq_host_pipe_device_bytes(int64_t K, int64_t N, int64_t E, int64_t chunk_rows);
int w8a8_gmsq_host_pipe_create(W8A8HostPipe** pipe, const int8_t* w, const float* w_scale, int64_t K, int64_t N,
                               int64_t E, int w_layout, int64_t chunk_rows, void* device_mem, size_t device_bytes);
int w8a8_gmsq_host_pipe_run(W8A8HostPipe* pipe, const int8_t* x_host, const float* x_scale_host,
                            const int64_t* group_list_host, int64_t M, int8_t* y_host, float* y_scale_host, int flags,
                            void* stream);
int w8a8_gmsq_host_pipe_destroy(W8A8HostPipe* pipe);

/*
 * The whole expert-parallel MoE FFN step as one host call (no reference counterpart: the reference is
 * single-device and has no step function; this is the C++ host side of benchmark configuration 5).  One call
 * enqueues on `stream`, with no host readback: add_rms_norm_dynamic_quant -> w8a8_route_plan -> all-gather of the
 * per-expert counts -> w8a8_ep_tables -> w8a8_dispatch_rows (rows stored straight into the owning rank's
 * expert-major buffer) -> barrier -> grouped_matmul_swiglu_quant -> w8a8_grouped_matmul_to_rows (int8 down
 * projection whose epilogue stores each row where its home rank's combine reads it) -> barrier -> w8a8_combine.
 * Rank r owns tokens [r * tokens, (r + 1) * tokens) and experts [r * E / world, (r + 1) * E / world).
 *
 * Every rank owns one buffer laid out as int8 rows [cap_rows, hidden] at off_x, fp32 row scales [cap_rows] at off_s
 * and 16-bit return rows [home_rows, hidden] at off_back; peer_base (a device array of `world` addresses) says where
 * each rank's buffer is mapped in this rank's address space, local_base is this rank's own buffer.  Those mappings
 * (CUDA IPC, virtual memory management, torch symmetric memory ...) are the caller's business; this library only
 * stores through them.
 *
 * Collectives (the count all-gather and two one-word all-reduces used as stream-ordered barriers) run on an NCCL
 * communicator made by w8a8_ep_comm_create: rank 0 calls w8a8_ep_unique_id, hands the 128 bytes to every rank by
 * any means, every rank calls w8a8_ep_comm_create.  NCCL is looked up in the process at that moment (no link-time
 * dependency): W8A8_ERR_UNSUPPORTED when it is not there.  world == 1 needs no communicator (comm NULL).
 *
 * A step that routes more than cap_rows rows to some rank stores nothing out of bounds: that step's tables are
 * zeroed, its output is meaningless, and a sticky flag is raised that w8a8_moe_ffn_step_status reads and clears
 * (returns 1; it synchronises the stream).  Every rank must make the same sequence of step calls.
 * The step runs two of its pieces (the normalisation + quantisation of the tokens, the row-pointer expansion) on a
 * second stream that the library keeps per device, forked from and joined to `stream` by events: for the caller
 * the step is ordered on `stream` like any other call, a stream capture follows both streams, and one step at a
 * time may be in the making per device (two host threads must not call it for the same device at once).
 */
typedef struct W8A8MoeFfnStep {
    int32_t world, rank;
    int32_t num_experts; /* global; a multiple of world */
    int32_t topk;
    int32_t dtype;       /* W8A8_DT_F16 / W8A8_DT_BF16: x, residual, gamma, outputs */
    int32_t reserved;
    int64_t tokens;      /* rows of x on this rank */
    int64_t hidden, inter;
    int64_t cap_rows;    /* rows every rank's receive buffer holds */
    int64_t home_rows;   /* rows every rank's return buffer holds (>= tokens * topk) */
    const uint64_t* peer_base; /* device array [world] */
    void* local_base;
    uint64_t off_x, off_s, off_back;
    const int8_t* w_up;   /* [E / world, hidden, 2 * inter] */
    const float* s_up;    /* [E / world, 2 * inter] */
    const int8_t* w_down; /* [E / world, inter, hidden] */
    const float* s_down;  /* [E / world, hidden] */
    void* comm;           /* from w8a8_ep_comm_create; NULL when world == 1 */
    void* workspace;      /* device, w8a8_moe_ffn_step_workspace_size bytes, zeroed once before the first step */
    size_t workspace_bytes;
} W8A8MoeFfnStep;

int w8a8_ep_unique_id(void* id128);
int w8a8_ep_comm_create(const void* id128, int world, int rank, void** comm);
int w8a8_ep_comm_destroy(void* comm);
size_t w8a8_moe_ffn_step_workspace_size(const W8A8MoeFfnStep* step);
int w8a8_moe_ffn_step(const W8A8MoeFfnStep* step, const void* x, const void* residual, const void* gamma,
                      float epsilon, const int32_t* expert_idx, const float* probs, void* out, void* x_out,
                      void* stream);
int w8a8_moe_ffn_step_status(const W8A8MoeFfnStep* step, void* stream);

/*
 * Measurement and self-test entry points of the tensor-core layer.  (No
 * counterparts in the reference, whose matmuls are calls into the Ascend Matmul
 * library.)
 *
 * w8a8_mma_issue_probe: every SM (cta_group 1) or SM pair (cta_group 2) issues
 * `batches` x per_commit tcgen05.mma kind::i8 instructions (one tcgen05.commit
 * per batch, per_commit a multiple of 4 up to 256, at most `depth` <= 8 batches in flight) of shape umma_m x umma_n x 32
 * on operands resident in shared memory (fill 0 = zeros, 1 = pseudo-random
 * bytes), with no loads and no epilogue: timed with CUDA events it gives the
 * rate the tensor pipe sustains for that shape, the ceiling the matmul kernels
 * are compared with.  a_mn_major / b_mn_major select the operand majors the
 * instruction descriptor names.  cta_group 1: umma_m 64 or 128; cta_group 2:
 * umma_m 128 or 256 (both CTAs together); umma_n a multiple of 16 (8 for
 * umma_m 64) up to 256.  accumulators = 1: every instruction adds to the
 * result of the one before it, as in a matmul's K loop; 2 or 4: successive
 * instructions add to different accumulators (umma_n x accumulators <= 512).
 * pattern varies what the issuing thread does around a batch, to price each
 * piece: 0 = wait, instructions, commit; 1 = a second (already satisfied) wait;
 * 2 = an extra commit after every four instructions; 3 = a cluster-scope
 * wait plus tcgen05.fence; 4 = non-blocking mbarrier.test_wait polls before
 * the blocking wait.  error_word (device, may be NULL) receives 2 if a wait
 * ran out.  w8a8_mma_issue_probe_ops returns the integer operations one such
 * launch performs on the current device.
 *
 * w8a8_selftest_bounded_wait: one thread waits, with the matmul kernels' wait
 * helper and a limit of limit_cycles SM clocks, on a barrier nothing arrives
 * at; the kernel ends by itself and reports the way the matmul kernels do:
 * error_words[0] = 2 (a pipeline wait ran out), error_words[1] = 1 (the other
 * threads of the CTA saw the abort flag).  error_words: two zeroed int32 in
 * device memory.
 */
int w8a8_mma_issue_probe(int cta_group, int umma_m, int umma_n, int a_mn_major, int b_mn_major, int fill,
                         int accumulators, int per_commit, int depth, int pattern, int64_t batches,
                         int32_t* error_word, void* stream);
int64_t w8a8_mma_issue_probe_ops(int cta_group, int umma_m, int umma_n, int per_commit, int64_t batches);
int w8a8_selftest_bounded_wait(int64_t limit_cycles, int32_t* error_words, void* stream);

/* Self-test (no reference counterpart): evaluates the library's fp32 exp (the one the SwiGLU epilogues and the
 * router softmax use) and the operation sequence that defines it on all 2^32 fp32 bit patterns.  result: two
 * uint64 in device memory; [0] = number of patterns whose results differ in any bit (0 expected), [1] = the smallest
 * such pattern (all ones when there is none).  One launch of a few milliseconds. */
int w8a8_selftest_exp(uint64_t* result, void* stream);

/* Measurement aid (no reference counterpart): one launch that reads `bytes` (a multiple of 16, 16-byte aligned) of
 * device memory once with streaming loads and does nothing else - what pulling that many bytes out of HBM costs in
 * a single launch, the yardstick bench.py prints beside the weight-streaming quant_matmul shapes.  sink: 4 bytes of
 * device memory that are practically never written, or NULL. */
int w8a8_stream_read_probe(const void* src, int64_t bytes, void* sink, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* W8A8FFN_H */
