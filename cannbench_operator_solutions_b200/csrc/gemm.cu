// Host side of the tensor-core operators: argument validation (mirroring the
// reference plugins' checks), TMA tensor maps, the device-side group planner,
// kernel selection, and the C-ABI entry points for quant_matmul,
// grouped_matmul_swiglu_quant and grouped_matmul.
#include <cuda.h>

#include <atomic>
#include <mutex>

#include "gemm_kernel.cuh"

namespace w8a8 {

// ---------------------------------------------------------------------------
// cuTensorMapEncodeTiled through the runtime's driver entry point lookup (the
// library does not link libcuda directly).
// ---------------------------------------------------------------------------
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_fn()
{
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess) {
            fn = reinterpret_cast<EncodeTiledFn>(sym);
        }
    });
    return fn;
}

static CUtensorMapDataType tm_dtype(int kind)
{
    switch (kind) {
    case KIND_F16:
        return CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    case KIND_BF16:
        return CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    default:
        return CU_TENSOR_MAP_DATA_TYPE_UINT8;
    }
}

// A: [rows, K] row-major.  Box = 128 bytes of K x 128 rows.
static bool make_map_a(CUtensorMap* m, const void* base, int64_t rows, int64_t K, int kind, int box_rows = 128)
{
    EncodeTiledFn fn = encode_tiled_fn();
    if (fn == nullptr) {
        return false;
    }
    const int elem = (kind == KIND_I8) ? 1 : 2;
    cuuint64_t dims[2] = {static_cast<cuuint64_t>(K), static_cast<cuuint64_t>(rows)};
    cuuint64_t strides[1] = {static_cast<cuuint64_t>(K) * elem};
    cuuint32_t box[2] = {static_cast<cuuint32_t>(128 / elem), static_cast<cuuint32_t>(box_rows)};
    cuuint32_t estr[2] = {1, 1};
    return fn(m, tm_dtype(kind), 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
              CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// B: [G, K, N] (mn_major) or [G, N, K].  Box = 128 bytes of the contiguous
// dimension x 128 bytes-worth of K rows (mn_major: BLOCK_K rows) or 128 N rows.
static bool make_map_b(CUtensorMap* m, const void* base, int64_t G, int64_t N, int64_t K, int kind, bool mn_major)
{
    EncodeTiledFn fn = encode_tiled_fn();
    if (fn == nullptr) {
        return false;
    }
    const int elem = (kind == KIND_I8) ? 1 : 2;
    const int64_t inner = mn_major ? N : K;
    const int64_t outer = mn_major ? K : N;
    cuuint64_t dims[3] = {static_cast<cuuint64_t>(inner), static_cast<cuuint64_t>(outer), static_cast<cuuint64_t>(G)};
    cuuint64_t strides[2] = {static_cast<cuuint64_t>(inner) * elem, static_cast<cuuint64_t>(inner) * outer * elem};
    cuuint32_t box[3] = {static_cast<cuuint32_t>(128 / elem), static_cast<cuuint32_t>(mn_major ? 128 / elem : 128), 1};
    cuuint32_t estr[3] = {1, 1, 1};
    return fn(m, tm_dtype(kind), 3, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
              CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int CG, int BLOCK_N>
constexpr size_t gemm_smem_bytes()
{
    return static_cast<size_t>(gemm_stages(CG, BLOCK_N)) * (GEMM_A_BYTES + (BLOCK_N / CG) * GEMM_KBYTES) +
           1024 /*alignment slack*/ + 512 /*barriers, tmem slot, abort flag*/ + GEMM_EPI_PATCH_BYTES /*store patches*/;
}

// number of workers (CTAs, or CTA pairs) a persistent launch uses
template <int CG>
static int64_t worker_count(int64_t max_tiles)
{
    int64_t workers = sm_count() / CG;
    if (max_tiles < workers) {
        workers = max_tiles;
    }
    return workers < 1 ? 1 : workers;
}

template <int CG, int BLOCK_N, int KIND, int EPI, bool B_MN, int EPI_WARPS = 8>
static cudaError_t launch_gemm(const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, int64_t max_tiles,
                               cudaStream_t st)
{
    auto kern = gemm_tc_kernel<CG, BLOCK_N, KIND, EPI, B_MN, EPI_WARPS>;
    constexpr size_t smem = gemm_smem_bytes<CG, BLOCK_N>();
    // the attribute is per device; setting it on every call is cheap and covers multi-GPU processes
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) {
        return e;
    }
    const int64_t workers = worker_count<CG>(max_tiles);
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(static_cast<unsigned>(workers * CG), 1, 1);
    cfg.blockDim = dim3(gemm_threads(EPI_WARPS), 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    if (CG == 2) {
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
    }
    note_launch();
    return cudaLaunchKernelEx(&cfg, kern, ta, tb, p);
}

static std::atomic<int> g_gmsq_epilogue_warps{16};

template <int KIND, int EPI>
static cudaError_t dispatch_gemm(int cta_group, int block_n, bool b_mn, const CUtensorMap& ta, const CUtensorMap& tb,
                                 const GemmParams& p, int64_t max_tiles, cudaStream_t st)
{
    if constexpr (EPI == EPI_GMSQ) {
        // the SwiGLU epilogue with sixteen epilogue warps (see w8a8_set_gmsq_epilogue_warps)
        if (g_gmsq_epilogue_warps.load(std::memory_order_relaxed) == 16) {
            if (cta_group == 2) {
                return b_mn ? launch_gemm<2, 256, KIND, EPI, true, 16>(ta, tb, p, max_tiles, st)
                            : launch_gemm<2, 256, KIND, EPI, false, 16>(ta, tb, p, max_tiles, st);
            }
            return b_mn ? launch_gemm<1, 256, KIND, EPI, true, 16>(ta, tb, p, max_tiles, st)
                        : launch_gemm<1, 256, KIND, EPI, false, 16>(ta, tb, p, max_tiles, st);
        }
    }
    if (cta_group == 2) {
        return b_mn ? launch_gemm<2, 256, KIND, EPI, true>(ta, tb, p, max_tiles, st)
                    : launch_gemm<2, 256, KIND, EPI, false>(ta, tb, p, max_tiles, st);
    }
    if constexpr (EPI != EPI_GMSQ) {
        if (block_n == 128) {
            return b_mn ? launch_gemm<1, 128, KIND, EPI, true>(ta, tb, p, max_tiles, st)
                        : launch_gemm<1, 128, KIND, EPI, false>(ta, tb, p, max_tiles, st);
        }
    }
    return b_mn ? launch_gemm<1, 256, KIND, EPI, true>(ta, tb, p, max_tiles, st)
                : launch_gemm<1, 256, KIND, EPI, false>(ta, tb, p, max_tiles, st);
}

// Kernel shape: CTA pairs for dense problems with enough rows to fill 256-row tiles.  w8a8_set_gemm_shape()
// (1, 2, or 3 = pairs plus singles for grouped problems; 0 = the library's choice) overrides it process-wide; the
// tests use it to run every case on every shape.
constexpr int GEMM_SHAPE_HYBRID = 3;
static std::atomic<int> g_shape_override{0};
static std::atomic<int> g_fuse_requant{0};  // see w8a8_set_gmsq_fused_requant

static int choose_cta_group(int64_t rows, bool grouped)
{
    const int v = g_shape_override.load(std::memory_order_relaxed);
    if (v == 1 || v == 2 || (v == GEMM_SHAPE_HYBRID && grouped)) {
        return v;
    }
    // Grouped problems with enough rows run in two launches: CTA pairs on every group's 256-row blocks (the last
    // one partial when it holds more than 128 rows) and single CTAs on leftovers of at most 128 rows.  Pairs on everything would pad the end of every group to 256 rows,
    // which with skewed group sizes costs more than pairing gains (measured on the 256-expert Zipf configuration:
    // 4.94 ms against 4.66 ms with 128-row tiles only).
    if (grouped) {
        return rows >= 2048 ? GEMM_SHAPE_HYBRID : 1;
    }
    return rows >= 256 ? 2 : 1;
}

// ---------------------------------------------------------------------------
// Group planner: cumulative group list -> table of row tiles (128 rows for single CTAs, 256 for CTA pairs).
// The list arrives by value (host lists, validated by the caller) or from
// device memory (validated here; an invalid list yields zero tiles and
// error = 1).
// ---------------------------------------------------------------------------
constexpr int PLAN_MAX_BY_VALUE = 1024;
struct GroupEndsByValue {
    int32_t ends[PLAN_MAX_BY_VALUE];
};

// mode PLAN_ALL: every row of a group, in tiles of tile_m (the last one partial).
// mode PLAN_WHOLE: the whole tile_m-row tiles of a group, plus its last partial tile when that holds more than
//                  tile_m / 2 rows (as a pair tile it pads no more rows than two single tiles would).
// mode PLAN_LEFTOVER: what a group leaves over after its (2 * tile_m)-row blocks when that is at most tile_m rows:
//                  one tile of tile_m.
// PLAN_WHOLE at 256 rows and PLAN_LEFTOVER at 128 rows together cover every row exactly once.
constexpr int PLAN_ALL = 0;
constexpr int PLAN_WHOLE = 1;
constexpr int PLAN_LEFTOVER = 2;
constexpr int PLAN_BOTH = 3;  // host side only: PLAN_WHOLE at 256 rows and PLAN_LEFTOVER at 128 rows in one launch

__device__ __forceinline__ void plan_groups_body(const int64_t* __restrict__ dev_list,
                                                 const GroupEndsByValue& by_value, int use_by_value, int64_t E,
                                                 int64_t M, GroupedHeader* header, TileEntry* tiles,
                                                 int64_t max_tiles, int tile_m, int mode, int32_t* shared_error,
                                                 int allow_prefix)
{
    extern __shared__ int32_t s_first[];  // first tile index of each group, E + 1 entries
    __shared__ int32_t s_warp_sum[8];
    __shared__ int s_bad;
    __shared__ int32_t s_carry;
    auto end_of = [&](int64_t g) -> int64_t {
        return use_by_value ? static_cast<int64_t>(by_value.ends[g]) : dev_list[g];
    };
    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int wid = tid >> 5;
    if (tid == 0) {
        s_bad = 0;
        s_carry = 0;
    }
    __syncthreads();
    // groups in chunks of 256: validate, count tiles, block-wide exclusive scan
    for (int64_t base = 0; base < E; base += 256) {
        const int64_t g = base + tid;
        int32_t cnt = 0;
        if (g < E) {
            const int64_t prev = (g == 0) ? 0 : end_of(g - 1);
            const int64_t e = end_of(g);
            if (e < prev || e > M || (g == E - 1 && e != M && !allow_prefix)) {
                s_bad = 1;
            } else {
                const uint32_t rows = static_cast<uint32_t>(e - prev);
                const uint32_t tm = static_cast<uint32_t>(tile_m);
                if (mode == PLAN_WHOLE) {
                    cnt = static_cast<int32_t>(rows / tm) + ((rows % tm > tm / 2) ? 1 : 0);
                } else if (mode == PLAN_LEFTOVER) {
                    const uint32_t rest = rows % (2 * tm);
                    cnt = (rest >= 1 && rest <= tm) ? 1 : 0;
                } else {
                    cnt = static_cast<int32_t>((rows + tm - 1) / tm);
                }
            }
        }
        int32_t incl = cnt;
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) {
            const int32_t v = __shfl_up_sync(0xffffffffu, incl, off);
            if (lane >= off) {
                incl += v;
            }
        }
        if (lane == 31) {
            s_warp_sum[wid] = incl;
        }
        __syncthreads();
        int32_t warp_off = 0;
        for (int w = 0; w < wid; ++w) {
            warp_off += s_warp_sum[w];
        }
        const int32_t carry = s_carry;
        if (g < E) {
            s_first[g] = carry + warp_off + incl - cnt;
        }
        __syncthreads();
        if (tid == 255) {
            s_carry = carry + warp_off + incl;
        }
        __syncthreads();
    }
    const int32_t total = s_carry;
    const int bad = (s_bad != 0 || total > max_tiles) ? 1 : 0;
    if (tid == 0) {
        s_first[E] = total;
        header->num_m_tiles = bad ? 0 : total;
        header->error = bad;
        header->rows_total = bad ? 0 : static_cast<int32_t>(end_of(E - 1));
        if (bad && shared_error != nullptr) {
            *shared_error = 1;  // the error word the caller reads lives in the first header
        }
    }
    __syncthreads();
    if (bad) {
        return;
    }
    // one warp per group at a time fills that group's tile entries
    for (int64_t g = wid; g < E; g += 8) {
        int64_t start = (g == 0) ? 0 : end_of(g - 1);
        int64_t rows = end_of(g) - start;
        if (mode == PLAN_LEFTOVER) {
            const int64_t whole = rows / (2 * tile_m) * (2 * tile_m);
            start += whole;
            rows -= whole;
        }
        const int32_t first = s_first[g];
        const int32_t cnt = s_first[g + 1] - first;
        for (int32_t t = lane; t < cnt; t += 32) {
            TileEntry te;
            te.group = static_cast<int32_t>(g);
            te.m_start = static_cast<int32_t>(start + static_cast<int64_t>(t) * tile_m);
            const int64_t left = rows - static_cast<int64_t>(t) * tile_m;
            te.m_rows = static_cast<int32_t>(left < tile_m ? left : tile_m);
            te.pad = 0;
            tiles[first + t] = te;
        }
    }
}

__global__ void __launch_bounds__(256) plan_groups_kernel(const int64_t* __restrict__ dev_list,
                                                          const GroupEndsByValue by_value, int use_by_value,
                                                          int64_t E, int64_t M, GroupedHeader* header,
                                                          TileEntry* tiles, int64_t max_tiles, int tile_m, int mode,
                                                          int32_t* shared_error, int allow_prefix)
{
    plan_groups_body(dev_list, by_value, use_by_value, E, M, header, tiles, max_tiles, tile_m, mode, shared_error,
                     allow_prefix);
}

// Both tile tables of the two-launch form in one launch: CTA 0 plans the 256-row blocks, CTA 1 the leftovers of at
// most 128 rows (each validates the list itself; the leftover table cannot overflow, every group adds at most one
// tile to it), and the remaining CTAs zero `clear16` 16-byte words at `clear` (row maxima and tile counters of the
// SwiGLU form), which saves a second planner launch and a memset per call.
constexpr int PLAN_CLEAR_CTAS = 30;

__global__ void __launch_bounds__(256) plan_groups_both_kernel(const int64_t* __restrict__ dev_list,
                                                               const GroupEndsByValue by_value, int use_by_value,
                                                               int64_t E, int64_t M, GroupedHeader* header,
                                                               TileEntry* tiles, int64_t max_tiles,
                                                               GroupedHeader* tail_header, TileEntry* tail_tiles,
                                                               int64_t tail_max_tiles, int allow_prefix,
                                                               uint4* __restrict__ clear, int64_t clear16)
{
    if (blockIdx.x == 0) {
        plan_groups_body(dev_list, by_value, use_by_value, E, M, header, tiles, max_tiles, 256, PLAN_WHOLE, nullptr,
                         allow_prefix);
    } else if (blockIdx.x == 1) {
        plan_groups_body(dev_list, by_value, use_by_value, E, M, tail_header, tail_tiles, tail_max_tiles, 128,
                         PLAN_LEFTOVER, nullptr, allow_prefix);
    } else {
        const int64_t stride = static_cast<int64_t>(gridDim.x - 2) * blockDim.x;
        for (int64_t i = static_cast<int64_t>(blockIdx.x - 2) * blockDim.x + threadIdx.x; i < clear16; i += stride) {
            clear[i] = make_uint4(0u, 0u, 0u, 0u);
        }
    }
}

// ---------------------------------------------------------------------------
// Requantisation of the SwiGLU activations (second, bandwidth-bound half of
// grouped_matmul_swiglu_quant): amax clamp at FLT_MIN, y_scale = amax*(1/127),
// inv = 127/amax, clamp to [-128,127], two-step narrowing
// (gmsq_vec_kernel.cpp:233-257).  One warp per row.
// ---------------------------------------------------------------------------
template <bool DIRECT>
__global__ void __launch_bounds__(256) gmsq_requant_kernel(const float* __restrict__ act,
                                                           const uint32_t* __restrict__ amax_bits,
                                                           int8_t* __restrict__ y, float* __restrict__ y_scale,
                                                           int64_t M, int64_t H, const GroupedHeader* header)
{
    if (header->error != 0) {
        return;
    }
    const int lane = threadIdx.x & 31;
    const int64_t warp_global = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    const int64_t warps_total = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
    const int64_t n4 = H / 4;
    const int64_t rows = min(M, static_cast<int64_t>(header->rows_total));  // a device list may end before M
    for (int64_t row = warp_global; row < rows; row += warps_total) {
        float amax = __uint_as_float(amax_bits[row]);
        if (!(amax > 1.1754944e-38f)) {
            amax = 1.1754944e-38f;
        }
        if (lane == 0) {
            y_scale[row] = __fmul_rn(amax, INV127);
        }
        const float inv = __fdiv_rn(127.0f, amax);
        const float4* src = reinterpret_cast<const float4*>(act + row * H);
        uint32_t* dst = reinterpret_cast<uint32_t*>(y + row * H);
        for (int64_t c = lane; c < n4; c += 32) {
            const float4 a = __ldcs(src + c);
            float v[4] = {__fmul_rn(a.x, inv), __fmul_rn(a.y, inv), __fmul_rn(a.z, inv), __fmul_rn(a.w, inv)};
            bool any_nan = false;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                any_nan |= (v[j] != v[j]);
                v[j] = fminf(fmaxf(v[j], -128.0f), 127.0f);
            }
            uint32_t packed = narrow4_fast<DIRECT>(v[0], v[1], v[2], v[3]);
            if (any_nan) {
                // a NaN activation narrows to 0 (fmaxf/fminf above turned it into a bound)
                const float w[4] = {__fmul_rn(a.x, inv), __fmul_rn(a.y, inv), __fmul_rn(a.z, inv),
                                    __fmul_rn(a.w, inv)};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    if (w[j] != w[j]) {
                        packed &= ~(0xffu << (8 * j));
                    }
                }
            }
            __stcs(dst + c, packed);
        }
    }
}

static inline size_t align_up_sz(size_t v, size_t a) { return (v + a - 1) / a * a; }

// ---------------------------------------------------------------------------
// fp32 operands on the bf16 tensor path: v = hi + mid + lo with three bf16 pieces (8 + 8 + 8 significand bits,
// each remainder exact in fp32), and x.w is the sum of the six piece products whose orders add up to at most two
// (hi.hi, hi.mid, mid.hi, hi.lo, mid.mid, lo.hi; what is dropped is below 2^-24 of |x||w|).  The pieces are laid
// out along K, small terms first, so that ONE bf16 matmul over 6K accumulates all six in fp32:
//   x' [M, 6K]  = [ lo | mid | mid | hi | hi  | hi ]
//   w' [.., 6K] = [ hi | mid | hi  | lo | mid | hi ]   (K-blocks of the weight's K dimension, either layout)
// ---------------------------------------------------------------------------
constexpr int SPLIT_TERMS = 6;

__device__ __forceinline__ void split3(float v, __nv_bfloat16 (&piece)[3])
{
    piece[0] = __float2bfloat16_rn(v);
    const float r1 = __fsub_rn(v, __bfloat162float(piece[0]));
    piece[1] = __float2bfloat16_rn(r1);
    const float r2 = __fsub_rn(r1, __bfloat162float(piece[1]));
    piece[2] = __float2bfloat16_rn(r2);
}

// src [rows, K] fp32 -> dst [rows, 6K] bf16; which piece (0 hi, 1 mid, 2 lo) fills K-block b is pick[b]
__global__ void __launch_bounds__(256) split_rows_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst,
                                                         int64_t rows, int64_t K, int is_weight)
{
    const int pick_x[SPLIT_TERMS] = {2, 1, 1, 0, 0, 0};
    const int pick_w[SPLIT_TERMS] = {0, 1, 0, 2, 1, 0};
    const int64_t total = rows * K;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
         i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int64_t r = i / K, c = i - r * K;
        __nv_bfloat16 piece[3];
        split3(src[i], piece);
        __nv_bfloat16* out = dst + r * (SPLIT_TERMS * K) + c;
#pragma unroll
        for (int b = 0; b < SPLIT_TERMS; ++b) {
            out[b * K] = piece[is_weight ? pick_w[b] : pick_x[b]];
        }
    }
}

// weight [E, K, N] fp32 (N contiguous) -> [E, 6K, N] bf16: K-block b of expert e holds piece pick_w[b]
__global__ void __launch_bounds__(256) split_weight_kn_kernel(const float* __restrict__ src,
                                                              __nv_bfloat16* __restrict__ dst, int64_t E, int64_t K,
                                                              int64_t N)
{
    const int pick_w[SPLIT_TERMS] = {0, 1, 0, 2, 1, 0};
    const int64_t per_expert = K * N;
    const int64_t total = E * per_expert;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
         i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int64_t e = i / per_expert, rest = i - e * per_expert;  // rest = k * N + n
        __nv_bfloat16 piece[3];
        split3(src[i], piece);
        __nv_bfloat16* out = dst + e * (SPLIT_TERMS * per_expert) + rest;
#pragma unroll
        for (int b = 0; b < SPLIT_TERMS; ++b) {
            out[b * per_expert] = piece[pick_w[b]];
        }
    }
}

struct GroupedWorkspace {
    GroupedHeader* header;
    TileEntry* tiles;
    int64_t max_tiles;
    uint32_t* amax;
    float* act;
    // second tile table: what a group leaves over after its 256-row blocks when that is at most 128 rows (one tile
    // per group), used when the blocks run on CTA pairs and these leftovers on single CTAs
    GroupedHeader* tail_header;
    TileEntry* tail_tiles;
    int64_t tail_max_tiles;
    // finished-column-tile counters of the fused requantisation, one per (row tile, CTA of the tile): for the first
    // table, then for the tail table; they follow the row maxima so that one memset clears both
    int32_t* tile_done;
    int32_t* tail_tile_done;
    size_t clear_bytes;  // from `amax`: row maxima + counters
    size_t total;
};

static GroupedWorkspace carve_workspace(void* ws, int64_t M, int64_t E, int64_t act_cols)
{
    GroupedWorkspace g;
    uint8_t* p = static_cast<uint8_t*>(ws);
    size_t off = 0;
    g.header = reinterpret_cast<GroupedHeader*>(p + off);
    off += align_up_sz(sizeof(GroupedHeader), 256);
    g.max_tiles = M / GEMM_BLOCK_M + E + 1;
    g.tiles = reinterpret_cast<TileEntry*>(p + off);
    off += align_up_sz(static_cast<size_t>(g.max_tiles) * sizeof(TileEntry), 256);
    g.amax = reinterpret_cast<uint32_t*>(p + off);
    const size_t clear_from = off;
    off += (act_cols > 0) ? align_up_sz(static_cast<size_t>(M) * sizeof(uint32_t), 256) : 0;
    g.tile_done = reinterpret_cast<int32_t*>(p + off);
    off += (act_cols > 0) ? align_up_sz(static_cast<size_t>(g.max_tiles) * 2 * sizeof(int32_t), 256) : 0;
    g.tail_tile_done = reinterpret_cast<int32_t*>(p + off);
    off += (act_cols > 0) ? align_up_sz(static_cast<size_t>(E + 1) * 2 * sizeof(int32_t), 256) : 0;
    g.clear_bytes = off - clear_from;
    g.act = reinterpret_cast<float*>(p + off);
    off += (act_cols > 0) ? align_up_sz(static_cast<size_t>(M) * act_cols * sizeof(float), 256) : 0;
    g.tail_header = reinterpret_cast<GroupedHeader*>(p + off);
    off += align_up_sz(sizeof(GroupedHeader), 256);
    g.tail_max_tiles = E + 1;
    g.tail_tiles = reinterpret_cast<TileEntry*>(p + off);
    off += align_up_sz(static_cast<size_t>(g.tail_max_tiles) * sizeof(TileEntry), 256);
    g.total = off;
    return g;
}

// A host group list is checked before any CUDA call is made for the operator.
static int check_host_group_list(const int64_t* group_list, int list_on_device, int64_t E, int64_t M)
{
    if (list_on_device < 0 || list_on_device > 2) {
        return W8A8_ERR_INVALID;
    }
    if (list_on_device) {
        return W8A8_OK;
    }
    if (E > PLAN_MAX_BY_VALUE) {
        return W8A8_ERR_UNSUPPORTED;
    }
    int64_t prev = 0;
    for (int64_t i = 0; i < E; ++i) {
        const int64_t v = group_list[i];
        if (v < prev || v > M) {
            return W8A8_ERR_GROUP_LIST;
        }
        prev = v;
    }
    return (prev == M) ? W8A8_OK : W8A8_ERR_GROUP_LIST;
}

// returns W8A8_OK or an error; launches the planner on `st`
static int plan_groups(const int64_t* group_list, int list_on_device, int64_t E, int64_t M,
                       const GroupedWorkspace& g, int tile_m, cudaStream_t st, int mode = PLAN_ALL,
                       void* clear = nullptr, size_t clear_bytes = 0)
{
    GroupedHeader* header = (mode == PLAN_LEFTOVER) ? g.tail_header : g.header;
    TileEntry* tiles = (mode == PLAN_LEFTOVER) ? g.tail_tiles : g.tiles;
    const int64_t max_tiles = (mode == PLAN_LEFTOVER) ? g.tail_max_tiles : g.max_tiles;
    int32_t* shared_error = (mode == PLAN_LEFTOVER) ? &g.header->error : nullptr;
    GroupEndsByValue bv;
    int use_bv = 0;
    const int64_t* dev_list = group_list;
    if (!list_on_device) {
        if (E > PLAN_MAX_BY_VALUE) {
            return W8A8_ERR_UNSUPPORTED;
        }
        int64_t prev = 0;
        for (int64_t i = 0; i < E; ++i) {
            const int64_t v = group_list[i];
            if (v < prev || v > M) {
                return W8A8_ERR_GROUP_LIST;
            }
            bv.ends[i] = static_cast<int32_t>(v);
            prev = v;
        }
        if (prev != M) {
            return W8A8_ERR_GROUP_LIST;
        }
        for (int64_t i = E; i < PLAN_MAX_BY_VALUE; ++i) {
            bv.ends[i] = 0;
        }
        use_bv = 1;
        dev_list = nullptr;
    }
    const size_t smem = static_cast<size_t>(E + 1) * sizeof(int32_t);
    if (smem > 48 * 1024) {
        return W8A8_ERR_UNSUPPORTED;
    }
    if (mode == PLAN_BOTH) {
        const int64_t clear16 = static_cast<int64_t>(clear_bytes / 16);
        const unsigned grid = 2 + (clear16 > 0 ? PLAN_CLEAR_CTAS : 0);
        plan_groups_both_kernel<<<grid, 256, smem, st>>>(dev_list, bv, use_bv, E, M, g.header, g.tiles, g.max_tiles,
                                                         g.tail_header, g.tail_tiles, g.tail_max_tiles,
                                                         list_on_device == 2 ? 1 : 0, static_cast<uint4*>(clear),
                                                         clear16);
    } else {
        plan_groups_kernel<<<1, 256, smem, st>>>(dev_list, bv, use_bv, E, M, header, tiles, max_tiles, tile_m, mode,
                                                 shared_error, list_on_device == 2 ? 1 : 0);
    }
    w8a8::note_launch();
    return (cudaGetLastError() == cudaSuccess) ? W8A8_OK : W8A8_ERR_CUDA;
}

// Runs a grouped problem whose GemmParams are filled in except for the tile table: plans the groups and launches
// the kernel shape(s) choose_cta_group picked.
template <int KIND, int EPI>
static int run_grouped(const int64_t* group_list, int list_on_device, int64_t E, int64_t M, const GroupedWorkspace& g,
                       bool b_mn, const CUtensorMap& ta, const CUtensorMap& tb, GemmParams p, cudaStream_t st,
                       void* clear = nullptr, size_t clear_bytes = 0)
{
    const int shape = choose_cta_group(M, true);
    // (Rows stored one by one at caller-given addresses, possibly in peer memory, use the same shapes.  Single
    // tiles for them once measured faster on two GPUs; with the present kernels the chain steps are 13.26 against
    // 13.25 - 13.5 ms on two GPUs, 7.62 against 7.73 - 7.83 ms on four and 26.4 against 28.0 ms on one.)
    p.grouped = 1;
    p.error = &g.header->error;
    // `clear` (the SwiGLU form's row maxima and tile counters) must be zero before the first matmul launch: the
    // two-table planner does it in its own launch, the other shapes with a memset
    if (shape != GEMM_SHAPE_HYBRID) {
        if (clear_bytes != 0 && cudaMemsetAsync(clear, 0, clear_bytes, st) != cudaSuccess) {
            return W8A8_ERR_CUDA;
        }
        const int rc = plan_groups(group_list, list_on_device, E, M, g, 128 * shape, st);
        if (rc != W8A8_OK) {
            return rc;
        }
        p.tiles = g.tiles;
        p.header = g.header;
        p.tile_done = g.tile_done;
        const cudaError_t e = dispatch_gemm<KIND, EPI>(shape, 256, b_mn, ta, tb, p, g.max_tiles * p.n_tiles, st);
        return (e == cudaSuccess) ? W8A8_OK : W8A8_ERR_CUDA;
    }
    const int rc = plan_groups(group_list, list_on_device, E, M, g, 256, st, PLAN_BOTH, clear, clear_bytes);
    if (rc != W8A8_OK) {
        return rc;
    }
    p.tiles = g.tiles;
    p.header = g.header;
    p.tile_done = g.tile_done;
    cudaError_t e = dispatch_gemm<KIND, EPI>(2, 256, b_mn, ta, tb, p, (M / 256 + E + 1) * p.n_tiles, st);
    if (e != cudaSuccess) {
        return W8A8_ERR_CUDA;
    }
    p.tiles = g.tail_tiles;
    p.header = g.tail_header;
    p.tile_done = g.tail_tile_done;
    e = dispatch_gemm<KIND, EPI>(1, 256, b_mn, ta, tb, p, g.tail_max_tiles * p.n_tiles, st);
    return (e == cudaSuccess) ? W8A8_OK : W8A8_ERR_CUDA;
}

// ---------------------------------------------------------------------------
// Error word of launches that have no workspace to carry one (the dense matmuls): one int32 in the library's
// device image per GPU.  A kernel whose bounded wait ran out stores 2 there; w8a8_pipeline_error() reads and
// clears it.  The address is looked up once per device, with that device current.
// ---------------------------------------------------------------------------
static __device__ int32_t g_pipeline_error_word;

static int32_t* pipeline_error_word()
{
    constexpr int MAX_DEVICES = 64;
    static std::atomic<int32_t*> cache[MAX_DEVICES];
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) {
        return nullptr;
    }
    int32_t* p = cache[dev].load(std::memory_order_relaxed);
    if (p == nullptr) {
        void* sym = nullptr;
        if (cudaGetSymbolAddress(&sym, g_pipeline_error_word) != cudaSuccess) {
            return nullptr;
        }
        p = static_cast<int32_t*>(sym);
        cache[dev].store(p, std::memory_order_relaxed);
    }
    return p;
}

}  // namespace w8a8

using namespace w8a8;

// ===========================================================================
// quant_matmul
// ===========================================================================
static int quant_matmul_impl(const int8_t* x1, const int8_t* x2, const void* scale, const float* offset,
                             const float* pertoken, const void* bias, void* out, int64_t batch, int64_t M, int64_t N,
                             int64_t K, int64_t flags, int out_dtype, int x2_layout, int64_t bias_batch_stride,
                             bool raw_i32, void* stream)
{
    if (batch <= 0 || M <= 0 || N <= 0 || K <= 0) {
        return W8A8_ERR_INVALID;  // quant_matmul_plugin.cpp:100 "requires non-empty shapes"
    }
    if (x1 == nullptr || x2 == nullptr || out == nullptr) {
        return W8A8_ERR_INVALID;
    }
    if (x2_layout != W8A8_W_KN && x2_layout != W8A8_W_NK) {
        return W8A8_ERR_INVALID;
    }
    if (!raw_i32) {
        if (scale == nullptr || (out_dtype != W8A8_DT_F16 && out_dtype != W8A8_DT_BF16)) {
            return W8A8_ERR_INVALID;
        }
        const int64_t bias_kind = (flags & W8A8_QM_BIAS_MASK) >> W8A8_QM_BIAS_SHIFT;
        if (bias_kind > W8A8_QM_BIAS_F32 || (bias_kind != W8A8_QM_BIAS_NONE && bias == nullptr)) {
            return W8A8_ERR_INVALID;
        }
        if (((flags & W8A8_QM_HAS_OFFSET) && offset == nullptr) || ((flags & W8A8_QM_HAS_PT) && pertoken == nullptr)) {
            return W8A8_ERR_INVALID;
        }
    }
    if ((K % 16) != 0 || (N % 16) != 0) {
        return W8A8_ERR_UNSUPPORTED;
    }
    if (!is_aligned(x1, 16) || !is_aligned(x2, 16) || !is_aligned(out, 16)) {
        return W8A8_ERR_ALIGN;
    }
    if (batch * M >= (int64_t(1) << 31) || N >= (int64_t(1) << 31) || K >= (int64_t(1) << 31)) {
        return W8A8_ERR_UNSUPPORTED;
    }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const bool b_mn = (x2_layout == W8A8_W_KN);
    // With fewer than 128 rows in all, the A load only brings the rows that exist (rounded up to 8): the rest of the
    // 128-row shared-memory tile keeps whatever it held, which only reaches accumulator rows the epilogue never stores.
    const int a_box_rows = (batch * M < 128) ? static_cast<int>((batch * M + 7) / 8 * 8) : 128;
    CUtensorMap ta, tb;
    if (!make_map_a(&ta, x1, batch * M, K, KIND_I8, a_box_rows) || !make_map_b(&tb, x2, batch, N, K, KIND_I8, b_mn)) {
        return W8A8_ERR_CUDA;
    }
    GemmParams p{};
    p.a_box_bytes = a_box_rows * GEMM_KBYTES;
    p.M = M;
    p.N = N;
    p.K = K;
    p.num_k_blocks = static_cast<int32_t>((K + GEMM_KBYTES - 1) / GEMM_KBYTES);
    p.m_tiles_per_batch = static_cast<int32_t>((M + GEMM_BLOCK_M - 1) / GEMM_BLOCK_M);
    p.batch = static_cast<int32_t>(batch);
    p.grouped = 0;
    p.scale = scale;
    p.offset = offset;
    p.row_scale = pertoken;
    p.bias = bias;
    p.out = out;
    p.flags = flags;
    p.out_dtype = out_dtype;
    p.bias_batch_stride = bias_batch_stride;
    p.error = pipeline_error_word();  // null (no report) only if the symbol lookup failed
    const int cg = choose_cta_group(M, false);
    const int tile_m = 128 * cg;
    p.m_tiles_per_batch = static_cast<int32_t>((M + tile_m - 1) / tile_m);
    // narrow tiles when wide ones would leave most SMs idle (single-CTA tiles only)
    const int64_t m_tiles = batch * p.m_tiles_per_batch;
    const int64_t tiles256 = m_tiles * ((N + 255) / 256);
    const int block_n = (cg == 1 && tiles256 < sm_count()) ? 128 : 256;
    p.n_tiles = static_cast<int32_t>((N + block_n - 1) / block_n);
    const int64_t total = m_tiles * p.n_tiles;
    cudaError_t e;
    if (raw_i32) {
        e = dispatch_gemm<KIND_I8, EPI_RAW>(cg, block_n, b_mn, ta, tb, p, total, st);
    } else {
        e = dispatch_gemm<KIND_I8, EPI_QMM>(cg, block_n, b_mn, ta, tb, p, total, st);
    }
    return (e == cudaSuccess) ? W8A8_OK : W8A8_ERR_CUDA;
}

extern "C" int w8a8_quant_matmul(const int8_t* x1, const int8_t* x2, const void* scale, const float* offset,
                                 const float* pertoken, const void* bias, void* out, int64_t batch, int64_t M,
                                 int64_t N, int64_t K, int64_t flags, int out_dtype, int x2_layout,
                                 int64_t bias_batch_stride, void* stream)
{
    return quant_matmul_impl(x1, x2, scale, offset, pertoken, bias, out, batch, M, N, K, flags, out_dtype, x2_layout,
                             bias_batch_stride, false, stream);
}

extern "C" int w8a8_matmul_i8_i32(const int8_t* x1, const int8_t* x2, int32_t* c, int64_t batch, int64_t M, int64_t N,
                                  int64_t K, int x2_layout, void* stream)
{
    return quant_matmul_impl(x1, x2, nullptr, nullptr, nullptr, nullptr, c, batch, M, N, K, 0, 0, x2_layout, 0, true,
                             stream);
}

// ===========================================================================
// grouped_matmul_swiglu_quant
// ===========================================================================
extern "C" size_t w8a8_grouped_matmul_swiglu_quant_workspace_size(int64_t M, int64_t K, int64_t N, int64_t E)
{
    (void)K;
    if (M < 0 || N <= 0 || E <= 0) {
        return 0;
    }
    return carve_workspace(nullptr, M, E, N / 2).total;
}

extern "C" int w8a8_grouped_matmul_swiglu_quant(const int8_t* x, const int8_t* w, const float* w_scale,
                                                const float* x_scale, int8_t* y, float* y_scale, int64_t M, int64_t K,
                                                int64_t N, int64_t E, const int64_t* group_list, int list_on_device,
                                                int w_layout, int flags, void* workspace, size_t workspace_bytes,
                                                void* stream)
{
    if (M < 0 || K <= 0 || N <= 0 || E <= 0 || (N & 1) != 0) {
        return W8A8_ERR_INVALID;  // gmsq_plugin.cpp:52 "N must be even"
    }
    if ((flags & ~(W8A8_F_ROUND_DIRECT | W8A8_F_STAGE_MATMUL | W8A8_F_STAGE_REQUANT)) != 0 ||
        (w_layout != W8A8_W_KN && w_layout != W8A8_W_NK)) {
        return W8A8_ERR_INVALID;
    }
    const int stages = flags & (W8A8_F_STAGE_MATMUL | W8A8_F_STAGE_REQUANT);
    const bool run_matmul = (stages == 0) || (stages & W8A8_F_STAGE_MATMUL);
    const bool run_requant = (stages == 0) || (stages & W8A8_F_STAGE_REQUANT);
    if (M == 0) {
        return W8A8_OK;  // gmsq_plugin.cpp:93-95
    }
    if (x == nullptr || w == nullptr || w_scale == nullptr || x_scale == nullptr || y == nullptr ||
        y_scale == nullptr || group_list == nullptr) {
        return W8A8_ERR_INVALID;
    }
    if ((K % 16) != 0 || (N % 32) != 0) {
        return W8A8_ERR_UNSUPPORTED;
    }
    if (!is_aligned(x, 16) || !is_aligned(w, 16) || !is_aligned(w_scale, 16) || !is_aligned(y, 4)) {
        return W8A8_ERR_ALIGN;
    }
    if (M >= (int64_t(1) << 31) - 256 || N >= (int64_t(1) << 31) || K >= (int64_t(1) << 31)) {
        return W8A8_ERR_UNSUPPORTED;
    }
    const int64_t H = N / 2;
    const size_t need = w8a8_grouped_matmul_swiglu_quant_workspace_size(M, K, N, E);
    if (workspace == nullptr || workspace_bytes < need) {
        return W8A8_ERR_WORKSPACE;
    }
    if (!is_aligned(workspace, 256)) {
        return W8A8_ERR_ALIGN;
    }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const GroupedWorkspace g = carve_workspace(workspace, M, E, H);
    bool fused = false;
    if (run_matmul) {
        const int list_rc = check_host_group_list(group_list, list_on_device, E, M);
        if (list_rc != W8A8_OK) {
            return list_rc;
        }
        const bool b_mn = (w_layout == W8A8_W_KN);
        CUtensorMap ta, tb;
        if (!make_map_a(&ta, x, M, K, KIND_I8) || !make_map_b(&tb, w, E, N, K, KIND_I8, b_mn)) {
            return W8A8_ERR_CUDA;
        }
        GemmParams p{};
        p.a_box_bytes = GEMM_A_BYTES;
        p.M = M;
        p.N = N;
        p.K = K;
        p.num_k_blocks = static_cast<int32_t>((K + GEMM_KBYTES - 1) / GEMM_KBYTES);
        p.n_tiles = static_cast<int32_t>((H + 127) / 128);
        p.scale = w_scale;
        p.row_scale = x_scale;
        p.act = g.act;
        p.amax = g.amax;
        // Optional (off by default, it measures slower): the matmul kernels quantise each row block themselves as
        // soon as its last column tile is done, and no second kernel runs.
        // (a CTA waits for the other column tiles of its rows, which must then be running on other CTAs: only with
        // at least as many workers as column tiles)
        p.fuse_requant =
            (run_requant && g_fuse_requant.load(std::memory_order_relaxed) && p.n_tiles <= sm_count() / 2) ? 1 : 0;
        p.y = y;
        p.y_scale = y_scale;
        p.round_direct = (flags & W8A8_F_ROUND_DIRECT) ? 1 : 0;
        fused = p.fuse_requant != 0;
        // row maxima and finished-tile counters start at zero
        const int rc = run_grouped<KIND_I8, EPI_GMSQ>(group_list, list_on_device, E, M, g, b_mn, ta, tb, p, st, g.amax,
                                                      g.clear_bytes);
        if (rc != W8A8_OK) {
            return rc;
        }
    }
    if (!run_requant || fused) {
        return W8A8_OK;
    }
    const int64_t warps_needed = M;
    int64_t blocks = (warps_needed + 7) / 8;
    const int64_t cap = static_cast<int64_t>(sm_count()) * 8;
    if (blocks > cap) {
        blocks = cap;
    }
    if (flags & W8A8_F_ROUND_DIRECT) {
        gmsq_requant_kernel<true><<<static_cast<unsigned>(blocks), 256, 0, st>>>(g.act, g.amax, y, y_scale, M, H,
                                                                                g.header); w8a8::note_launch();
    } else {
        gmsq_requant_kernel<false><<<static_cast<unsigned>(blocks), 256, 0, st>>>(g.act, g.amax, y, y_scale, M, H,
                                                                                 g.header); w8a8::note_launch();
    }
    return (cudaGetLastError() == cudaSuccess) ? W8A8_OK : W8A8_ERR_CUDA;
}

// ===========================================================================
// grouped_matmul
// ===========================================================================
extern "C" size_t w8a8_grouped_matmul_workspace_size(int64_t M, int64_t N, int64_t K, int64_t E)
{
    (void)N;
    (void)K;
    if (M < 0 || E <= 0) {
        return 0;
    }
    return carve_workspace(nullptr, M, E, 0).total;
}

extern "C" size_t w8a8_grouped_matmul_f32_workspace_size(int64_t M, int64_t N, int64_t K, int64_t E)
{
    if (M < 0 || N <= 0 || K <= 0 || E <= 0) {
        return 0;
    }
    const size_t base = carve_workspace(nullptr, M, E, 0).total;
    const size_t xs = align_up_sz(static_cast<size_t>(M) * SPLIT_TERMS * K * 2, 256);
    const size_t ws = align_up_sz(static_cast<size_t>(E) * SPLIT_TERMS * K * N * 2, 256);
    return base + xs + ws;
}

static int grouped_matmul_impl(const void* x, const void* w, const void* bias, void* y, const uint64_t* out_row_ptrs,
                               const float* x_scale, const float* w_scale, int64_t M, int64_t N, int64_t K, int64_t E,
                               const int64_t* group_list, int list_on_device, int dtype, int bias_dtype,
                               int out_dtype, int w_layout, void* workspace, size_t workspace_bytes, void* stream)
{
    if (M < 0 || K <= 0 || N <= 0 || E <= 0) {
        return W8A8_ERR_INVALID;
    }
    if (w_layout != W8A8_W_KN && w_layout != W8A8_W_NK) {
        return W8A8_ERR_INVALID;
    }
    int kind;
    if (dtype == W8A8_DT_I8) {
        kind = KIND_I8;
        if (x_scale == nullptr || w_scale == nullptr) {
            return W8A8_ERR_INVALID;
        }
        if (out_dtype != W8A8_DT_F16 && out_dtype != W8A8_DT_BF16) {
            return W8A8_ERR_INVALID;
        }
    } else if (dtype == W8A8_DT_F16 || dtype == W8A8_DT_BF16) {
        kind = (dtype == W8A8_DT_F16) ? KIND_F16 : KIND_BF16;
        if (out_dtype != dtype) {
            return W8A8_ERR_INVALID;  // the reference's output takes x's dtype
        }
    } else if (dtype == W8A8_DT_F32) {
        kind = KIND_BF16;  // three-piece bf16 split of both operands, fp32 accumulation (see split3)
        if (out_dtype != W8A8_DT_F32 || out_row_ptrs != nullptr) {
            return W8A8_ERR_INVALID;
        }
    } else {
        return W8A8_ERR_INVALID;
    }
    if (bias != nullptr && bias_dtype != W8A8_DT_F16 && bias_dtype != W8A8_DT_BF16 && bias_dtype != W8A8_DT_F32) {
        return W8A8_ERR_INVALID;
    }
    if (M == 0) {
        return W8A8_OK;
    }
    if (x == nullptr || w == nullptr || (y == nullptr && out_row_ptrs == nullptr) || group_list == nullptr) {
        return W8A8_ERR_INVALID;
    }
    const int elem = (kind == KIND_I8) ? 1 : 2;
    const bool f32 = (dtype == W8A8_DT_F32);
    // the epilogue fetches per-channel operands and stores outputs in 16-column pieces
    if ((K * elem) % 16 != 0 || (N % 16) != 0) {
        return W8A8_ERR_UNSUPPORTED;
    }
    if (!is_aligned(x, 16) || !is_aligned(w, 16) || (y != nullptr && !is_aligned(y, 16))) {
        return W8A8_ERR_ALIGN;
    }
    if (M >= (int64_t(1) << 31) - 256 || N >= (int64_t(1) << 31) || K >= (int64_t(1) << 31)) {
        return W8A8_ERR_UNSUPPORTED;
    }
    const size_t need = f32 ? w8a8_grouped_matmul_f32_workspace_size(M, N, K, E)
                            : w8a8_grouped_matmul_workspace_size(M, N, K, E);
    if (workspace == nullptr || workspace_bytes < need) {
        return W8A8_ERR_WORKSPACE;
    }
    if (!is_aligned(workspace, 256)) {
        return W8A8_ERR_ALIGN;
    }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const GroupedWorkspace g = carve_workspace(workspace, M, E, 0);
    const int list_rc = check_host_group_list(group_list, list_on_device, E, M);
    if (list_rc != W8A8_OK) {
        return list_rc;
    }
    const bool b_mn = (w_layout == W8A8_W_KN);
    if (f32) {
        // split both operands into bf16 pieces laid out along K (6K in all), then run the bf16 path on them
        if (SPLIT_TERMS * K >= (int64_t(1) << 31)) {
            return W8A8_ERR_UNSUPPORTED;
        }
        uint8_t* base = static_cast<uint8_t*>(workspace) + g.total;
        __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(base);
        __nv_bfloat16* wsplit =
            reinterpret_cast<__nv_bfloat16*>(base + align_up_sz(static_cast<size_t>(M) * SPLIT_TERMS * K * 2, 256));
        const unsigned grid = static_cast<unsigned>(sm_count()) * 8;
        split_rows_kernel<<<grid, 256, 0, st>>>(static_cast<const float*>(x), xs, M, K, 0); w8a8::note_launch();
        if (b_mn) {
            split_weight_kn_kernel<<<grid, 256, 0, st>>>(static_cast<const float*>(w), wsplit, E, K, N); w8a8::note_launch();
        } else {
            split_rows_kernel<<<grid, 256, 0, st>>>(static_cast<const float*>(w), wsplit, E * N, K, 1); w8a8::note_launch();
        }
        if (cudaGetLastError() != cudaSuccess) {
            return W8A8_ERR_CUDA;
        }
        x = xs;
        w = wsplit;
        K = SPLIT_TERMS * K;
    }
    CUtensorMap ta, tb;
    if (!make_map_a(&ta, x, M, K, kind) || !make_map_b(&tb, w, E, N, K, kind, b_mn)) {
        return W8A8_ERR_CUDA;
    }
    GemmParams p{};
    p.a_box_bytes = GEMM_A_BYTES;
    p.M = M;
    p.N = N;
    p.K = K;
    const int block_k = GEMM_KBYTES / elem;
    p.num_k_blocks = static_cast<int32_t>((K + block_k - 1) / block_k);
    p.scale = w_scale;
    p.row_scale = x_scale;
    p.bias = bias;
    p.out = y;
    p.out_row_ptrs = out_row_ptrs;
    p.flags = (bias != nullptr ? 4 : 0) | (bias_dtype & 3);
    p.out_dtype = out_dtype;
    p.n_tiles = static_cast<int32_t>((N + 255) / 256);
    if (kind == KIND_I8) {
        return run_grouped<KIND_I8, EPI_GMM>(group_list, list_on_device, E, M, g, b_mn, ta, tb, p, st);
    }
    if (kind == KIND_F16) {
        return run_grouped<KIND_F16, EPI_GMM>(group_list, list_on_device, E, M, g, b_mn, ta, tb, p, st);
    }
    return run_grouped<KIND_BF16, EPI_GMM>(group_list, list_on_device, E, M, g, b_mn, ta, tb, p, st);
}

extern "C" int w8a8_grouped_matmul(const void* x, const void* w, const void* bias, void* y, const float* x_scale,
                                   const float* w_scale, int64_t M, int64_t N, int64_t K, int64_t E,
                                   const int64_t* group_list, int list_on_device, int dtype, int bias_dtype,
                                   int out_dtype, int w_layout, void* workspace, size_t workspace_bytes, void* stream)
{
    return grouped_matmul_impl(x, w, bias, y, nullptr, x_scale, w_scale, M, N, K, E, group_list, list_on_device, dtype,
                               bias_dtype, out_dtype, w_layout, workspace, workspace_bytes, stream);
}

extern "C" int w8a8_grouped_matmul_to_rows(const void* x, const void* w, const void* bias,
                                           const uint64_t* out_row_ptrs, const float* x_scale, const float* w_scale,
                                           int64_t M, int64_t N, int64_t K, int64_t E, const int64_t* group_list,
                                           int list_on_device, int dtype, int bias_dtype, int out_dtype, int w_layout,
                                           void* workspace, size_t workspace_bytes, void* stream)
{
    if (out_row_ptrs == nullptr) {
        return W8A8_ERR_INVALID;
    }
    return grouped_matmul_impl(x, w, bias, nullptr, out_row_ptrs, x_scale, w_scale, M, N, K, E, group_list,
                               list_on_device, dtype, bias_dtype, out_dtype, w_layout, workspace, workspace_bytes,
                               stream);
}

extern "C" int w8a8_pipeline_error(void* stream)
{
    int32_t* word = pipeline_error_word();
    if (word == nullptr) {
        return W8A8_ERR_CUDA;
    }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    int32_t v = 0;
    if (cudaMemcpyAsync(&v, word, sizeof(v), cudaMemcpyDeviceToHost, st) != cudaSuccess ||
        cudaMemsetAsync(word, 0, sizeof(v), st) != cudaSuccess || cudaStreamSynchronize(st) != cudaSuccess) {
        return W8A8_ERR_CUDA;
    }
    return v;
}

extern "C" int w8a8_set_gmsq_epilogue_warps(int warps)
{
    if (warps != 8 && warps != 16) {
        return W8A8_ERR_INVALID;
    }
    return g_gmsq_epilogue_warps.exchange(warps, std::memory_order_relaxed);
}

extern "C" int w8a8_set_gmsq_fused_requant(int on)
{
    return g_fuse_requant.exchange(on ? 1 : 0, std::memory_order_relaxed);
}

extern "C" int w8a8_set_gemm_shape(int shape)
{
    if (shape < 0 || shape > GEMM_SHAPE_HYBRID) {
        return W8A8_ERR_INVALID;
    }
    return g_shape_override.exchange(shape, std::memory_order_relaxed);
}

extern "C" int w8a8_workspace_error(const void* workspace, void* stream)
{
    if (workspace == nullptr) {
        return W8A8_ERR_INVALID;
    }
    GroupedHeader h;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (cudaMemcpyAsync(&h, workspace, sizeof(int32_t) * 2, cudaMemcpyDeviceToHost, st) != cudaSuccess) {
        return W8A8_ERR_CUDA;
    }
    if (cudaStreamSynchronize(st) != cudaSuccess) {
        return W8A8_ERR_CUDA;
    }
    return h.error;
}

// ===========================================================================
// grouped_matmul_swiglu_quant without a caller workspace
// ===========================================================================
// Scratch for w8a8_grouped_matmul_swiglu_quant_static: lives in the library's
// device image, so every GPU that loads the library sets these bytes aside
// until the process exits.  In host code this name is only a handle for
// cudaGetSymbolAddress; it is never a device address by itself.
static __device__ __align__(256) unsigned char g_gmsq_static_scratch[W8A8_STATIC_SCRATCH_BYTES];

// One address lookup per device, made with that device current.  Racing first calls store the same value.
static int static_scratch_address(void** out)
{
    constexpr int MAX_DEVICES = 64;
    static std::atomic<void*> scratch_of_device[MAX_DEVICES];
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0) {
        return W8A8_ERR_CUDA;
    }
    if (dev >= MAX_DEVICES) {
        return W8A8_ERR_LIMIT;  // the address cache is fixed-size; nothing in CUDA failed
    }
    void* scratch = scratch_of_device[dev].load(std::memory_order_relaxed);
    if (scratch == nullptr) {
        if (cudaGetSymbolAddress(&scratch, g_gmsq_static_scratch) != cudaSuccess || scratch == nullptr) {
            return W8A8_ERR_CUDA;
        }
        scratch_of_device[dev].store(scratch, std::memory_order_relaxed);
    }
    *out = scratch;
    return W8A8_OK;
}

// The error word of the last *_static call on the current device (it lives in the built-in scratch, which the
// caller never sees): 0 = none, 1 = invalid device group list (y was left untouched), 2 = a pipeline wait ran out.
extern "C" int w8a8_static_scratch_error(void* stream)
{
    void* scratch = nullptr;
    const int rc = static_scratch_address(&scratch);
    if (rc != W8A8_OK) {
        return rc;
    }
    return w8a8_workspace_error(scratch, stream);
}

extern "C" int w8a8_grouped_matmul_swiglu_quant_static(const int8_t* x, const int8_t* w, const float* w_scale,
                                                       const float* x_scale, int8_t* y, float* y_scale, int64_t M,
                                                       int64_t K, int64_t N, int64_t E, const int64_t* group_list,
                                                       int list_on_device, int w_layout, int flags, void* stream)
{
    if (M < 0 || K <= 0 || N <= 0 || E <= 0) {
        return W8A8_ERR_INVALID;
    }
    // the built-in scratch is fixed: refuse anything whose workspace would not fit
    const size_t need = w8a8_grouped_matmul_swiglu_quant_workspace_size(M, K, N, E);
    if (need == 0 || need > static_cast<size_t>(W8A8_STATIC_SCRATCH_BYTES)) {
        return W8A8_ERR_LIMIT;
    }
    void* scratch = nullptr;
    const int rc = static_scratch_address(&scratch);
    if (rc != W8A8_OK) {
        return rc;
    }
    // From here on this is the ordinary operator with the built-in bytes as its workspace.  That path rewrites
    // the header and tile table and zeroes the row maxima on the stream before it uses them, so whatever the
    // previous call left behind is never read.
    return w8a8_grouped_matmul_swiglu_quant(x, w, w_scale, x_scale, y, y_scale, M, K, N, E, group_list, list_on_device,
                                            w_layout, flags, scratch, static_cast<size_t>(W8A8_STATIC_SCRATCH_BYTES),
                                            stream);
}
