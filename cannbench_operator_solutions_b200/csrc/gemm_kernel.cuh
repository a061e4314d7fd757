// Persistent, warp-specialised tcgen05 GEMM for sm_100a with fused epilogues.
//
// One CTA per SM, 192 threads:
//   warp 0      TMA producer: fills a 4-deep ring of {A 128x128B, B BLOCK_N x128B}
//               shared-memory stages (128-byte swizzle), one mbarrier per stage.
//   warp 1      MMA issuer: one thread issues tcgen05.mma (UMMA 128 x BLOCK_N x 32B)
//               into one of two TMEM accumulator stages; tcgen05.commit releases
//               the shared-memory stage and finally publishes the accumulator.
//   warps 2-5   epilogue: tcgen05.ld the accumulator (each warp owns the 32 TMEM
//               lanes its index selects), apply the operator's dequant chain,
//               store.  Double-buffered TMEM lets the epilogue of tile i overlap
//               the main loop of tile i+1.
//
// A is always K-major ([rows, K], K contiguous).  B is either K-major
// ([.., N, K]) or MN-major ([.., K, N], the reference catalog's weight layout);
// both are consumed directly by the tensor core through the descriptor's
// major bit, no transposition pass.
//
// Tiles: 128 rows x BLOCK_N columns.  Dense problems enumerate (row tile, column
// tile) with the row index fastest so that concurrently running CTAs share a B
// column block in L2.  Grouped problems read a tile table built on the device
// from the cumulative group list (tiles never straddle groups; rows past a
// group's end inside a tile are computed and discarded) with the column index
// fastest, so the A tile and the expert's weights stay L2-resident.
#pragma once

#include "common.cuh"
#include "tc_ptx.cuh"

namespace w8a8 {

constexpr int GEMM_THREADS = 192;
constexpr int GEMM_BLOCK_M = 128;
constexpr int GEMM_STAGES = 4;
constexpr int GEMM_KBYTES = 128;  // bytes of K per stage row (one swizzle atom)
constexpr int GEMM_A_BYTES = GEMM_BLOCK_M * GEMM_KBYTES;

enum GemmKind { KIND_I8 = 0, KIND_F16 = 1, KIND_BF16 = 2 };
enum GemmEpi { EPI_RAW = 0, EPI_QMM = 1, EPI_GMSQ = 2, EPI_GMM = 3 };

struct TileEntry {
    int32_t group;
    int32_t m_start;
    int32_t m_rows;
    int32_t pad;
};

struct GroupedHeader {
    int32_t num_m_tiles;
    int32_t error;  // 0 ok, 1 invalid group list, 2 pipeline wait ran out
    int32_t pad[62];
};

struct GemmParams {
    int64_t M;  // rows per batch (dense) or total rows (grouped)
    int64_t N;  // logical output columns of the matmul
    int64_t K;
    int32_t num_k_blocks;
    int32_t n_tiles;
    int32_t m_tiles_per_batch;
    int32_t batch;
    int32_t grouped;
    const TileEntry* tiles;
    GroupedHeader* header;  // grouped: tile count + error word; dense: may be null
    int32_t* error;         // device error word (may be null)
    // epilogue operands
    const void* scale;       // QMM: scale; GMSQ/GMM: w_scale [E, N]
    const float* offset;     // QMM
    const float* row_scale;  // QMM: pertoken; GMSQ/GMM: x_scale
    const void* bias;
    void* out;
    int64_t flags;  // QMM flag word; GMM: bias dtype in bits 0-1, bit 2 = has bias
    int32_t out_dtype;
    int64_t bias_batch_stride;
    float* act;       // GMSQ: fp32 activations [M, N/2]
    uint32_t* amax;   // GMSQ: per-row max|act| bit patterns
};

// fp32 exp shared with the CPU oracle: Cody-Waite reduction by ln2 in two
// pieces, degree-5 polynomial (the classic single-precision coefficients
// published with the Cephes library), two-step power-of-two scaling.  Built
// from IEEE mul / add / fma only, so host and device agree bit for bit.
__device__ __forceinline__ float canonical_expf(float x)
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

// silu(l) = l / (1 + exp(-l)), the operation sequence of the reference
// (gmsq_vec_kernel.cpp:213-217).
__device__ __forceinline__ float canonical_silu(float l)
{
    const float e = __fadd_rn(canonical_expf(-l), 1.0f);
    return __fdiv_rn(l, e);
}

__device__ __forceinline__ float vec_elem_as_float(const void* p, int64_t i, int kind)
{
    switch (kind) {
    case W8A8_QM_BIAS_I32:
        return static_cast<float>(static_cast<const int32_t*>(p)[i]);
    case W8A8_QM_BIAS_F16:
        return __half2float(static_cast<const __half*>(p)[i]);
    case W8A8_QM_BIAS_BF16:
        return __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i]);
    default:
        return static_cast<const float*>(p)[i];
    }
}

template <int BLOCK_N, int KIND, int EPI, bool B_MN>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
    gemm_tc_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                   const GemmParams p)
{
    constexpr int ELEM = (KIND == KIND_I8) ? 1 : 2;
    constexpr int BLOCK_K = GEMM_KBYTES / ELEM;   // elements of K per stage
    constexpr int UMMA_K = 32 / ELEM;             // elements of K per instruction
    constexpr int NBOX = BLOCK_N * ELEM / 128;    // MN-major: 128-byte-wide column blocks per tile
    constexpr int B_BYTES = BLOCK_N * GEMM_KBYTES;
    constexpr int STAGE_BYTES = GEMM_A_BYTES + B_BYTES;
    constexpr uint32_t TMEM_COLS = 2 * BLOCK_N;  // 256 or 512: power of two
    constexpr uint32_t IDESC =
        (KIND == KIND_I8) ? tc::instr_desc(2u, 1u, B_MN ? 1u : 0u, GEMM_BLOCK_M, BLOCK_N)
                          : tc::instr_desc(1u, (KIND == KIND_BF16) ? 1u : 0u, B_MN ? 1u : 0u, GEMM_BLOCK_M, BLOCK_N);
    static_assert(BLOCK_N == 128 || BLOCK_N == 256, "BLOCK_N");
    static_assert(EPI != EPI_GMSQ || BLOCK_N == 256, "the SwiGLU epilogue pairs 128 gate with 128 up columns");

    extern __shared__ uint8_t smem_raw[];
    // 1024-byte alignment: required by the 128-byte swizzle atoms
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + GEMM_STAGES * STAGE_BYTES);
    // bars[0..S) full, [S..2S) empty, [2S..2S+2) tmem_full, [2S+2..2S+4) tmem_empty
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * GEMM_STAGES + 4);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t smem_base = tc::smem_u32(smem);
    const uint32_t bar_base = tc::smem_u32(bars);
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (GEMM_STAGES + s); };
    auto tfull_bar = [&](int s) { return bar_base + 8u * (2 * GEMM_STAGES + s); };
    auto tempty_bar = [&](int s) { return bar_base + 8u * (2 * GEMM_STAGES + 2 + s); };

    if (threadIdx.x == 0) {
        for (int s = 0; s < GEMM_STAGES; ++s) {
            tc::mbar_init(full_bar(s), 1);
            tc::mbar_init(empty_bar(s), 1);
        }
        for (int s = 0; s < 2; ++s) {
            tc::mbar_init(tfull_bar(s), 1);
            tc::mbar_init(tempty_bar(s), 128);
        }
        *abort_flag = 0;
        tc::fence_mbar_init();
        tc::prefetch_tensormap(&tm_a);
        tc::prefetch_tensormap(&tm_b);
    }
    if (warp == 1) {
        tc::tmem_alloc(tc::smem_u32(tmem_slot), TMEM_COLS);
        tc::tmem_relinquish();
    }
    tc::tc_fence_before_sync();
    __syncthreads();
    tc::tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    // ---- tile enumeration (identical in every role) ----
    int64_t total_tiles;
    int32_t dense_m_tiles = 0;
    if (p.grouped) {
        const int32_t nmt = p.header->num_m_tiles;
        total_tiles = static_cast<int64_t>(nmt) * p.n_tiles;
    } else {
        dense_m_tiles = p.batch * p.m_tiles_per_batch;
        total_tiles = static_cast<int64_t>(dense_m_tiles) * p.n_tiles;
    }
    const int64_t H = p.N / 2;  // GMSQ half width

    struct Tile {
        int32_t a_row0;   // first row of the A tile (global row index)
        int32_t m_rows;   // valid rows
        int32_t group;    // expert / batch (B's outermost coordinate)
        int32_t nt;       // column tile
    };
    auto decode = [&](int64_t t) {
        Tile tl;
        if (p.grouped) {
            const int32_t mt = static_cast<int32_t>(t / p.n_tiles);
            tl.nt = static_cast<int32_t>(t % p.n_tiles);
            const TileEntry e = p.tiles[mt];
            tl.a_row0 = e.m_start;
            tl.m_rows = e.m_rows;
            tl.group = e.group;
        } else {
            const int32_t mg = static_cast<int32_t>(t % dense_m_tiles);
            tl.nt = static_cast<int32_t>(t / dense_m_tiles);
            const int32_t b = mg / p.m_tiles_per_batch;
            const int32_t mt = mg % p.m_tiles_per_batch;
            const int64_t m0 = static_cast<int64_t>(mt) * GEMM_BLOCK_M;
            tl.a_row0 = static_cast<int32_t>(b * p.M + m0);
            const int64_t left = p.M - m0;
            tl.m_rows = static_cast<int32_t>(left < GEMM_BLOCK_M ? left : GEMM_BLOCK_M);
            tl.group = b;
        }
        return tl;
    };
    // first column of 128-element column block `i` of column tile nt
    auto box_col = [&](int32_t nt, int i) -> int32_t {
        if constexpr (EPI == EPI_GMSQ) {
            // 128-byte blocks [0, NBOX/2) are gate columns, the rest the matching up columns
            constexpr int HB = NBOX / 2;
            const int32_t within = (i % HB) * (128 / ELEM);
            return static_cast<int32_t>((i < HB ? 0 : H) + static_cast<int64_t>(nt) * (BLOCK_N / 2) + within);
        } else {
            return nt * BLOCK_N + i * (128 / ELEM);
        }
    };

    if (warp == 0) {
        // ===================== TMA producer =====================
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int64_t t = blockIdx.x; ok && t < total_tiles; t += gridDim.x) {
                const Tile tl = decode(t);
                for (int kb = 0; kb < p.num_k_blocks; ++kb) {
                    if (!tc::mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag)) {
                        ok = false;
                        break;
                    }
                    const uint32_t a_dst = smem_base + stage * STAGE_BYTES;
                    const uint32_t b_dst = a_dst + GEMM_A_BYTES;
                    tc::mbar_arrive_expect_tx(full_bar(stage), STAGE_BYTES);
                    tc::tma_load_2d(a_dst, &tm_a, full_bar(stage), kb * BLOCK_K, tl.a_row0);
                    if constexpr (B_MN) {
                        // boxes of {128 bytes of N, BLOCK_K rows of K}
                        constexpr int BOX_BYTES = BLOCK_K * 128;
#pragma unroll
                        for (int i = 0; i < NBOX; ++i) {
                            tc::tma_load_3d(b_dst + i * BOX_BYTES, &tm_b, full_bar(stage), box_col(tl.nt, i),
                                            kb * BLOCK_K, tl.group);
                        }
                    } else {
                        // boxes of {128 bytes of K, 128 rows of N}
                        constexpr int ROWS_PER_BOX = 128;
                        constexpr int BOXES = BLOCK_N / ROWS_PER_BOX;
#pragma unroll
                        for (int i = 0; i < BOXES; ++i) {
                            int32_t n_row;
                            if constexpr (EPI == EPI_GMSQ) {
                                n_row = static_cast<int32_t>((i == 0 ? 0 : H) + static_cast<int64_t>(tl.nt) * 128);
                            } else {
                                n_row = tl.nt * BLOCK_N + i * ROWS_PER_BOX;
                            }
                            tc::tma_load_3d(b_dst + i * ROWS_PER_BOX * GEMM_KBYTES, &tm_b, full_bar(stage),
                                            kb * BLOCK_K, n_row, tl.group);
                        }
                    }
                    if (++stage == GEMM_STAGES) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ===================== MMA issuer =====================
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            int64_t it = 0;
            bool ok = true;
            for (int64_t t = blockIdx.x; ok && t < total_tiles; t += gridDim.x, ++it) {
                const int acc = static_cast<int>(it & 1);
                const uint32_t acc_phase = static_cast<uint32_t>((it >> 1) & 1);
                if (!tc::mbar_wait(tempty_bar(acc), acc_phase ^ 1u, abort_flag)) {
                    ok = false;
                    break;
                }
                tc::tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * BLOCK_N);
                for (int kb = 0; kb < p.num_k_blocks; ++kb) {
                    if (!tc::mbar_wait(full_bar(stage), phase, abort_flag)) {
                        ok = false;
                        break;
                    }
                    tc::tc_fence_after_sync();
                    const uint32_t a_src = smem_base + stage * STAGE_BYTES;
                    const uint32_t b_src = a_src + GEMM_A_BYTES;
#pragma unroll
                    for (int k = 0; k < BLOCK_K / UMMA_K; ++k) {
                        const uint64_t a_desc = tc::smem_desc_sw128(a_src + k * 32, 16, 1024);
                        uint64_t b_desc;
                        if constexpr (B_MN) {
                            // K advances by UMMA_K rows of 128 bytes; column blocks are BLOCK_K rows apart
                            b_desc = tc::smem_desc_sw128(b_src + k * UMMA_K * 128, BLOCK_K * 128, 1024);
                        } else {
                            b_desc = tc::smem_desc_sw128(b_src + k * 32, 16, 1024);
                        }
                        const uint32_t accumulate = (kb > 0 || k > 0) ? 1u : 0u;
                        if constexpr (KIND == KIND_I8) {
                            tc::mma_i8(d_tmem, a_desc, b_desc, IDESC, accumulate);
                        } else {
                            tc::mma_f16(d_tmem, a_desc, b_desc, IDESC, accumulate);
                        }
                    }
                    tc::tc_commit(empty_bar(stage));
                    if (++stage == GEMM_STAGES) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
                if (ok) {
                    tc::tc_commit(tfull_bar(acc));
                }
            }
        }
        __syncwarp();
    } else {
        // ===================== epilogue (warps 2..5) =====================
        const int quarter = warp & 3;  // TMEM lanes [32*quarter, 32*quarter+32)
        const int row_in_tile = quarter * 32 + lane;
        int64_t it = 0;
        bool ok = true;
        for (int64_t t = blockIdx.x; ok && t < total_tiles; t += gridDim.x, ++it) {
            const Tile tl = decode(t);
            const int acc = static_cast<int>(it & 1);
            const uint32_t acc_phase = static_cast<uint32_t>((it >> 1) & 1);
            if (!tc::mbar_wait(tfull_bar(acc), acc_phase, abort_flag)) {
                ok = false;
                break;
            }
            tc::tc_fence_after_sync();
            const uint32_t t_addr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) +
                                    static_cast<uint32_t>(acc * BLOCK_N);
            const bool row_ok = row_in_tile < tl.m_rows;
            const int64_t row = static_cast<int64_t>(tl.a_row0) + row_in_tile;  // global row (A and output)

            if constexpr (EPI == EPI_GMSQ) {
                const float xs = row_ok ? p.row_scale[row] : 0.0f;
                const float* wsg = static_cast<const float*>(p.scale) + static_cast<int64_t>(tl.group) * p.N;
                float local_max = 0.0f;
#pragma unroll 1
                for (int c = 0; c < 128; c += 32) {
                    uint32_t g[32], u[32];
                    tc::tmem_ld_32x32(t_addr + c, g);
                    tc::tmem_ld_32x32(t_addr + 128 + c, u);
                    tc::tmem_ld_wait();
                    const int64_t col0 = static_cast<int64_t>(tl.nt) * 128 + c;  // column in [0, H)
                    if (row_ok) {
#pragma unroll
                        for (int q = 0; q < 8; ++q) {
                            const int64_t col = col0 + q * 4;
                            if (col < H) {
                                const float4 wg = __ldg(reinterpret_cast<const float4*>(wsg + col));
                                const float4 wu = __ldg(reinterpret_cast<const float4*>(wsg + H + col));
                                const float wga[4] = {wg.x, wg.y, wg.z, wg.w};
                                const float wua[4] = {wu.x, wu.y, wu.z, wu.w};
                                float a[4];
#pragma unroll
                                for (int j = 0; j < 4; ++j) {
                                    const float l = __fmul_rn(
                                        __fmul_rn(static_cast<float>(static_cast<int32_t>(g[q * 4 + j])), xs), wga[j]);
                                    const float r = __fmul_rn(
                                        __fmul_rn(static_cast<float>(static_cast<int32_t>(u[q * 4 + j])), xs), wua[j]);
                                    a[j] = __fmul_rn(canonical_silu(l), r);
                                    local_max = fmaxf(local_max, fabsf(a[j]));
                                }
                                *reinterpret_cast<float4*>(p.act + row * H + col) = make_float4(a[0], a[1], a[2], a[3]);
                            }
                        }
                    }
                }
                if (row_ok) {
                    atomicMax(reinterpret_cast<int*>(p.amax + row), __float_as_int(local_max));
                }
            } else {
                float row_mul = 1.0f;
                if constexpr (EPI == EPI_QMM) {
                    if ((p.flags & W8A8_QM_HAS_PT) && row_ok) {
                        // the plugin's layouts make (row mod M) the token index in every case
                        row_mul = p.row_scale[row % p.M];
                    }
                } else if constexpr (EPI == EPI_GMM && KIND == KIND_I8) {
                    row_mul = row_ok ? p.row_scale[row] : 0.0f;
                }
#pragma unroll 1
                for (int c = 0; c < BLOCK_N; c += 32) {
                    uint32_t r[32];
                    tc::tmem_ld_32x32(t_addr + c, r);
                    tc::tmem_ld_wait();
                    const int64_t col0 = static_cast<int64_t>(tl.nt) * BLOCK_N + c;
                    if (!row_ok || col0 >= p.N) {
                        continue;
                    }
                    if constexpr (EPI == EPI_RAW) {
                        int32_t* dst = static_cast<int32_t*>(p.out) + row * p.N + col0;
#pragma unroll
                        for (int q = 0; q < 8; ++q) {
                            if (col0 + q * 4 < p.N) {
                                *reinterpret_cast<uint4*>(dst + q * 4) =
                                    make_uint4(r[q * 4], r[q * 4 + 1], r[q * 4 + 2], r[q * 4 + 3]);
                            }
                        }
                    } else {
                        float v[32];
                        if constexpr (EPI == EPI_QMM) {
                            const int64_t f = p.flags;
                            const int bias_kind = static_cast<int>((f & W8A8_QM_BIAS_MASK) >> W8A8_QM_BIAS_SHIFT);
                            const void* bias = p.bias;
                            if (bias != nullptr && p.bias_batch_stride != 0) {
                                const int64_t esz = (bias_kind == W8A8_QM_BIAS_F16 || bias_kind == W8A8_QM_BIAS_BF16) ? 2 : 4;
                                bias = static_cast<const uint8_t*>(bias) + tl.group * p.bias_batch_stride * esz;
                            }
#pragma unroll
                            for (int j = 0; j < 32; ++j) {
                                const int64_t col = col0 + j;
                                float x = static_cast<float>(static_cast<int32_t>(r[j]));
                                if (col < p.N) {
                                    if (bias_kind == W8A8_QM_BIAS_I32) {
                                        x = __fadd_rn(x, vec_elem_as_float(bias, (f & W8A8_QM_BIAS_PERCHAN) ? col : 0,
                                                                           bias_kind));
                                    }
                                    const int64_t si = (f & W8A8_QM_SCALE_PERCHAN) ? col : 0;
                                    const float sc = (f & W8A8_QM_SCALE_BF16)
                                                         ? __bfloat162float(static_cast<const __nv_bfloat16*>(p.scale)[si])
                                                         : static_cast<const float*>(p.scale)[si];
                                    x = __fmul_rn(x, sc);
                                    if (f & W8A8_QM_HAS_OFFSET) {
                                        x = __fadd_rn(x, p.offset[(f & W8A8_QM_OFFSET_PERCHAN) ? col : 0]);
                                    }
                                    if (f & W8A8_QM_HAS_PT) {
                                        x = __fmul_rn(x, row_mul);
                                    }
                                    if (bias_kind >= W8A8_QM_BIAS_F16) {
                                        x = __fadd_rn(x, vec_elem_as_float(bias, (f & W8A8_QM_BIAS_PERCHAN) ? col : 0,
                                                                           bias_kind));
                                    }
                                }
                                v[j] = x;
                            }
                        } else {  // EPI_GMM
                            const int has_bias = static_cast<int>(p.flags & 4);
                            const int bias_dt = static_cast<int>(p.flags & 3);
                            const int64_t gbase = static_cast<int64_t>(tl.group) * p.N;
#pragma unroll
                            for (int j = 0; j < 32; ++j) {
                                const int64_t col = col0 + j;
                                float x;
                                if constexpr (KIND == KIND_I8) {
                                    x = static_cast<float>(static_cast<int32_t>(r[j]));
                                } else {
                                    x = __uint_as_float(r[j]);
                                }
                                if (col < p.N) {
                                    if constexpr (KIND == KIND_I8) {
                                        x = __fmul_rn(__fmul_rn(x, static_cast<const float*>(p.scale)[gbase + col]),
                                                      row_mul);
                                    }
                                    if (has_bias) {
                                        float bv;
                                        if (bias_dt == W8A8_DT_F16) {
                                            bv = __half2float(static_cast<const __half*>(p.bias)[gbase + col]);
                                        } else if (bias_dt == W8A8_DT_BF16) {
                                            bv = __bfloat162float(static_cast<const __nv_bfloat16*>(p.bias)[gbase + col]);
                                        } else {
                                            bv = static_cast<const float*>(p.bias)[gbase + col];
                                        }
                                        x = __fadd_rn(x, bv);
                                    }
                                }
                                v[j] = x;
                            }
                        }
                        // 32 outputs -> four 16-byte stores of 16-bit values
                        uint16_t* dst = static_cast<uint16_t*>(p.out) + row * p.N + col0;
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            if (col0 + q * 8 < p.N) {
                                uint4 o;
                                if (p.out_dtype == W8A8_DT_BF16) {
                                    o = make_uint4(pack2<W8A8_DT_BF16>(v[q * 8], v[q * 8 + 1]),
                                                   pack2<W8A8_DT_BF16>(v[q * 8 + 2], v[q * 8 + 3]),
                                                   pack2<W8A8_DT_BF16>(v[q * 8 + 4], v[q * 8 + 5]),
                                                   pack2<W8A8_DT_BF16>(v[q * 8 + 6], v[q * 8 + 7]));
                                } else {
                                    o = make_uint4(pack2<W8A8_DT_F16>(v[q * 8], v[q * 8 + 1]),
                                                   pack2<W8A8_DT_F16>(v[q * 8 + 2], v[q * 8 + 3]),
                                                   pack2<W8A8_DT_F16>(v[q * 8 + 4], v[q * 8 + 5]),
                                                   pack2<W8A8_DT_F16>(v[q * 8 + 6], v[q * 8 + 7]));
                                }
                                *reinterpret_cast<uint4*>(dst + q * 8) = o;
                            }
                        }
                    }
                }
            }
            // accumulator stage drained: hand it back to the MMA issuer
            tc::tc_fence_before_sync();
            tc::mbar_arrive(tempty_bar(acc));
        }
    }

    // ---- teardown ----
    tc::tc_fence_before_sync();
    __syncthreads();
    if (*abort_flag != 0) {
        // a wait ran out: record it, then give copies still in flight time to land
        if (threadIdx.x == 0) {
            if (p.error != nullptr) {
                atomicExch(p.error, 2);
            }
        }
        const unsigned long long t0 = tc::global_ns();
        while (tc::global_ns() - t0 < 200000ull) {
            __nanosleep(1000);
        }
        __syncthreads();
    }
    if (warp == 1) {
        tc::tc_fence_after_sync();
        tc::tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

}  // namespace w8a8
