// Persistent, warp-specialised tcgen05 GEMM for sm_100a with fused epilogues.
//
// One CTA per SM, 320 threads (576 with the SwiGLU epilogue's sixteen epilogue warps):
//   warp 0      TMA producer: fills a ring of shared-memory stages (128-byte
//               swizzle) with A and B tiles, one mbarrier per stage.
//   warp 1      MMA issuer: one thread issues tcgen05.mma into one of two TMEM
//               accumulator stages; tcgen05.commit releases the shared-memory
//               stage and finally publishes the accumulator.
//   warps 2-9   epilogue: tcgen05.ld the accumulator (a warp may read the 32 TMEM
//               lanes its index modulo 4 selects; two warps share each lane
//               quarter and split the columns), apply the operator's dequant
//               chain, store.  Double-buffered TMEM lets the epilogue of tile i
//               overlap the main loop of tile i+1.  The SwiGLU epilogue (an
//               exponential and an IEEE division per element) runs on warps
//               2-17, four per lane quarter: with eight warps it took as long
//               per tile as the main loop.
//
// Two shapes of the same kernel (template parameter CG):
//   CG = 1  one CTA per tile of 128 rows x BLOCK_N columns, 4 stages of
//           {A 128x128 B, B BLOCK_N x128 B}.  Used for small row counts.
//   CG = 2  a pair of CTAs (cluster of 2, tcgen05 cta_group::2) per tile of 256
//           rows x 256 columns.  Each CTA loads its 128 rows of A and its 128
//           columns of B (6 stages of 32 KB), the even CTA issues the MMAs for
//           both, each CTA's tensor memory receives its 128 rows of the
//           accumulator and each CTA runs its own epilogue.  Halving the B bytes
//           per CTA takes shared-memory and L2->SM traffic per MMA from 96 to 64
//           bytes per clock, which is what lets the tensor pipe stay busy.  No
//           load is multicast: each CTA fetches exactly what it stores.
//
// A is always K-major ([rows, K], K contiguous).  B is either K-major
// ([.., N, K]) or MN-major ([.., K, N], the reference catalog's weight layout);
// both are consumed directly by the tensor core through the descriptor's
// major bit, no transposition pass.
//
// Dense problems enumerate (row tile, column tile) with the row index fastest
// so that concurrently running CTAs share a B column block in L2.  Grouped
// problems read a tile table built on the device from the cumulative group
// list (tiles never straddle groups; rows past a group's end inside a tile
// are computed and discarded) with the column index fastest, so the A tile
// and the expert's weights stay L2-resident.
#pragma once

#include "common.cuh"
#include "tc_ptx.cuh"

namespace w8a8 {

// producer warp, MMA warp and the epilogue warps (8, or 16 for the SwiGLU epilogue, whose per-element arithmetic -
// exp and an IEEE division - otherwise keeps eight warps busy for as long as the MMA warp needs for the tile)
__host__ __device__ constexpr int gemm_threads(int epi_warps) { return 64 + 32 * epi_warps; }
constexpr int GEMM_EPI_PATCH_BYTES = 8 * 4096;  // shared by the epilogue warps: 4 KB each for 8, 2 KB each for 16
constexpr int GEMM_BLOCK_M = 128;
constexpr int GEMM_KBYTES = 128;  // bytes of K per stage row (one swizzle atom)
constexpr int GEMM_A_BYTES = GEMM_BLOCK_M * GEMM_KBYTES;

// pipeline depth: as many 1 KB-aligned stages as fit beside the barriers
__host__ __device__ constexpr int gemm_stages(int cg, int block_n)
{
    return (GEMM_A_BYTES + (block_n / cg) * GEMM_KBYTES) <= 32768 ? 6 : 4;
}

// K blocks (128 bytes of K each) per pipeline stage.  The thread that issues the MMAs pays a fixed price for every
// barrier wait, satisfied or not (measured with the issue probe: about 0.3 us per wait-and-commit against 45 ns
// per instruction, so 4 instructions per wait sustain 2.5 - 3.0 POPS at full clock, 8 per wait 3.5 - 4.3): a stage
// therefore carries two K blocks wherever that still leaves three stages.
__host__ __device__ constexpr int gemm_kblocks_per_stage(int cg, int block_n)
{
#ifdef W8A8_ONE_KBLOCK_PER_STAGE  // comparison builds only
    return 1;
#else
    return (GEMM_A_BYTES + (block_n / cg) * GEMM_KBYTES) <= 32768 ? 2 : 1;
#endif
}

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
    int32_t rows_total;  // the list's last entry: rows the groups cover (may be below M for a device prefix list)
    int32_t pad[61];
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
    const uint64_t* out_row_ptrs;  // GMM: when set, row r is stored at this address instead of out + r*N
    int32_t a_box_bytes;  // bytes one A load delivers: GEMM_A_BYTES, or less when the A map's box has fewer rows
    float* act;       // GMSQ: fp32 activations [M, N/2]
    uint32_t* amax;   // GMSQ: per-row max|act| bit patterns
    // GMSQ with the requantisation fused in: the CTA that finishes the last column tile of its rows quantises them
    int32_t* tile_done;   // per (row tile, CTA of the tile): epilogue warps done with a column tile (zeroed by the caller)
    int8_t* y;            // [M, N/2]
    float* y_scale;       // [M]
    int32_t fuse_requant;
    int32_t round_direct;
};

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

// 32 consecutive per-channel values starting at element `idx0` (16-byte aligned
// for every kind because idx0 is a multiple of 16), widened to fp32; a vector
// that is not per-channel broadcasts element 0.  `valid` is 32 or 16.
__device__ __forceinline__ void load_vec32(const void* base, int64_t idx0, int kind, bool perchan, int valid,
                                           float (&out)[32])
{
    if (!perchan) {
        const float s = vec_elem_as_float(base, 0, kind);
#pragma unroll
        for (int j = 0; j < 32; ++j) {
            out[j] = s;
        }
        return;
    }
    if (kind == W8A8_QM_BIAS_F32 || kind == W8A8_QM_BIAS_I32) {
        const uint4* p4 = reinterpret_cast<const uint4*>(static_cast<const uint32_t*>(base) + idx0);
#pragma unroll
        for (int q = 0; q < 8; ++q) {
            uint4 t = make_uint4(0, 0, 0, 0);
            if (q * 4 < valid) {
                t = __ldg(p4 + q);
            }
            if (kind == W8A8_QM_BIAS_I32) {
                out[q * 4 + 0] = static_cast<float>(static_cast<int32_t>(t.x));
                out[q * 4 + 1] = static_cast<float>(static_cast<int32_t>(t.y));
                out[q * 4 + 2] = static_cast<float>(static_cast<int32_t>(t.z));
                out[q * 4 + 3] = static_cast<float>(static_cast<int32_t>(t.w));
            } else {
                out[q * 4 + 0] = __uint_as_float(t.x);
                out[q * 4 + 1] = __uint_as_float(t.y);
                out[q * 4 + 2] = __uint_as_float(t.z);
                out[q * 4 + 3] = __uint_as_float(t.w);
            }
        }
    } else {
        const uint4* p4 = reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(base) + idx0);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            uint4 t = make_uint4(0, 0, 0, 0);
            if (q * 8 < valid) {
                t = __ldg(p4 + q);
            }
            const uint32_t w[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                if (kind == W8A8_QM_BIAS_BF16) {
                    unpack2<W8A8_DT_BF16>(w[i], out[q * 8 + 2 * i], out[q * 8 + 2 * i + 1]);
                } else {
                    unpack2<W8A8_DT_F16>(w[i], out[q * 8 + 2 * i], out[q * 8 + 2 * i + 1]);
                }
            }
        }
    }
}


// Requantisation of one finished row of SwiGLU activations, 16-byte pieces [c_lo, c_hi) of it, by one warp:
// amax clamp at FLT_MIN, y_scale = amax * (1/127), inv = 127 / amax, clamp to [-128, 127], narrowing
// (gmsq_vec_kernel.cpp:233-257).  The activations and row maxima were written by other SMs: they are read through
// L2 (ld.global.cg), never through this SM's L1.
template <bool DIRECT>
__device__ __forceinline__ void requant_row_part(const float* act, const uint32_t* amax_bits, int8_t* y, float* y_scale,
                                                 int64_t row, int64_t H, int64_t c_lo, int64_t c_hi, bool write_scale,
                                                 int lane)
{
    float amax = __uint_as_float(__ldcg(amax_bits + row));
    if (!(amax > 1.1754944e-38f)) {
        amax = 1.1754944e-38f;
    }
    if (write_scale && lane == 0) {
        y_scale[row] = __fmul_rn(amax, INV127);
    }
    const float inv = __fdiv_rn(127.0f, amax);
    const float4* src = reinterpret_cast<const float4*>(act + row * H);
    uint32_t* dst = reinterpret_cast<uint32_t*>(y + row * H);
    // eight independent 16-byte loads in flight per lane: few warps work here, and a load at a time would leave
    // them waiting on L2 latency
    constexpr int DEPTH = 8;
    for (int64_t c0 = c_lo; c0 < c_hi; c0 += 32 * DEPTH) {
        float4 a[DEPTH];
#pragma unroll
        for (int j = 0; j < DEPTH; ++j) {
            const int64_t c = c0 + lane + 32 * j;
            a[j] = (c < c_hi) ? __ldcg(src + c) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        }
#pragma unroll
        for (int j = 0; j < DEPTH; ++j) {
            const int64_t c = c0 + lane + 32 * j;
            if (c >= c_hi) {
                continue;
            }
            const float w[4] = {__fmul_rn(a[j].x, inv), __fmul_rn(a[j].y, inv), __fmul_rn(a[j].z, inv),
                                __fmul_rn(a[j].w, inv)};
            float v[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                v[q] = fminf(fmaxf(w[q], -128.0f), 127.0f);
            }
            uint32_t packed = narrow4_fast<DIRECT>(v[0], v[1], v[2], v[3]);
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                if (w[q] != w[q]) {  // a NaN activation narrows to 0 (fmaxf / fminf turned it into a bound)
                    packed &= ~(0xffu << (8 * q));
                }
            }
            __stcs(dst + c, packed);
        }
    }
}

struct TileInfo {
    int32_t a_row0;  // first row this CTA loads and owns (global row index)
    int32_t m_rows;  // valid rows among this CTA's 128
    int32_t group;   // expert / batch (B's outermost coordinate)
    int32_t nt;      // column tile
    int32_t mt;      // row tile (grouped: index into the tile table)
};

// The work of one epilogue thread on one tile: row `row_in_tile` of this CTA's
// accumulator, columns [col_half * BLOCK_N/2, (col_half+1) * BLOCK_N/2).
template <int BLOCK_N, int KIND, int EPI, int EPI_WARPS>
__device__ __forceinline__ void epilogue_tile(const GemmParams& p, const TileInfo& tl, uint32_t t_addr,
                                              int row_in_tile, int col_half, int64_t H, bool no_epilogue,
                                              uint4* stage)
{
    const bool row_ok = (row_in_tile < tl.m_rows) && !no_epilogue;
    const int64_t row = static_cast<int64_t>(tl.a_row0) + row_in_tile;  // global row (A and output)
    if constexpr (EPI == EPI_GMSQ) {
        const float xs = row_ok ? p.row_scale[row] : 0.0f;
        const float* wsg = static_cast<const float*>(p.scale) + static_cast<int64_t>(tl.group) * p.N;
        float local_max = 0.0f;
        // `col_half` counts this warp among the EPI_WARPS / 4 warps that share a TMEM lane quarter: each takes
        // 128 / (EPI_WARPS / 4) activation columns, 16 at a time
        constexpr int WARP_COLS = 128 / (EPI_WARPS / 4);
#pragma unroll 1
        for (int cc = 0; cc < WARP_COLS; cc += 16) {
            const int c = col_half * WARP_COLS + cc;
            uint32_t g[16], u[16];
            tc::tmem_ld_32x16(t_addr + c, g);
            tc::tmem_ld_32x16(t_addr + 128 + c, u);
            tc::tmem_ld_wait();
            const int64_t col0 = static_cast<int64_t>(tl.nt) * 128 + c;  // column in [0, H)
            const int lane = row_in_tile & 31;
            if (row_ok) {
#pragma unroll
                for (int q = 0; q < 4; ++q) {
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
                        // parked in the warp's shared-memory patch: piece q of row `lane`, the pieces permuted by
                        // the row so that the eight lanes of a store phase hit eight different bank groups
                        stage[lane * 4 + (q ^ ((lane ^ (lane >> 2)) & 3))] =
                            make_uint4(__float_as_uint(a[0]), __float_as_uint(a[1]), __float_as_uint(a[2]),
                                       __float_as_uint(a[3]));
                    }
                }
            }
            // the 16 activations of each row are a 64-byte piece of a line: written by 4 lanes per row, 8 rows per
            // instruction, instead of 16-byte pieces of 32 different rows
            __syncwarp();
            {
                const int piece = lane & 3;
                const int64_t col = col0 + piece * 4;
                const int first_row = row_in_tile & ~31;
#pragma unroll
                for (int it = 0; it < 4; ++it) {
                    const int rr = it * 8 + (lane >> 2);
                    if (first_row + rr < tl.m_rows && !no_epilogue && col < H) {
                        const uint4 val = stage[rr * 4 + (piece ^ ((rr ^ (rr >> 2)) & 3))];
                        *reinterpret_cast<uint4*>(p.act + (static_cast<int64_t>(tl.a_row0) + first_row + rr) * H + col) =
                            val;
                    }
                }
            }
            __syncwarp();
        }
        if (row_ok) {
            atomicMax(reinterpret_cast<int*>(p.amax + row), __float_as_int(local_max));
        }
    } else {
        // per-tile invariants of the dequant chain, hoisted out of the column loops
        float row_mul = 1.0f;
        bool has_pt = false;
        int bias_kind = W8A8_QM_BIAS_NONE;
        bool bias_perchan = false, scale_perchan = true, scale_bf16 = false, has_offset = false,
             offset_perchan = false;
        const void* bias = p.bias;
        int64_t vec_base = 0;  // first element of the per-channel vectors for this tile's group
        if constexpr (EPI == EPI_QMM) {
            const int64_t f = p.flags;
            has_pt = (f & W8A8_QM_HAS_PT) != 0;
            if (has_pt && row_ok) {
                // the plugin's layouts make (row mod M) the token index in every case
                row_mul = p.row_scale[(tl.group == 0) ? row : (row - static_cast<int64_t>(tl.group) * p.M)];
            }
            bias_kind = static_cast<int>((f & W8A8_QM_BIAS_MASK) >> W8A8_QM_BIAS_SHIFT);
            bias_perchan = (f & W8A8_QM_BIAS_PERCHAN) != 0;
            scale_perchan = (f & W8A8_QM_SCALE_PERCHAN) != 0;
            scale_bf16 = (f & W8A8_QM_SCALE_BF16) != 0;
            has_offset = (f & W8A8_QM_HAS_OFFSET) != 0;
            offset_perchan = (f & W8A8_QM_OFFSET_PERCHAN) != 0;
            if (bias != nullptr && p.bias_batch_stride != 0) {
                const int64_t esz = (bias_kind == W8A8_QM_BIAS_F16 || bias_kind == W8A8_QM_BIAS_BF16) ? 2 : 4;
                bias = static_cast<const uint8_t*>(bias) + tl.group * p.bias_batch_stride * esz;
            }
        } else if constexpr (EPI == EPI_GMM) {
            if constexpr (KIND == KIND_I8) {
                row_mul = row_ok ? p.row_scale[row] : 0.0f;
            }
            vec_base = static_cast<int64_t>(tl.group) * p.N;
            if (p.flags & 4) {
                const int bdt = static_cast<int>(p.flags & 3);
                bias_kind = (bdt == W8A8_DT_F16) ? W8A8_QM_BIAS_F16
                                                  : (bdt == W8A8_DT_BF16 ? W8A8_QM_BIAS_BF16 : W8A8_QM_BIAS_F32);
                bias_perchan = true;
            }
        }
        constexpr int HALF_COLS = BLOCK_N / 2;
        // byte address of this thread's output row (16-bit outputs; fp32 outputs are addressed where they are stored)
        uint64_t row_ptr = reinterpret_cast<uint64_t>(p.out) + static_cast<uint64_t>(row) * p.N * 2;
        if constexpr (EPI == EPI_GMM) {
            if (p.out_row_ptrs != nullptr) {
                // the row's home may be another GPU's memory: plain peer stores over NVLink
                row_ptr = (row_in_tile < tl.m_rows) ? p.out_row_ptrs[row] : 0;
            }
        }
#pragma unroll 1
        for (int cc = 0; cc < HALF_COLS; cc += 32) {
            const int c = col_half * HALF_COLS + cc;
            uint32_t r[32];
            tc::tmem_ld_32x32(t_addr + c, r);
            tc::tmem_ld_wait();
            const int64_t col0 = static_cast<int64_t>(tl.nt) * BLOCK_N + c;
            if constexpr (EPI == EPI_RAW) {
                if (!row_ok || col0 >= p.N) {
                    continue;
                }
            }
            // N is a multiple of 16: a chunk holds 32, 16 or no valid columns
            const int valid = (col0 >= p.N) ? 0 : ((col0 + 32 <= p.N) ? 32 : 16);
            if constexpr (EPI == EPI_RAW) {
                int32_t* dst = static_cast<int32_t*>(p.out) + row * p.N + col0;
#pragma unroll
                for (int q = 0; q < 8; ++q) {
                    if (q * 4 < valid) {
                        *reinterpret_cast<uint4*>(dst + q * 4) =
                            make_uint4(r[q * 4], r[q * 4 + 1], r[q * 4 + 2], r[q * 4 + 3]);
                    }
                }
            } else {
                float v[32];
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                    if constexpr (KIND == KIND_I8) {
                        v[j] = static_cast<float>(static_cast<int32_t>(r[j]));
                    } else {
                        v[j] = __uint_as_float(r[j]);
                    }
                }
                float w[32];
                if constexpr (EPI == EPI_QMM) {
                    if (bias_kind == W8A8_QM_BIAS_I32) {
                        load_vec32(bias, col0, bias_kind, bias_perchan, valid, w);
#pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            v[j] = __fadd_rn(v[j], w[j]);
                        }
                    }
                    load_vec32(p.scale, col0, scale_bf16 ? W8A8_QM_BIAS_BF16 : W8A8_QM_BIAS_F32, scale_perchan,
                               valid, w);
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        v[j] = __fmul_rn(v[j], w[j]);
                    }
                    if (has_offset) {
                        load_vec32(p.offset, col0, W8A8_QM_BIAS_F32, offset_perchan, valid, w);
#pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            v[j] = __fadd_rn(v[j], w[j]);
                        }
                    }
                    if (has_pt) {
#pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            v[j] = __fmul_rn(v[j], row_mul);
                        }
                    }
                    if (bias_kind >= W8A8_QM_BIAS_F16) {
                        load_vec32(bias, col0, bias_kind, bias_perchan, valid, w);
#pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            v[j] = __fadd_rn(v[j], w[j]);
                        }
                    }
                } else {  // EPI_GMM
                    if constexpr (KIND == KIND_I8) {
                        load_vec32(p.scale, vec_base + col0, W8A8_QM_BIAS_F32, true, valid, w);
#pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            v[j] = __fmul_rn(__fmul_rn(v[j], w[j]), row_mul);
                        }
                    }
                    if (bias_kind != W8A8_QM_BIAS_NONE) {
                        load_vec32(bias, vec_base + col0, bias_kind, true, valid, w);
#pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            v[j] = __fadd_rn(v[j], w[j]);
                        }
                    }
                }
                if constexpr (EPI == EPI_GMM && KIND == KIND_BF16) {
                    if (p.out_dtype == W8A8_DT_F32) {
                        // fp32 output (the split-operand path): 32 values are one whole 128-byte line of the row
                        if (row_ok) {
                            float* dst = static_cast<float*>(p.out) + row * p.N + col0;
#pragma unroll
                            for (int q = 0; q < 8; ++q) {
                                if (q * 4 < valid) {
                                    *reinterpret_cast<float4*>(dst + q * 4) =
                                        make_float4(v[q * 4], v[q * 4 + 1], v[q * 4 + 2], v[q * 4 + 3]);
                                }
                            }
                        }
                        continue;
                    }
                }
                // 32 outputs = 64 bytes of this thread's row.  They are not stored from here (every lane would
                // write 16-byte pieces of a different row): the warp parks two such chunks, 128 bytes per row, in
                // its private shared-memory patch and then writes whole 128-byte row segments, 8 lanes per row.
                // That matters most when the row's home is another GPU: NVLink carries full lines, not fragments.
                uint4 o[4];
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    if (p.out_dtype == W8A8_DT_BF16) {
                        o[q] = make_uint4(pack2<W8A8_DT_BF16>(v[q * 8], v[q * 8 + 1]),
                                          pack2<W8A8_DT_BF16>(v[q * 8 + 2], v[q * 8 + 3]),
                                          pack2<W8A8_DT_BF16>(v[q * 8 + 4], v[q * 8 + 5]),
                                          pack2<W8A8_DT_BF16>(v[q * 8 + 6], v[q * 8 + 7]));
                    } else {
                        o[q] = make_uint4(pack2<W8A8_DT_F16>(v[q * 8], v[q * 8 + 1]),
                                          pack2<W8A8_DT_F16>(v[q * 8 + 2], v[q * 8 + 3]),
                                          pack2<W8A8_DT_F16>(v[q * 8 + 4], v[q * 8 + 5]),
                                          pack2<W8A8_DT_F16>(v[q * 8 + 6], v[q * 8 + 7]));
                    }
                }
                const int lane = row_in_tile & 31;
                const int sub = (cc >> 5) & 1;  // which half of the 64-column patch
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    // row `lane`, 16-byte piece (sub*4 + q), pieces xor-swizzled by the row so that the eight
                    // lanes of a quarter-warp hit eight different bank groups
                    stage[lane * 8 + ((sub * 4 + q) ^ (lane & 7))] = o[q];
                }
                if (sub == 1) {
                    __syncwarp();
                    const int64_t patch_col0 = col0 - 32;  // first column of the 64-column patch
                    const int piece = lane & 7;
                    const int64_t pc = patch_col0 + piece * 8;
                    const int first_row = row_in_tile & ~31;
#pragma unroll
                    for (int it = 0; it < 8; ++it) {
                        const int rr = it * 4 + (lane >> 3);  // row within the warp's 32
                        const uint64_t rp = __shfl_sync(FULL_MASK, row_ptr, rr);
                        const uint4 val = stage[rr * 8 + (piece ^ (rr & 7))];
                        if (first_row + rr < tl.m_rows && !no_epilogue && pc < p.N) {
                            *reinterpret_cast<uint4*>(rp + static_cast<uint64_t>(pc) * 2) = val;
                        }
                    }
                    __syncwarp();
                }
            }
        }
    }
}

template <int CG, int BLOCK_N, int KIND, int EPI, bool B_MN, int EPI_WARPS>
__global__ void __launch_bounds__(gemm_threads(EPI_WARPS), 1)
    gemm_tc_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                   const GemmParams p)
{
    constexpr int ELEM = (KIND == KIND_I8) ? 1 : 2;
    constexpr int BLOCK_K = GEMM_KBYTES / ELEM;    // elements of K per stage
    constexpr int UMMA_K = 32 / ELEM;              // elements of K per instruction
    constexpr int CTA_N = BLOCK_N / CG;            // B columns this CTA loads
    constexpr int NBOX = CTA_N * ELEM / 128;       // MN-major: 128-byte-wide column blocks this CTA loads
    constexpr int B_BYTES = CTA_N * GEMM_KBYTES;
    constexpr int KB_BYTES = GEMM_A_BYTES + B_BYTES;           // one K block: 128 bytes of K of A and of B
    constexpr int KPS = gemm_kblocks_per_stage(CG, BLOCK_N);   // K blocks per stage
    constexpr int STAGE_BYTES = KPS * KB_BYTES;
    constexpr int STAGES = gemm_stages(CG, BLOCK_N) / KPS;
    constexpr uint32_t TMEM_COLS = 2 * BLOCK_N;    // 256 or 512: power of two
    constexpr uint32_t UMMA_M = 128 * CG;
    constexpr uint32_t IDESC =
        (KIND == KIND_I8) ? tc::instr_desc(2u, 1u, B_MN ? 1u : 0u, UMMA_M, BLOCK_N)
                          : tc::instr_desc(1u, (KIND == KIND_BF16) ? 1u : 0u, B_MN ? 1u : 0u, UMMA_M, BLOCK_N);
    static_assert(BLOCK_N == 128 || BLOCK_N == 256, "BLOCK_N");
    static_assert(CG == 1 || BLOCK_N == 256, "CTA pairs use 256-column tiles");
    static_assert(EPI != EPI_GMSQ || BLOCK_N == 256, "the SwiGLU epilogue pairs 128 gate with 128 up columns");
    static_assert(EPI_WARPS == 8 || (EPI_WARPS == 16 && EPI == EPI_GMSQ), "16 epilogue warps: SwiGLU epilogue only");

    extern __shared__ uint8_t smem_raw[];
    // 1024-byte alignment: required by the 128-byte swizzle atoms.  The dynamic shared memory window starts at
    // the same offset in both CTAs of a pair, so the layout below is identical in both.
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
    // bars[0..S) full, [S..2S) empty, [2S..2S+2) tmem_full, [2S+2..2S+4) tmem_empty
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 6);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t cta_rank = (CG == 2) ? tc::cluster_ctarank() : 0u;
    const bool leader = (cta_rank == 0);
    const uint32_t smem_base = tc::smem_u32(smem);
    const uint32_t bar_base = tc::smem_u32(bars);
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
    auto tfull_bar = [&](int s) { return bar_base + 8u * (2 * STAGES + s); };
    auto tempty_bar = [&](int s) { return bar_base + 8u * (2 * STAGES + 2 + s); };

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            tc::mbar_init(full_bar(s), 1);   // the (leader's) producer's arrive.expect_tx; bytes from every CTA of the tile
            tc::mbar_init(empty_bar(s), 1);  // one commit (multicast to both CTAs of a pair)
        }
        for (int s = 0; s < 2; ++s) {
            tc::mbar_init(tfull_bar(s), 1);
            tc::mbar_init(tempty_bar(s), EPI_WARPS * CG);  // one arrival per epilogue warp of every CTA on the tile
        }
        *abort_flag = 0;
        tc::fence_mbar_init();
        tc::prefetch_tensormap(&tm_a);
        tc::prefetch_tensormap(&tm_b);
    }
    if (warp == 1) {
        // each CTA allocates its own tensor memory; a pair asks for all 512 columns in both CTAs, so the
        // accumulator has the same column address in both, as the paired MMA requires
        tc::tmem_alloc(tc::smem_u32(tmem_slot), TMEM_COLS);
        tc::tmem_relinquish();
    }
    tc::tc_fence_before_sync();
    __syncthreads();
    if constexpr (CG == 2) {
        // both CTAs' barriers must be initialised before either signals the other
        tc::cluster_arrive();
        tc::cluster_wait();
    }
    tc::tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    // ---- tile enumeration (identical in every role and in both CTAs of a pair) ----
    constexpr int TILE_M = 128 * CG;
    int64_t total_tiles;
    int32_t dense_m_tiles = 0;
    if (p.grouped) {
        total_tiles = static_cast<int64_t>(p.header->num_m_tiles) * p.n_tiles;
    } else {
        dense_m_tiles = p.batch * p.m_tiles_per_batch;
        total_tiles = static_cast<int64_t>(dense_m_tiles) * p.n_tiles;
    }
    const int64_t H = p.N / 2;  // GMSQ half width
    const int64_t worker = blockIdx.x / CG;
    const int64_t num_workers = gridDim.x / CG;

    auto decode = [&](int64_t t) {
        TileInfo tl;
        int64_t tile_row0;
        int32_t tile_rows;
        if (p.grouped) {
            const int32_t mt = static_cast<int32_t>(t / p.n_tiles);
            tl.nt = static_cast<int32_t>(t % p.n_tiles);
            tl.mt = mt;
            const TileEntry e = p.tiles[mt];
            tile_row0 = e.m_start;
            tile_rows = e.m_rows;
            tl.group = e.group;
        } else {
            const int32_t mg = static_cast<int32_t>(t % dense_m_tiles);
            tl.nt = static_cast<int32_t>(t / dense_m_tiles);
            tl.mt = mg;
            const int32_t b = mg / p.m_tiles_per_batch;
            const int32_t mt = mg % p.m_tiles_per_batch;
            const int64_t m0 = static_cast<int64_t>(mt) * TILE_M;
            tile_row0 = b * p.M + m0;
            const int64_t left = p.M - m0;
            tile_rows = static_cast<int32_t>(left < TILE_M ? left : TILE_M);
            tl.group = b;
        }
        tl.a_row0 = static_cast<int32_t>(tile_row0 + 128 * static_cast<int64_t>(cta_rank));
        int32_t mine = tile_rows - 128 * static_cast<int32_t>(cta_rank);
        tl.m_rows = mine < 0 ? 0 : (mine > 128 ? 128 : mine);
        return tl;
    };
    // first column (MN-major) / first N row (K-major) of block `i` among the blocks THIS CTA loads for column
    // tile nt.  With the SwiGLU epilogue the first half of the tile's columns are gate columns and the second
    // half the matching up columns, H apart in the weight.
    auto b_block_origin = [&](int32_t nt, int i, int block_width) -> int32_t {
        const int g = static_cast<int>(cta_rank) * (CTA_N / block_width) + i;  // block index within the full tile
        const int per_half = (BLOCK_N / 2) / block_width;
        if constexpr (EPI == EPI_GMSQ) {
            const int64_t base = (g < per_half ? 0 : H) + static_cast<int64_t>(nt) * (BLOCK_N / 2);
            return static_cast<int32_t>(base + (g % per_half) * block_width);
        } else {
            return nt * BLOCK_N + g * block_width;
        }
    };

    if (warp == 0) {
        // ===================== TMA producer =====================
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            // a pair credits both CTAs' bytes to the leader's barrier
            const uint32_t full0 = (CG == 2) ? tc::map_to_cta(full_bar(0), 0) : full_bar(0);
            for (int64_t t = worker; ok && t < total_tiles; t += num_workers) {
                const TileInfo tl = decode(t);
                for (int kb0 = 0; kb0 < p.num_k_blocks; kb0 += KPS) {
                    if (!tc::mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag)) {
                        ok = false;
                        break;
                    }
                    const int left = p.num_k_blocks - kb0;
                    const int n_sub = left < KPS ? left : KPS;  // K blocks this stage carries (the tile's last may be short)
                    const uint32_t fb = full0 + 8u * stage;
                    // Only the leader announces the bytes (its own and its partner's).  The partner's copies may
                    // complete first: the barrier's phase cannot end before the leader's arrival, and a
                    // transaction count may run ahead of its announcement.
                    if (leader) {
                        tc::mbar_arrive_expect_tx(full_bar(stage),
                                                  CG * n_sub * (static_cast<uint32_t>(p.a_box_bytes) + B_BYTES));
                    }
#pragma unroll
                    for (int sub = 0; sub < KPS; ++sub) {
                        if (sub >= n_sub) {
                            break;
                        }
                        const int kb = kb0 + sub;
                        const uint32_t a_dst = smem_base + stage * STAGE_BYTES + sub * KB_BYTES;
                        const uint32_t b_dst = a_dst + GEMM_A_BYTES;
                        if constexpr (CG == 2) {
                            tc::tma_load_2d_pair(a_dst, &tm_a, fb, kb * BLOCK_K, tl.a_row0);
                        } else {
                            tc::tma_load_2d(a_dst, &tm_a, fb, kb * BLOCK_K, tl.a_row0);
                        }
                        if constexpr (B_MN) {
                            // boxes of {128 bytes of N, BLOCK_K rows of K}
                            constexpr int BOX_BYTES = BLOCK_K * 128;
                            constexpr int BOX_COLS = 128 / ELEM;
#pragma unroll
                            for (int i = 0; i < NBOX; ++i) {
                                const int32_t col = b_block_origin(tl.nt, i, BOX_COLS);
                                if constexpr (CG == 2) {
                                    tc::tma_load_3d_pair(b_dst + i * BOX_BYTES, &tm_b, fb, col, kb * BLOCK_K, tl.group);
                                } else {
                                    tc::tma_load_3d(b_dst + i * BOX_BYTES, &tm_b, fb, col, kb * BLOCK_K, tl.group);
                                }
                            }
                        } else {
                            // boxes of {128 bytes of K, 128 rows of N}
                            constexpr int BOXES = CTA_N / 128;
#pragma unroll
                            for (int i = 0; i < BOXES; ++i) {
                                const int32_t n_row = b_block_origin(tl.nt, i, 128);
                                if constexpr (CG == 2) {
                                    tc::tma_load_3d_pair(b_dst + i * 128 * GEMM_KBYTES, &tm_b, fb, kb * BLOCK_K, n_row,
                                                         tl.group);
                                } else {
                                    tc::tma_load_3d(b_dst + i * 128 * GEMM_KBYTES, &tm_b, fb, kb * BLOCK_K, n_row,
                                                    tl.group);
                                }
                            }
                        }
                    }
                    if (++stage == STAGES) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ===================== MMA issuer (leader CTA only) =====================
        if (lane == 0 && leader) {
            // Descriptors as {lo, hi}: hi is loop invariant; a byte offset adds (offset >> 4) to lo.
            const uint64_t a_desc0 = tc::smem_desc_sw128(smem_base, 16, 1024);
            const uint64_t b_desc0 = B_MN ? tc::smem_desc_sw128(smem_base + GEMM_A_BYTES, BLOCK_K * 128, 1024)
                                          : tc::smem_desc_sw128(smem_base + GEMM_A_BYTES, 16, 1024);
            const uint32_t a_hi = static_cast<uint32_t>(a_desc0 >> 32);
            const uint32_t b_hi = static_cast<uint32_t>(b_desc0 >> 32);
            const uint32_t a_lo0 = static_cast<uint32_t>(a_desc0);
            const uint32_t b_lo0 = static_cast<uint32_t>(b_desc0);
            constexpr uint32_t STAGE_STEP = STAGE_BYTES >> 4;
            constexpr uint32_t KB_STEP = KB_BYTES >> 4;
            constexpr uint32_t A_KSTEP = 32 >> 4;                                   // 32 bytes of K
            constexpr uint32_t B_KSTEP = B_MN ? ((UMMA_K * 128) >> 4) : (32 >> 4);  // UMMA_K rows of 128 bytes, or 32 bytes
            constexpr int KSTEPS = BLOCK_K / UMMA_K;
            int stage = 0;
            uint32_t phase = 0;
            int64_t it = 0;
            bool ok = true;
            for (int64_t t = worker; ok && t < total_tiles; t += num_workers, ++it) {
                const int acc = static_cast<int>(it & 1);
                const uint32_t acc_phase = static_cast<uint32_t>((it >> 1) & 1);
                if (!tc::mbar_wait_cluster(tempty_bar(acc), acc_phase ^ 1u, abort_flag)) {
                    ok = false;
                    break;
                }
                tc::tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * BLOCK_N);
                uint32_t accumulate = 0;
                for (int kb0 = 0; kb0 < p.num_k_blocks; kb0 += KPS) {
                    // The copies are consumed by the tensor core (async proxy), not by this thread: the barrier's
                    // default acquire plus the tcgen05 fence is what orders them, also for the partner CTA's
                    // copies that complete on this barrier.
                    if (!tc::mbar_wait(full_bar(stage), phase, abort_flag)) {
                        ok = false;
                        break;
                    }
                    tc::tc_fence_after_sync();
                    const int left = p.num_k_blocks - kb0;
                    const int n_sub = left < KPS ? left : KPS;
#pragma unroll
                    for (int sub = 0; sub < KPS; ++sub) {
                        if (sub >= n_sub) {
                            break;
                        }
                        const uint32_t a_lo = a_lo0 + stage * STAGE_STEP + sub * KB_STEP;
                        const uint32_t b_lo = b_lo0 + stage * STAGE_STEP + sub * KB_STEP;
#pragma unroll
                        for (int k = 0; k < KSTEPS; ++k) {
                            tc::mma_lohi<CG, KIND == KIND_I8>(d_tmem, a_lo + k * A_KSTEP, a_hi, b_lo + k * B_KSTEP, b_hi,
                                                             IDESC, accumulate);
                            accumulate = 1;
                        }
                    }
                    // one commit hands the whole stage back to the producer
                    if constexpr (CG == 2) {
                        tc::tc_commit_pair(empty_bar(stage));
                    } else {
                        tc::tc_commit(empty_bar(stage));
                    }
                    if (++stage == STAGES) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
                if (ok) {
                    if constexpr (CG == 2) {
                        tc::tc_commit_pair(tfull_bar(acc));
                    } else {
                        tc::tc_commit(tfull_bar(acc));
                    }
                }
            }
        }
        __syncwarp();
    } else {
        // ===================== epilogue (warps 2 .. 2 + EPI_WARPS) =====================
        // EPI_WARPS / 4 warps per TMEM lane quarter; they split the tile's columns evenly.
        const int quarter = warp & 3;          // TMEM lanes [32*quarter, 32*quarter+32)
        const int col_half = (warp - 2) >> 2;  // which share of the columns
        const int row_in_tile = quarter * 32 + lane;
        const bool no_epilogue = false;
        // this warp's patch (4 KB, or 2 KB with 16 warps) for turning per-thread rows into whole-segment stores
        uint4* stage = reinterpret_cast<uint4*>(smem + STAGES * STAGE_BYTES + 512) +
                       (warp - 2) * (GEMM_EPI_PATCH_BYTES / 16 / EPI_WARPS);
        const uint32_t tempty0 = (CG == 2) ? tc::map_to_cta(tempty_bar(0), 0) : tempty_bar(0);
        int64_t it = 0;
        bool ok = true;
        // Requantisation inside this kernel (SwiGLU epilogue, optional).  The rows of a row tile are shared out
        // among the CTAs that compute its column tiles: the CTA of column tile nt quantises rows nt, nt + n_tiles,
        // ... of its 128, one row per warp at a time, once every column tile of the rows has been counted in
        // tile_done.  Column tiles of one row tile are consecutive tile numbers, so they run on different CTAs at
        // the same time (the host switches this on only when there are at least n_tiles workers): a wait here
        // only ever depends on tiles with smaller numbers than the waiter's current one, and it is bounded like
        // every other wait of the kernel.
        TileInfo late{};
        bool have_late = false;
        auto requant_share = [&](const TileInfo& d) -> bool {
            // work units of this CTA for the tile: (row d.nt + n_tiles * k, half h of the row), unit = 2 k + h
            const int units = 2 * ((d.m_rows - d.nt + p.n_tiles - 1) / p.n_tiles);
            if (warp - 2 >= units) {
                return true;
            }
            const int want = p.n_tiles * EPI_WARPS;
            int seen = 0;
            if (lane == 0) {
                const int* counter = p.tile_done + static_cast<int64_t>(d.mt) * CG + cta_rank;
                const long long t0 = clock64();
                while ((seen = tc::ld_acquire_gpu(counter)) < want) {
                    if (*abort_flag != 0 || clock64() - t0 > tc::WAIT_LIMIT_CYCLES) {
                        *abort_flag = 1;
                        break;
                    }
                    __nanosleep(100);
                }
            }
            seen = __shfl_sync(0xffffffffu, seen, 0);
            if (seen < want) {
                return false;
            }
            const int64_t n4 = H / 4, mid = n4 / 2;
            for (int u = warp - 2; u < units; u += EPI_WARPS) {
                const int64_t row = static_cast<int64_t>(d.a_row0) + d.nt + p.n_tiles * (u >> 1);
                const bool second = (u & 1) != 0;
                if (p.round_direct) {
                    requant_row_part<true>(p.act, p.amax, p.y, p.y_scale, row, H, second ? mid : 0, second ? n4 : mid,
                                           !second, lane);
                } else {
                    requant_row_part<false>(p.act, p.amax, p.y, p.y_scale, row, H, second ? mid : 0, second ? n4 : mid,
                                            !second, lane);
                }
            }
            return true;
        };
        for (int64_t t = worker; ok && t < total_tiles; t += num_workers, ++it) {
            const TileInfo tl = decode(t);
            const int acc = static_cast<int>(it & 1);
            const uint32_t acc_phase = static_cast<uint32_t>((it >> 1) & 1);
            if (!tc::mbar_wait(tfull_bar(acc), acc_phase, abort_flag)) {
                ok = false;
                break;
            }
            tc::tc_fence_after_sync();
            const uint32_t t_addr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) +
                                    static_cast<uint32_t>(acc * BLOCK_N);
            epilogue_tile<BLOCK_N, KIND, EPI, EPI_WARPS>(p, tl, t_addr, row_in_tile, col_half, H, no_epilogue, stage);
            // accumulator stage drained: hand it back to the MMA issuer (one arrival per warp)
            tc::tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) {
                if constexpr (CG == 2) {
                    tc::mbar_arrive_cluster(tempty0 + 8u * acc);
                } else {
                    tc::mbar_arrive(tempty0 + 8u * acc);
                }
            }
            if constexpr (EPI == EPI_GMSQ) {
                if (p.fuse_requant) {
                    // Publish this warp's activation stores and row maxima, then count the warp on its row tile:
                    // the rows are complete when n_tiles * EPI_WARPS warps have been counted.
                    __threadfence();
                    __syncwarp();
                    if (lane == 0) {
                        atomicAdd(p.tile_done + static_cast<int64_t>(tl.mt) * CG + cta_rank, 1);
                    }
                    // This tile's share of the requantisation is taken one tile late: by then the other column
                    // tiles of the same rows (on other CTAs, at about the same time) have been counted, so the wait
                    // inside costs one load.  (Two tiles late measured slower: the second pending tile goes to
                    // local memory.)
                    if (have_late && !requant_share(late)) {
                        ok = false;
                        break;
                    }
                    late = tl;
                    have_late = true;
                }
            }
        }
        if constexpr (EPI == EPI_GMSQ) {
            if (p.fuse_requant && ok && have_late) {
                requant_share(late);
            }
        }
    }

    // ---- teardown ----
    tc::tc_fence_before_sync();
    __syncthreads();
    if (*abort_flag != 0) {
        // a wait ran out: record it, then give copies still in flight time to land
        if (threadIdx.x == 0 && p.error != nullptr) {
            atomicExch(p.error, 2);
        }
        const long long t0 = clock64();
        while (clock64() - t0 < 400000ll) {
            __nanosleep(1000);
        }
        __syncthreads();
    }
    if constexpr (CG == 2) {
        // neither CTA may release tensor memory or exit while its partner can still signal it
        tc::cluster_arrive();
        tc::cluster_wait();
    }
    if (warp == 1) {
        tc::tc_fence_after_sync();
        tc::tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

}  // namespace w8a8
