// Measurement and self-test entry points of the tensor-core layer.
//
// w8a8_mma_issue_probe: every SM (or SM pair) issues a long run of tcgen05.mma
// kind::i8 instructions on operands that already sit in shared memory: no TMA,
// no epilogue.  Timed by the caller with CUDA events it gives the rate the
// tensor pipe sustains for one instruction shape (M, N, operand majors, one or
// two CTAs per instruction) - the ceiling the full matmul kernels are compared
// with, and the figure that says what a narrow or a half-height instruction
// costs.
//
// w8a8_selftest_bounded_wait: one CTA waits on a barrier nobody arrives at,
// with a caller-given cycle limit, and reports that the wait ran out the way
// the matmul kernels do (error word 2).  Ends by itself after `limit` cycles.
#include "common.cuh"
#include "tc_ptx.cuh"

namespace w8a8 {

constexpr int PROBE_THREADS = 128;
constexpr int PROBE_STAGES = 4;
constexpr int PROBE_A_BYTES = 16384;                       // 128 rows x 128 bytes of K
constexpr int PROBE_B_BYTES = 32768;                       // up to 256 columns x 128 bytes of K
constexpr int PROBE_STAGE_BYTES = PROBE_A_BYTES + PROBE_B_BYTES;
constexpr int PROBE_MAX_DEPTH = 8;                         // most batches in flight
constexpr int PROBE_KSTEPS = 4;                            // K steps of 32 bytes one stage holds

template <int CG>
__global__ void __launch_bounds__(PROBE_THREADS, 1)
    mma_issue_probe_kernel(uint32_t idesc, int a_mn, int b_mn, int fill, int accumulators, int per_commit, int depth,
                           int pattern, long long batches, int32_t* error)
{
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + PROBE_STAGES * PROBE_STAGE_BYTES);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + PROBE_MAX_DEPTH + 1);  // one spare barrier
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    const int warp = threadIdx.x >> 5;
    const uint32_t cta_rank = (CG == 2) ? tc::cluster_ctarank() : 0u;

    // operands: zeros, or bytes from a multiplicative hash of the address (every bit toggles)
    {
        uint32_t* words = reinterpret_cast<uint32_t*>(smem);
        const int n_words = PROBE_STAGES * PROBE_STAGE_BYTES / 4;
        for (int i = threadIdx.x; i < n_words; i += PROBE_THREADS) {
            uint32_t v = 0;
            if (fill != 0) {
                v = (static_cast<uint32_t>(i) + 0x9e3779b9u * (blockIdx.x + 1)) * 2654435761u;
                v ^= v >> 15;
                v *= 2246822519u;
                v ^= v >> 13;
            }
            words[i] = v;
        }
    }
    if (threadIdx.x == 0) {
        for (int i = 0; i < PROBE_MAX_DEPTH + 1; ++i) {
            tc::mbar_init(tc::smem_u32(bars + i), 1);
        }
        *abort_flag = 0;
        tc::fence_mbar_init();
    }
    if (warp == 0) {
        tc::tmem_alloc(tc::smem_u32(tmem_slot), 512);
        tc::tmem_relinquish();
    }
    // generic-proxy writes of the operands must be visible to the tensor core's async-proxy reads
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    tc::tc_fence_before_sync();
    __syncthreads();
    if constexpr (CG == 2) {
        tc::cluster_arrive();
        tc::cluster_wait();
    }
    tc::tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (threadIdx.x == 0 && cta_rank == 0) {
        const uint32_t smem_base = tc::smem_u32(smem);
        const uint64_t a_desc0 = a_mn ? tc::smem_desc_sw128(smem_base, 128 * 128, 1024)
                                      : tc::smem_desc_sw128(smem_base, 16, 1024);
        const uint64_t b_desc0 = b_mn ? tc::smem_desc_sw128(smem_base + PROBE_A_BYTES, 128 * 128, 1024)
                                      : tc::smem_desc_sw128(smem_base + PROBE_A_BYTES, 16, 1024);
        const uint32_t a_hi = static_cast<uint32_t>(a_desc0 >> 32);
        const uint32_t b_hi = static_cast<uint32_t>(b_desc0 >> 32);
        const uint32_t a_lo0 = static_cast<uint32_t>(a_desc0);
        const uint32_t b_lo0 = static_cast<uint32_t>(b_desc0);
        const uint32_t a_kstep = a_mn ? ((32 * 128) >> 4) : (32 >> 4);
        const uint32_t b_kstep = b_mn ? ((32 * 128) >> 4) : (32 >> 4);
        const uint32_t bar0 = tc::smem_u32(bars);
        // Everything the loop needs is precomputed and every counter is a 32-bit increment: this thread's own
        // instructions are part of what is measured, and a single thread retires one every few clocks.
        // one accumulator: every instruction adds to the result of the one before it (alternating between two
        // accumulator stages per batch, as a matmul's successive tiles do); several: successive instructions add
        // to different accumulators, so none waits for its predecessor's result
        const uint32_t acc_stride = 512u / static_cast<uint32_t>(accumulators);
        uint32_t d_of_k[PROBE_KSTEPS];
#pragma unroll
        for (int k = 0; k < PROBE_KSTEPS; ++k) {
            d_of_k[k] = tmem_base + static_cast<uint32_t>(k % accumulators) * acc_stride;
        }
        const uint32_t groups = static_cast<uint32_t>(per_commit / PROBE_KSTEPS);
        constexpr uint32_t STAGE_STEP = PROBE_STAGE_BYTES >> 4;
        bool ok = true;
        uint32_t slot = 0, round = 0, stage = 0;
        for (long long b = 0; ok && b < batches; ++b) {
            if (round != 0) {
                // pattern 3: the wait a matmul's issuing thread makes on a barrier other CTAs' copies complete
                bool got;
                if (pattern == 3) {
                    got = tc::mbar_wait_cluster(bar0 + 8u * slot, (round - 1u) & 1u, abort_flag);
                } else if (pattern == 4) {
                    // a few non-blocking tests first, the blocking bounded wait only if the phase is really open
                    got = false;
#pragma unroll 1
                    for (int spin = 0; spin < 16 && !got; ++spin) {
                        got = tc::mbar_test_wait(bar0 + 8u * slot, (round - 1u) & 1u);
                    }
                    if (!got) {
                        got = tc::mbar_wait(bar0 + 8u * slot, (round - 1u) & 1u, abort_flag);
                    }
                } else {
                    got = tc::mbar_wait(bar0 + 8u * slot, (round - 1u) & 1u, abort_flag);
                }
                if (!got) {
                    ok = false;
                    break;
                }
                if (pattern == 1) {  // a second wait, on a phase that is certainly over
                    (void)tc::mbar_wait(bar0 + 8u * slot, (round - 1u) & 1u, abort_flag);
                }
                if (pattern == 3) {
                    tc::tc_fence_after_sync();
                }
            }
            const uint32_t d_flip = (accumulators == 1) ? static_cast<uint32_t>(b & 1) * 256u : 0u;
#pragma unroll 1
            for (uint32_t g = 0; g < groups; ++g) {
                const uint32_t a_lo = a_lo0 + stage * STAGE_STEP;
                const uint32_t b_lo = b_lo0 + stage * STAGE_STEP;
#pragma unroll
                for (int k = 0; k < PROBE_KSTEPS; ++k) {
                    tc::mma_lohi<CG, true>(d_of_k[k] + d_flip, a_lo + k * a_kstep, a_hi, b_lo + k * b_kstep, b_hi,
                                           idesc, 1u);
                }
                stage = (stage + 1u) & (PROBE_STAGES - 1);
                if (pattern == 2 && g + 1 < groups) {  // an extra commit after every four instructions, never waited for
                    if constexpr (CG == 2) {
                        tc::tc_commit_pair(bar0 + 8u * PROBE_MAX_DEPTH);
                    } else {
                        tc::tc_commit(bar0 + 8u * PROBE_MAX_DEPTH);
                    }
                }
            }
            if constexpr (CG == 2) {
                tc::tc_commit_pair(bar0 + 8u * slot);
            } else {
                tc::tc_commit(bar0 + 8u * slot);
            }
            if (++slot == static_cast<uint32_t>(depth)) {
                slot = 0;
                ++round;
            }
        }
        // drain: every slot's last commit
        if (ok) {
            const long long last_round_batches = batches - static_cast<long long>(round) * depth;  // in slots [0, that)
            for (uint32_t sl = 0; ok && sl < static_cast<uint32_t>(depth); ++sl) {
                long long completions = static_cast<long long>(round) + (static_cast<long long>(sl) < last_round_batches ? 1 : 0);
                if (completions == 0) {
                    continue;
                }
                if (!tc::mbar_wait(bar0 + 8u * sl, static_cast<uint32_t>((completions - 1) & 1), abort_flag)) {
                    ok = false;
                }
            }
        }
        if (!ok && error != nullptr) {
            atomicExch(error, 2);
        }
    }
    tc::tc_fence_before_sync();
    __syncthreads();
    if constexpr (CG == 2) {
        tc::cluster_arrive();
        tc::cluster_wait();
    }
    if (warp == 0) {
        tc::tc_fence_after_sync();
        tc::tmem_dealloc(tmem_base, 512);
    }
}

__global__ void bounded_wait_selftest_kernel(long long limit_cycles, int32_t* error)
{
    __shared__ uint64_t bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        tc::mbar_init(tc::smem_u32(&bar), 1);
        abort_flag = 0;
        tc::fence_mbar_init();
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        // nothing ever arrives on this barrier: the wait has to give up by itself
        const bool done = tc::mbar_wait(tc::smem_u32(&bar), 0u, &abort_flag, limit_cycles);
        if (!done) {
            atomicExch(error, 2);
        }
    }
    __syncthreads();
    // every other thread sees what the matmul kernels' roles see: the CTA-wide abort flag
    if (threadIdx.x == 1 && abort_flag != 0) {
        atomicAdd(error + 1, 1);
    }
}

}  // namespace w8a8

using namespace w8a8;

extern "C" int w8a8_mma_issue_probe(int cta_group, int umma_m, int umma_n, int a_mn_major, int b_mn_major, int fill,
                                    int accumulators, int per_commit, int depth, int pattern, int64_t batches,
                                    int32_t* error_word, void* stream)
{
    if (pattern < 0 || pattern > 4) {
        return W8A8_ERR_INVALID;
    }
    if (per_commit < PROBE_KSTEPS || per_commit > 256 || (per_commit % PROBE_KSTEPS) != 0 || depth < 1 ||
        depth > PROBE_MAX_DEPTH) {
        return W8A8_ERR_INVALID;
    }
    if (batches <= 0 || batches > (int64_t(1) << 24)) {
        return W8A8_ERR_INVALID;
    }
    if ((accumulators != 1 && accumulators != 2 && accumulators != 4) || umma_n * accumulators > 512) {
        return W8A8_ERR_INVALID;
    }
    if (cta_group == 1) {
        if (umma_m != 64 && umma_m != 128) {
            return W8A8_ERR_INVALID;
        }
    } else if (cta_group == 2) {
        if (umma_m != 128 && umma_m != 256) {
            return W8A8_ERR_INVALID;
        }
    } else {
        return W8A8_ERR_INVALID;
    }
    const int n_step = (umma_m == 64) ? 8 : 16;
    if (umma_n < n_step || umma_n > 256 || (umma_n % n_step) != 0) {
        return W8A8_ERR_INVALID;
    }
    const uint32_t idesc = tc::instr_desc(2u, 1u, b_mn_major ? 1u : 0u, static_cast<uint32_t>(umma_m),
                                          static_cast<uint32_t>(umma_n), a_mn_major ? 1u : 0u);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const size_t smem = static_cast<size_t>(PROBE_STAGES) * PROBE_STAGE_BYTES + 1024 + 256;
    const int sms = sm_count();
    cudaLaunchConfig_t cfg{};
    cfg.blockDim = dim3(PROBE_THREADS, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    cudaError_t e;
    if (cta_group == 2) {
        e = cudaFuncSetAttribute(mma_issue_probe_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 static_cast<int>(smem));
        if (e != cudaSuccess) {
            return W8A8_ERR_CUDA;
        }
        cfg.gridDim = dim3(static_cast<unsigned>(sms / 2 * 2), 1, 1);
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        e = cudaLaunchKernelEx(&cfg, mma_issue_probe_kernel<2>, idesc, a_mn_major, b_mn_major, fill,
                               accumulators, per_commit, depth, pattern, static_cast<long long>(batches), error_word);
    } else {
        e = cudaFuncSetAttribute(mma_issue_probe_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 static_cast<int>(smem));
        if (e != cudaSuccess) {
            return W8A8_ERR_CUDA;
        }
        cfg.gridDim = dim3(static_cast<unsigned>(sms), 1, 1);
        e = cudaLaunchKernelEx(&cfg, mma_issue_probe_kernel<1>, idesc, a_mn_major, b_mn_major, fill,
                               accumulators, per_commit, depth, pattern, static_cast<long long>(batches), error_word);
    }
    note_launch();
    return (e == cudaSuccess) ? W8A8_OK : W8A8_ERR_CUDA;
}

extern "C" int64_t w8a8_mma_issue_probe_ops(int cta_group, int umma_m, int umma_n, int per_commit, int64_t batches)
{
    // integer operations (multiply and add counted separately) one probe launch issues on this device
    const int64_t groups = (cta_group == 2) ? sm_count() / 2 : sm_count();
    return groups * batches * per_commit * 2 * umma_m * umma_n * 32;
}

namespace w8a8 {

// canonical_expf against its defining sequence on every fp32 bit pattern: counts the patterns whose results differ
// in any bit and keeps the smallest of them.
__global__ void __launch_bounds__(256) exp_selftest_kernel(unsigned long long* out)
{
    unsigned long long bad = 0, first = ~0ull;
    const unsigned long long stride = static_cast<unsigned long long>(gridDim.x) * blockDim.x;
    for (unsigned long long i = static_cast<unsigned long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < (1ull << 32);
         i += stride) {
        const float x = __uint_as_float(static_cast<uint32_t>(i));
        if (__float_as_uint(canonical_expf(x)) != __float_as_uint(canonical_expf_as_defined(x))) {
            ++bad;
            first = (i < first) ? i : first;
        }
    }
    if (bad != 0) {
        atomicAdd(out, bad);
        atomicMin(out + 1, first);
    }
}

}  // namespace w8a8

extern "C" int w8a8_selftest_exp(uint64_t* result, void* stream)
{
    if (result == nullptr) {
        return W8A8_ERR_INVALID;
    }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (cudaMemsetAsync(result, 0, 8, st) != cudaSuccess || cudaMemsetAsync(result + 1, 0xff, 8, st) != cudaSuccess) {
        return W8A8_ERR_CUDA;
    }
    w8a8::exp_selftest_kernel<<<w8a8::sm_count() * 8, 256, 0, st>>>(reinterpret_cast<unsigned long long*>(result));
    w8a8::note_launch();
    return (cudaGetLastError() == cudaSuccess) ? W8A8_OK : W8A8_ERR_CUDA;
}

namespace w8a8 {

// Reads `bytes` once with 16-byte streaming loads and nothing else: what one launch that only has to pull that
// many bytes out of HBM costs, as the yardstick for the weight-streaming matmul shapes.
__global__ void __launch_bounds__(256) stream_read_probe_kernel(const uint4* __restrict__ src, int64_t n16,
                                                                uint32_t* __restrict__ sink)
{
    uint32_t acc = 0;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    for (; i + 7 * stride < n16; i += 8 * stride) {
        uint4 v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            v[j] = __ldcs(src + i + j * stride);
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            acc ^= v[j].x ^ v[j].y ^ v[j].z ^ v[j].w;
        }
    }
    for (; i < n16; i += stride) {
        const uint4 v = __ldcs(src + i);
        acc ^= v.x ^ v.y ^ v.z ^ v.w;
    }
    if (acc == 0x9e3779b9u && sink != nullptr) {  // keeps the loads alive; practically never true
        *sink = acc;
    }
}

}  // namespace w8a8

extern "C" int w8a8_stream_read_probe(const void* src, int64_t bytes, void* sink, void* stream)
{
    if (src == nullptr || bytes < 0 || (bytes % 16) != 0 || !w8a8::is_aligned(src, 16)) {
        return W8A8_ERR_INVALID;
    }
    if (bytes == 0) {
        return W8A8_OK;
    }
    w8a8::stream_read_probe_kernel<<<w8a8::sm_count() * 8, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint4*>(src), bytes / 16, static_cast<uint32_t*>(sink));
    w8a8::note_launch();
    return (cudaGetLastError() == cudaSuccess) ? W8A8_OK : W8A8_ERR_CUDA;
}

extern "C" int w8a8_selftest_bounded_wait(int64_t limit_cycles, int32_t* error_words, void* stream)
{
    if (limit_cycles <= 0 || limit_cycles > 4000000000ll || error_words == nullptr) {
        return W8A8_ERR_INVALID;
    }
    bounded_wait_selftest_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<long long>(limit_cycles),
                                                                                  error_words); w8a8::note_launch();
    return (cudaGetLastError() == cudaSuccess) ? W8A8_OK : W8A8_ERR_CUDA;
}
