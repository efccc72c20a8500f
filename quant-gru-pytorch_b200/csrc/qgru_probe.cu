// qgru_probe.cu - measurement aids of the library: the issue rate of tcgen05.mma kind::i8.
//
// qgru_probe_mma_i8 runs, on a given number of CTAs (one per SM), a chain of back-to-back
// tcgen05.mma.cta_group::1.kind::i8 instructions of one shape (M x N x 32) on operands that
// already sit in shared / tensor memory: no loads, no epilogue.  What it returns is the rate the
// tensor pipe itself sustains for that shape - the denominator the W*x GEMM's "tensor pipe
// busy" figure is quoted against (large N), and the cost model of the recurrence kernels, whose
// MMAs have few batch columns (small N).  The reference has no tensor-core code and no
// counterpart of this file.
#include <cuda_runtime.h>

#include <algorithm>
#include <vector>

#include "qgru.h"
#include "qgru_tc.cuh"

namespace qgru {
namespace {

constexpr long long PROBE_WAIT = 2000000000ll;

// `issuers` warps (lane 0 of each) issue `mmas` MMAs each, every warp into accumulators of its own
// (n_acc per warp), K-step i % 4 of a 128-byte slab.  A: 128 rows x 128 bytes (shared memory,
// 128-byte swizzle, or 32 columns of tensor memory); B: N rows x 128 bytes in shared memory.  The
// operands are zeros: an integer pipe does not care.  `spinners` further warps poll an mbarrier
// the way the recurrence kernels' waiting warps do, until the issuers are done: they show what
// waiting neighbours cost the issuing threads.  cycles[cta] = clock ticks from the first issue to
// the completion of the last MMA of the slowest issuer.
__global__ void __launch_bounds__(1024, 1)
k_probe_mma_i8(int M, int N, int a_in_tmem, int n_acc, int mmas, int issuers, int neighbour_mode, int commit_every,
               long long *cycles, int *timeouts, const unsigned char *src) {
    extern __shared__ unsigned char smem_raw[];
    const uint32_t raw = tc::smem_u32(smem_raw);
    unsigned char *base = smem_raw + (((raw + 1023u) & ~1023u) - raw);
    unsigned char *a_tile = base;                    // 16 KB
    unsigned char *b_tile = base + 16384;            // up to 32 KB
    uint64_t *bar = reinterpret_cast<uint64_t *>(base + 16384 + 32768);   // [issuers] + one nobody completes
    uint32_t *slot = reinterpret_cast<uint32_t *>(bar + 10);
    volatile int *done = reinterpret_cast<volatile int *>(slot + 1);
    long long *cyc_w = reinterpret_cast<long long *>(bar + 12);           // [issuers]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // operand bytes: zeros, or (neighbour_mode bit 8) pseudo-random, which is what a real product
    // toggles in the multipliers - the two differ in power, not in the instruction stream
    const bool random_fill = (neighbour_mode & 256) != 0;
    // bit 9: the issuing warps keep all 32 lanes in the loop and one elected lane issues, so that the
    // control flow around the MMAs is warp-uniform and their operands can live in uniform registers
    const bool uniform_flow = (neighbour_mode & 512) != 0;
    // bit 10: every MMA of a pass reads operand tiles of its own (eight A and eight B tiles spread over
    // 128 KB of shared memory), as a GEMM that streams its operands does; without it the four K
    // steps of one 16 KB tile pair repeat
    const bool rotate = (neighbour_mode & 1024) != 0;
    neighbour_mode &= 255;
    for (int i = threadIdx.x; i < (16384 + 32768) / 4; i += blockDim.x)
        reinterpret_cast<uint32_t *>(base)[i] = random_fill ? ((uint32_t)i * 2654435761u) ^ ((uint32_t)i * 40503u << 13) ^ (blockIdx.x * 97u) : 0u;
    if (threadIdx.x == 0) {
        for (int i = 0; i < 10; ++i) tc::mbar_init(&bar[i], 1);   // 0-3 chain ends, 4 never completes, 5-8 periodic commits, 9 bulk copies
        *done = 0;
        tc::fence_barrier_init();
    }
    if (warp == 0) tc::tmem_alloc(slot, 512);
    tc::tc_fence_before_sync();
    __syncthreads();
    tc::tc_fence_after_sync();
    const uint32_t tmem = *slot;
    if (warp < issuers && uniform_flow) {
        uint32_t leader;
        asm volatile(
            "{\n"
            ".reg .pred p;\n"
            "elect.sync _|p, 0xffffffff;\n"
            "selp.u32 %0, 1, 0, p;\n"
            "}\n"
            : "=r"(leader));
        const uint32_t idesc = tc::idesc_i8(M, N, true, true);
        const uint32_t a_lo = tc::smem_desc_sw128_lo(tc::smem_u32(a_tile));
        const uint32_t b_lo = tc::smem_desc_sw128_lo(tc::smem_u32(b_tile));
        const uint32_t a_col = tmem + (uint32_t)(issuers * n_acc * N);
        const uint32_t d0 = tmem + (uint32_t)(warp * n_acc * N);
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        const int passes = mmas / 8;
        const long long t0 = clock64();
        uint32_t acc = 0;   // accumulator rotation, advanced in the loop like a GEMM's ring position
        for (int i = 0; i < passes; ++i) {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const uint32_t d = d0 + acc * (uint32_t)N;
                if (leader) {
                    if (a_in_tmem) tc::mma_i8_ts_lo(d, a_col + (uint32_t)(j & 3) * 8, b_lo + 2 * (uint32_t)(j & 3), idesc, 1u);
                    else tc::mma_i8_lo(d, a_lo + 2 * (uint32_t)(j & 3), b_lo + 2 * (uint32_t)(j & 3), idesc, 1u);
                }
                if (++acc == (uint32_t)n_acc) acc = 0;
                if (commit_every == 4 && j == 3 && leader) tc::mma_commit(&bar[5 + warp]);
            }
            if ((commit_every == 4 || commit_every == 8) && leader) tc::mma_commit(&bar[5 + warp]);
        }
        if (leader) tc::mma_commit(&bar[warp]);
        const bool ok = tc::mbar_wait(&bar[warp], 0, PROBE_WAIT);
        const long long t1 = clock64();
        if (lane == 0) {
            cyc_w[warp] = t1 - t0;
            if (!ok) atomicAdd(timeouts, 1);
            __threadfence_block();
            atomicAdd(const_cast<int *>(done), 1);
        }
    } else if (warp < issuers) {
        if (lane == 0) {
            const uint32_t idesc = tc::idesc_i8(M, N, true, true);
            const uint64_t adesc = tc::smem_desc_sw128(tc::smem_u32(a_tile));
            const uint64_t bdesc = tc::smem_desc_sw128(tc::smem_u32(b_tile));
            const uint32_t a_col = tmem + (uint32_t)(issuers * n_acc * N);   // 32 columns after the accumulators
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            // Every operand of the 8 MMAs of a loop pass is prepared before the clock starts, so that the
            // issuing thread's own arithmetic does not set the pace: the body is 8 MMA instructions.
            uint32_t dcol[8], acol[8];
            uint64_t ad[8], bd[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                dcol[j] = tmem + (uint32_t)((warp * n_acc + j % n_acc) * N);
                acol[j] = a_col + (uint32_t)(j & 3) * 8;
                ad[j] = adesc + 2 * (uint64_t)(j & 3);
                bd[j] = bdesc + 2 * (uint64_t)(j & 3);
                if (rotate) {
                    // tile j of A at base + 16 KB * j (j < 4) and of B behind them: (16384 >> 4) descriptor units apart
                    ad[j] = tc::smem_desc_sw128(tc::smem_u32(base) + (uint32_t)(j & 3) * 16384u) + 2 * (uint64_t)(j >> 2);
                    bd[j] = tc::smem_desc_sw128(tc::smem_u32(base) + 65536u + (uint32_t)(j & 3) * 16384u) + 2 * (uint64_t)(j >> 2);
                }
            }
            const int passes = mmas / 8;
            const long long t0 = clock64();
            // commit_every = 4 or 8: a tcgen05.commit after every 4 / 8 MMAs, as a GEMM main loop does to hand
            // its shared-memory stages back (the barrier it arrives on is nobody's concern here)
            if (a_in_tmem) {
                for (int i = 0; i < passes; ++i) {
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        tc::mma_i8_ts(dcol[j], acol[j], bd[j], idesc, 1u);
                        if (commit_every == 4 && j == 3) tc::mma_commit(&bar[5 + warp]);
                    }
                    if (commit_every == 4 || commit_every == 8) tc::mma_commit(&bar[5 + warp]);
                }
            } else {
                for (int i = 0; i < passes; ++i) {
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        tc::mma_i8(dcol[j], ad[j], bd[j], idesc, 1u);
                        if (commit_every == 4 && j == 3) tc::mma_commit(&bar[5 + warp]);
                    }
                    if (commit_every == 4 || commit_every == 8) tc::mma_commit(&bar[5 + warp]);
                }
            }
            tc::mma_commit(&bar[warp]);
            const bool ok = tc::mbar_wait(&bar[warp], 0, PROBE_WAIT);
            const long long t1 = clock64();
            cyc_w[warp] = t1 - t0;
            if (!ok) atomicAdd(timeouts, 1);
            __threadfence_block();
            atomicAdd(const_cast<int *>(done), 1);
        }
    } else {
        // a neighbour warp, until the issuers are done (bounded): mode 0 polls a barrier that stays incomplete
        // (a waiting warp), mode 1 runs dependent integer arithmetic back to back (a busy warp), mode 2
        // runs dependent shared-memory loads (a warp doing table lookups)
        const long long t0 = clock64();
        uint32_t x = threadIdx.x;
        const uint32_t tb = tc::smem_u32(base);
        uint32_t bulk_phase = 0;
        long long bulk_rounds = 0;
        while (*done < issuers && clock64() - t0 < PROBE_WAIT) {
            if (neighbour_mode == 5) {
                // the copy engine writing shared memory as a GEMM's operand loads do: the first
                // neighbour warp keeps four 16 KB bulk copies from global memory in flight
                if (warp == issuers && lane == 0) {
                    tc::mbar_expect_tx(&bar[9], 65536u);
                    for (int i = 0; i < 4; ++i)
                        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::
                                     "r"(tb + 49152u + 4096u + (uint32_t)i * 16384u), "l"(src + (size_t)blockIdx.x * 65536 + (size_t)i * 16384),
                                     "r"(16384u), "r"(tc::smem_u32(&bar[9])) : "memory");
                    if (!tc::mbar_wait(&bar[9], bulk_phase, PROBE_WAIT)) atomicAdd(timeouts, 1);
                    bulk_phase ^= 1u;
                    ++bulk_rounds;
                } else {
                    tc::mbar_try_wait(&bar[4], 0);
                }
            } else if (neighbour_mode == 7) {
                // warps streaming global memory (read, add, write back) over 2 MB per CTA: DRAM and L2 busy
                // beside the tensor pipe, as in a GEMM whose operands and results move through HBM
                uint4 *gp = reinterpret_cast<uint4 *>(const_cast<unsigned char *>(src)) + (size_t)blockIdx.x * 131072;
                const uint32_t at = (x * 32u + (uint32_t)lane + (uint32_t)(warp - issuers) * 8192u) & 131071u;
                uint4 v = gp[at];
                v.x += 1u;
                gp[at] = v;
                x += 1u;
            } else if (neighbour_mode == 6) {
                // warps that follow the issuer's periodic commits as a GEMM's epilogue follows its accumulator
                // barrier: a suspending wait on the phase that the next commit completes (never blocking
                // for good: the loop condition ends it)
                if (tc::mbar_try_wait(&bar[5], bulk_phase)) bulk_phase ^= 1u;
            } else if (neighbour_mode == 0) {
                tc::mbar_try_wait(&bar[4], 0);
            } else if (neighbour_mode == 1) {
#pragma unroll
                for (int i = 0; i < 64; ++i) x = x * 1664525u + 1013904223u;
            } else if (neighbour_mode == 2) {
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    uint32_t v;
                    asm volatile("ld.shared.b32 %0, [%1];" : "=r"(v) : "r"(tb + ((x & 4095u) << 2)));
                    x = x * 1664525u + 1013904223u + v;
                }
            } else if (neighbour_mode == 3) {
                // a warp draining accumulators: 16-column loads from its quadrant of tensor memory
                int32_t v[16];
                tc::tmem_ld16(tmem + ((uint32_t)((warp & 3) * 32) << 16), v);
                tc::tmem_ld_wait();
                x += (uint32_t)v[0];
            } else {
                // a warp writing 128-bit words into the operand tiles' neighbourhood of shared memory
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(tb + 49152u + 4096u + ((threadIdx.x * 16u + i * 16384u) & 65535u)), "r"(0u) : "memory");
                }
            }
        }
        if (x == 0xdeadbeefu) atomicAdd(timeouts, 0);   // keeps the arithmetic alive
        if (neighbour_mode == 5 && warp == issuers && lane == 0) cycles[gridDim.x + blockIdx.x] = bulk_rounds * 65536;
    }
    tc::tc_fence_before_sync();
    __syncthreads();
    if (threadIdx.x == 0) {
        long long worst = 0;
        for (int i = 0; i < issuers; ++i) worst = worst > cyc_w[i] ? worst : cyc_w[i];
        cycles[blockIdx.x] = worst;
    }
    if (warp == 0) tc::tmem_dealloc(tmem, 512);
}

}  // namespace
}  // namespace qgru

static double g_probe_bulk_bytes_per_cycle = 0.0;
/* bytes per SM clock the copy engine moved into CTA 0's shared memory during the last probe with neighbour_mode 5 */
extern "C" QGRU_API double qgru_probe_last_bulk_rate(void) { return g_probe_bulk_bytes_per_cycle; }

extern "C" int qgru_probe_mma_i8_ex(int device, int M, int N, int a_in_tmem, int accumulators, int mmas, int ctas,
                                    int issuers, int spinners, int neighbour_mode, double *cycles_per_mma,
                                    double *tera_ops) {
    return qgru_probe_mma_i8_commits(device, M, N, a_in_tmem, accumulators, mmas, ctas, issuers, spinners, neighbour_mode,
                                     0, cycles_per_mma, tera_ops);
}

extern "C" int qgru_probe_mma_i8_commits(int device, int M, int N, int a_in_tmem, int accumulators, int mmas, int ctas,
                                         int issuers, int spinners, int neighbour_mode, int commit_every,
                                         double *cycles_per_mma, double *tera_ops) {
    using namespace qgru;
    if (!cycles_per_mma || !tera_ops) return QGRU_ERR_BAD_ARG;
    if (!((M == 128 && N % 16 == 0) || (M == 64 && N % 8 == 0)) || N < 8 || N > 256) return QGRU_ERR_BAD_ARG;
    if (issuers < 1 || issuers > 4 || spinners < 0 || issuers + spinners > 32) return QGRU_ERR_BAD_ARG;
    // the rotating operand tiles are 16 KB apart: rows of at most 128 tokens
    if ((neighbour_mode & 1024) != 0 && N > 128) return QGRU_ERR_BAD_ARG;
    if ((neighbour_mode & 255) == 5 && spinners < 1) return QGRU_ERR_BAD_ARG;
    if (accumulators < 1 || issuers * accumulators * N + (a_in_tmem ? 32 : 0) > 512 || mmas < 8 || mmas % 8 != 0 || mmas > (1 << 22) || ctas < 1)
        return QGRU_ERR_BAD_ARG;
    if (cudaSetDevice(device) != cudaSuccess) return QGRU_ERR_CUDA;
    int sms = 0;
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    ctas = std::min(ctas, sms);
    long long *d_cycles = nullptr;
    int *d_to = nullptr;
    unsigned char *d_src = nullptr;
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    int rc = QGRU_ERR_CUDA;
    const size_t smem = 16384 + 32768 + 4096 + 65536 + 16384 + 1024;
    const int threads = 32 * (issuers + spinners);
    do {
        if (cudaMalloc(&d_cycles, sizeof(long long) * ctas * 2) != cudaSuccess) break;
        if (cudaMemset(d_cycles, 0, sizeof(long long) * ctas * 2) != cudaSuccess) break;
        if ((neighbour_mode & 255) == 5 && (cudaMalloc(&d_src, (size_t)ctas * 65536) != cudaSuccess || cudaMemset(d_src, 1, (size_t)ctas * 65536) != cudaSuccess)) break;
        if ((neighbour_mode & 255) == 7 && (cudaMalloc(&d_src, (size_t)ctas * 2097152) != cudaSuccess || cudaMemset(d_src, 1, (size_t)ctas * 2097152) != cudaSuccess)) break;
        if (cudaMalloc(&d_to, sizeof(int)) != cudaSuccess) break;
        if (cudaMemset(d_to, 0, sizeof(int)) != cudaSuccess) break;
        if (cudaFuncSetAttribute(k_probe_mma_i8, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) break;
        if (cudaEventCreate(&e0) != cudaSuccess || cudaEventCreate(&e1) != cudaSuccess) break;
        k_probe_mma_i8<<<ctas, threads, smem>>>(M, N, a_in_tmem, accumulators, std::min(mmas, 256) / 8 * 8, issuers, neighbour_mode, commit_every, d_cycles, d_to, d_src);   // warm-up
        cudaEventRecord(e0);
        k_probe_mma_i8<<<ctas, threads, smem>>>(M, N, a_in_tmem, accumulators, mmas, issuers, neighbour_mode, commit_every, d_cycles, d_to, d_src);
        cudaEventRecord(e1);
        if (cudaEventSynchronize(e1) != cudaSuccess || cudaGetLastError() != cudaSuccess) break;
        float ms = 0.f;
        cudaEventElapsedTime(&ms, e0, e1);
        std::vector<long long> cyc(ctas * 2);
        int to = 0;
        if (cudaMemcpy(cyc.data(), d_cycles, sizeof(long long) * ctas * 2, cudaMemcpyDeviceToHost) != cudaSuccess) break;
        if (cudaMemcpy(&to, d_to, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) break;
        if (to) {
            rc = QGRU_ERR_TIMEOUT;
            break;
        }
        long long worst = 0;
        for (int i = 0; i < ctas; ++i) worst = std::max(worst, cyc[i]);
        g_probe_bulk_bytes_per_cycle = worst > 0 ? (double)cyc[ctas] / (double)worst : 0.0;
        *cycles_per_mma = (double)worst / mmas;
        *tera_ops = 2.0 * M * N * 32.0 * (double)mmas * issuers * ctas / (ms * 1e-3) / 1e12;
        rc = QGRU_OK;
    } while (false);
    cudaGetLastError();
    if (e0) cudaEventDestroy(e0);
    if (e1) cudaEventDestroy(e1);
    cudaFree(d_cycles);
    cudaFree(d_to);
    cudaFree(d_src);
    return rc;
}

extern "C" int qgru_probe_mma_i8(int device, int M, int N, int a_in_tmem, int accumulators, int mmas, int ctas,
                                 double *cycles_per_mma, double *tera_ops) {
    return qgru_probe_mma_i8_ex(device, M, N, a_in_tmem, accumulators, mmas, ctas, 1, 3, 0, cycles_per_mma, tera_ops);
}
