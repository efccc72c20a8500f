// qgru_rec_mma.cu - the persistent recurrence kernel on the tensor cores.
//
// One launch runs all T timesteps of one direction.  Replaces the reference's host loop of
// 2 launches per step (quantizedGemmBiasFused for R*h + br, then PointwiseOperationsQuant;
// src/gru_forward_gpu_quant.cu:565-668, 817-828), which re-reads R as int32 from memory every
// step and round-trips the R*h result through global memory.
//
// Work split: a CTA owns 128*MT hidden units (all three gates of each) of one group of NB batch
// rows.  Its slice of R (int8, K-major, 128-byte swizzle) is loaded once by TMA and stays in
// shared memory for all T steps.  Per step the group's h_{t-1} rows (8-bit) are TMA-loaded as
// the B operand and 3*MT accumulators D_g[unit][batch] = R_g * h^T are produced by
// tcgen05.mma kind::i8 into tensor memory.  TMEM lane = hidden unit, so epilogue thread j reads
// the three gate pre-activations of unit j for every batch column, requantizes them, applies
// the LUT gates and the state update in registers and stores h_t (8-bit state for the next
// step + the int32 / fp32 output).  CTAs of different groups never interact; the P CTAs of a
// group meet once per step at a counter in global memory (bounded spin).
//
// Warp roles: warp 0 = control (barrier wait, TMA, MMA issue), warps 1-16 = epilogue: four warps
// per TMEM lane quadrant, each taking 4-column chunks of the batch tile, so that every SM
// sub-partition has four warps to hide the latency of the 64-bit requantization chains.  The
// W*x+bw values and h_{t-1} of a chunk are fetched BEFORE the wait on the MMA, the gate
// constants sit in the kernel's constant bank (a __grid_constant__ parameter).
#include <cuda.h>
#include <cuda_runtime.h>

#include "qgru_device.cuh"
#include "qgru_rec_mma.cuh"
#include "qgru_tc.cuh"

namespace qgru {
namespace {

constexpr long long WAIT_BUDGET = 2000000000ll;  // ~1 s of SM clocks
constexpr int EPW = 4;                           // epilogue warps per TMEM lane quadrant
constexpr int EPI_THREADS = 32 * 4 * EPW;
constexpr int REC_THREADS = 32 + EPI_THREADS;
constexpr int CH = 4;                            // batch columns per chunk

__device__ __forceinline__ void fence_proxy_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }

struct Smem {
    // offsets from the 1024-aligned base
    size_t r_tiles, h_tile, bars, tables, total;
};

__host__ __device__ inline Smem smem_layout(int MT, int KBn, int NB, int n_table) {
    Smem s;
    s.r_tiles = 0;
    s.h_tile = (size_t)MT * 3 * KBn * 16384;
    s.bars = s.h_tile + (size_t)KBn * NB * 128;
    s.tables = s.bars + 64;
    s.total = s.tables + (((size_t)n_table * 4 + 15) & ~size_t(15));
    return s;
}

template <typename IhT, bool Narrow, bool Fused, int MT>
__global__ void __launch_bounds__(REC_THREADS, 1)
k_recurrence_mma(const __grid_constant__ CUtensorMap map_r, const __grid_constant__ CUtensorMap map_h,
                 const __grid_constant__ GateConsts gc, RecMmaArgs a) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char *base = reinterpret_cast<unsigned char *>(
        (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int KBn = a.Hpad >> 7;
    const Smem L = smem_layout(MT, KBn, a.NB, a.n_table);
    unsigned char *r_tiles = base + L.r_tiles;
    unsigned char *h_tile = base + L.h_tile;
    uint64_t *bars = reinterpret_cast<uint64_t *>(base + L.bars);
    uint64_t *r_full = bars, *h_full = bars + 1, *mma_done = bars + 2, *h_written = bars + 3;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 4);
    int *failed = reinterpret_cast<int *>(tmem_slot + 1);
    int32_t *tables = reinterpret_cast<int32_t *>(base + L.tables);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, tid = threadIdx.x;
    const int grp = blockIdx.x / a.P, p = blockIdx.x % a.P;
    const int j0 = p * 128 * MT;
    const int b0 = a.b_off + grp * a.NB;
    const int nb = min(a.NB, a.b_off + a.b_cnt - b0);
    unsigned *bar = a.bar + (size_t)(b0 / a.NB) * 32;
    const uint32_t tmem_cols = a.tmem_cols;

    for (int i = tid; i < a.n_table; i += blockDim.x) tables[i] = a.tables[i];
    if (tid == 0) {
        tc::mbar_init(r_full, 1);
        tc::mbar_init(h_full, 1);
        tc::mbar_init(mma_done, 1);
        tc::mbar_init(h_written, EPI_THREADS);
        *failed = 0;
        tc::fence_barrier_init();
        tc::tma_prefetch_desc(&map_r);
        tc::tma_prefetch_desc(&map_h);
    }
    if (warp == 0) tc::tmem_alloc(tmem_slot, tmem_cols);
    tc::tc_fence_before_sync();
    __syncthreads();
    tc::tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------------------------ control warp
        if (lane == 0) {
            bool ok = true;
            // the slice of R: MT x 3 gates x KBn slabs of [128 units x 128 bytes of K]
            tc::mbar_expect_tx(r_full, (uint32_t)(MT * 3 * KBn) * 16384u);
            for (int mt = 0; mt < MT; ++mt)
                for (int g = 0; g < 3; ++g)
                    for (int kb = 0; kb < KBn; ++kb)
                        tc::tma_load_2d(r_tiles + (size_t)((mt * 3 + g) * KBn + kb) * 16384, &map_r, r_full,
                                        kb * 128, g * a.H + j0 + mt * 128);
            ok = tc::mbar_wait(r_full, 0, WAIT_BUDGET);
            const uint32_t idesc = tc::idesc_i8(128, a.NB, true, !a.h_unsigned);
            const uint32_t h_bytes = (uint32_t)(KBn * a.NB * 128);
            const uint32_t r_lo0 = (tc::smem_u32(r_tiles) & 0x3FFFFu) >> 4;
            const uint32_t h_lo0 = (tc::smem_u32(h_tile) & 0x3FFFFu) >> 4;
            const uint32_t desc_hi = (uint32_t)(tc::smem_desc_sw128(0) >> 32);
            const uint32_t desc_lo = (uint32_t)tc::smem_desc_sw128(0);
            for (int s = 0; s < a.T && ok; ++s) {
                if (s > 0) {
                    // every epilogue thread of this CTA has stored its h_s values and fenced them
                    if (!tc::mbar_wait(h_written, (uint32_t)((s - 1) & 1), WAIT_BUDGET)) { ok = false; break; }
                    tc::tc_fence_after_sync();
                    if (a.P > 1) {
                        __threadfence();
                        atomicAdd(bar, 1u);
                        const unsigned want = (unsigned)a.P * (unsigned)s;
                        unsigned it = 0;
                        while (ld_acquire(bar) < want) {
                            if (++it > a.spin_limit || ((it & 1023u) == 0 && *(volatile int *)a.abort_flag)) {
                                ok = false;
                                break;
                            }
                        }
                        if (!ok) break;
                    }
                    fence_proxy_async_all();
                }
                // h_s rows of this group: KBn boxes of [NB rows x 128 bytes]
                tc::mbar_expect_tx(h_full, h_bytes);
                const int row = (s & 1) * a.B + b0;
                for (int kb = 0; kb < KBn; ++kb)
                    tc::tma_load_2d(h_tile + (size_t)kb * a.NB * 128, &map_h, h_full, kb * 128, row);
                if (!tc::mbar_wait(h_full, (uint32_t)(s & 1), WAIT_BUDGET)) { ok = false; break; }
                tc::tc_fence_after_sync();
                // Descriptors differ only in their 14-bit start-address field (bytes >> 4): the
                // high word and the LBO field are constants, so each MMA costs two adds.
                for (int mt = 0; mt < MT; ++mt)
                    for (int kb = 0; kb < KBn; ++kb) {
                        const uint32_t hb = h_lo0 + (uint32_t)(kb * a.NB * 8);
#pragma unroll
                        for (int g = 0; g < 3; ++g) {
                            const uint32_t d = tmem_base + (uint32_t)((mt * 3 + g) * a.NB);
                            const uint32_t rb = r_lo0 + (uint32_t)(((mt * 3 + g) * KBn + kb) * 1024);
#pragma unroll
                            for (int ks = 0; ks < 4; ++ks)
                                tc::mma_i8(d, ((uint64_t)desc_hi << 32) | (desc_lo | (rb + 2 * ks)),
                                           ((uint64_t)desc_hi << 32) | (desc_lo | (hb + 2 * ks)), idesc,
                                           (kb | ks) != 0);
                        }
                    }
                tc::mma_commit(mma_done);
            }
            if (!ok) {
                atomicExch(failed, 1);
                atomicOr(a.abort_flag, 1);
            }
        }
    } else {
        // ---------------------------------------------------------------- epilogue warps
        const int q = warp & 3;                      // TMEM lane quadrant this warp may read
        const int rank = (warp - 1) >> 2;            // 0..EPW-1 among the warps of that quadrant
        const int u = q * 32 + lane;                 // unit within a 128-unit tile = TMEM lane
        const size_t BH = (size_t)a.B * a.H;
        const IhT *ihp = reinterpret_cast<const IhT *>(a.ih);
        const int nchunks = a.NB / CH;
        int64_t corr[MT][3];
        Rescale rs[MT][3];
        bool j_ok[MT];
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
            const int j = j0 + mt * 128 + u;
            j_ok[mt] = j < a.H;
#pragma unroll
            for (int g = 0; g < 3; ++g) {
                corr[mt][g] = j_ok[mt] ? a.lc.corr[g * a.H + j] : 0;
                rs[mt][g] = j_ok[mt] ? a.lc.rs[g * a.H + j] : Rescale{1, 1, 0, 0, 0, 0, 0, 0};
            }
        }
        bool ok = true;
        for (int s = 0; s < a.T && ok; ++s) {
            const int t = a.reverse ? (a.T - 1 - s) : s;
            const long long out_slot = a.reverse ? (a.T - 1 - s) : (s + 1);
            const uint8_t *h_cur = a.h8 + (size_t)(s & 1) * a.B * a.Hpad;
            uint8_t *h_nxt = a.h8 + (size_t)((s + 1) & 1) * a.B * a.Hpad;
            bool waited = false;
            for (int c = rank; c < nchunks; c += EPW) {
                const int c0 = c * CH;
                // operands that do not depend on this step's MMA: issued first
                int32_t ihv[MT][CH][3];
                int32_t hold[MT][CH];
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
                    const int j = j0 + mt * 128 + u;
#pragma unroll
                    for (int i = 0; i < CH; ++i) {
                        const int b = c0 + i;
                        const bool v_ok = b < nb && j_ok[mt];
                        const size_t row = (size_t)t * a.B + b0 + b;
#pragma unroll
                        for (int g = 0; g < 3; ++g)
                            ihv[mt][i][g] = v_ok ? (int32_t)ihp[row * a.C + g * a.H + j] : 0;
                        const uint8_t hb = v_ok ? __ldcg(h_cur + (size_t)(b0 + b) * a.Hpad + j) : (uint8_t)0;
                        hold[mt][i] = a.h_unsigned ? (int32_t)hb : (int32_t)(int8_t)hb;
                    }
                }
                if (!waited) {
                    ok = tc::mbar_wait(mma_done, (uint32_t)(s & 1), WAIT_BUDGET);
                    if (!ok) break;
                    tc::tc_fence_after_sync();
                    waited = true;
                }
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
                    const int j = j0 + mt * 128 + u;
                    int32_t az[CH], ar[CH], an[CH];
                    const uint32_t ta = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(mt * 3 * a.NB + c0);
                    tc::tmem_ld4(ta, az);
                    tc::tmem_ld4(ta + a.NB, ar);
                    tc::tmem_ld4(ta + 2 * a.NB, an);
                    tc::tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < CH; ++i) {
                        const int b = c0 + i;
                        if (b >= nb || !j_ok[mt]) continue;
                        int32_t hh_z, hh_r, hh_n;
                        if (a.lc.fits32) {
                            hh_z = linear_epilogue32(az[i], (int32_t)corr[mt][0], rs[mt][0], a.lc.zp_out, a.lc.lo, a.lc.hi);
                            hh_r = linear_epilogue32(ar[i], (int32_t)corr[mt][1], rs[mt][1], a.lc.zp_out, a.lc.lo, a.lc.hi);
                            hh_n = linear_epilogue32(an[i], (int32_t)corr[mt][2], rs[mt][2], a.lc.zp_out, a.lc.lo, a.lc.hi);
                        } else {
                            hh_z = linear_epilogue(az[i], corr[mt][0], rs[mt][0], a.lc.zp_out, a.lc.lo, a.lc.hi);
                            hh_r = linear_epilogue(ar[i], corr[mt][1], rs[mt][1], a.lc.zp_out, a.lc.lo, a.lc.hi);
                            hh_n = linear_epilogue(an[i], corr[mt][2], rs[mt][2], a.lc.zp_out, a.lc.lo, a.lc.hi);
                        }
                        int32_t hn;
                        if constexpr (Fused)
                            hn = gru_cell_fused(gc, tables, ihv[mt][i][0], ihv[mt][i][1], ihv[mt][i][2], hh_z, hh_r,
                                                hh_n, hold[mt][i]);
                        else
                            hn = gru_cell<Narrow>(gc, tables, ihv[mt][i][0], ihv[mt][i][1], ihv[mt][i][2], hh_z,
                                                  hh_r, hh_n, hold[mt][i]);
                        h_nxt[(size_t)(b0 + b) * a.Hpad + j] = (uint8_t)hn;
                        const size_t o = (size_t)out_slot * BH + (size_t)(b0 + b) * a.H + j;
                        if (a.hq_out) a.hq_out[o] = hn;
                        if (a.hf_out) a.hf_out[o] = (float)(hn - gc.zp_h) * gc.h_scale;
                        if (a.h8_out) a.h8_out[o] = (uint8_t)hn;
                    }
                }
            }
            if (!ok) break;
            if (!waited) {   // a warp without a chunk still follows the phase of the MMA barrier
                ok = tc::mbar_wait(mma_done, (uint32_t)(s & 1), WAIT_BUDGET);
                if (!ok) break;
                tc::tc_fence_after_sync();
            }
            // publish h_{s+1}: order the generic-proxy stores before the async-proxy (TMA) reads.
            // The gpu-scope fence that makes them visible to the other CTAs of the group is
            // executed once, by the control thread, after it has observed every arrival below.
            fence_proxy_async_all();
            tc::tc_fence_before_sync();
            tc::mbar_arrive(h_written);
        }
        if (!ok && lane == 0) {
            atomicExch(failed, 1);
            atomicOr(a.abort_flag, 1);
        }
    }
    tc::tc_fence_before_sync();
    __syncthreads();
    if (warp == 0) tc::tmem_dealloc(tmem_base, tmem_cols);
}

template <typename IhT, bool Narrow, bool Fused, int MT>
cudaError_t launch_one(const CUtensorMap &mr, const CUtensorMap &mh, const GateConsts &gc, RecMmaArgs &a,
                       int grid, size_t smem, bool cooperative, cudaStream_t st) {
    auto kern = k_recurrence_mma<IhT, Narrow, Fused, MT>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    if (cooperative) {
        void *args[] = {(void *)&mr, (void *)&mh, (void *)&gc, (void *)&a};
        return cudaLaunchCooperativeKernel((void *)kern, dim3(grid), dim3(REC_THREADS), args, smem, st);
    }
    kern<<<grid, REC_THREADS, smem, st>>>(mr, mh, gc, a);
    return cudaGetLastError();
}

template <typename IhT, bool Narrow, bool Fused>
cudaError_t launch_mt(int MT, const CUtensorMap &mr, const CUtensorMap &mh, const GateConsts &gc,
                      RecMmaArgs &a, int grid, size_t smem, bool coop, cudaStream_t st) {
    return MT == 2 ? launch_one<IhT, Narrow, Fused, 2>(mr, mh, gc, a, grid, smem, coop, st)
                   : launch_one<IhT, Narrow, Fused, 1>(mr, mh, gc, a, grid, smem, coop, st);
}

// fused: pre-rescaled W*x+bw as int16 / int32; otherwise raw int8 / int16 with the generic cell
cudaError_t launch_any(bool fused, bool narrow, int ih_bytes, int MT, const CUtensorMap &mr,
                       const CUtensorMap &mh, const GateConsts &gc, RecMmaArgs &a, int grid, size_t smem,
                       bool coop, cudaStream_t st) {
    if (fused)
        return ih_bytes == 2 ? launch_mt<int16_t, false, true>(MT, mr, mh, gc, a, grid, smem, coop, st)
                             : launch_mt<int32_t, false, true>(MT, mr, mh, gc, a, grid, smem, coop, st);
    if (ih_bytes == 1)
        return narrow ? launch_mt<int8_t, true, false>(MT, mr, mh, gc, a, grid, smem, coop, st)
                      : launch_mt<int8_t, false, false>(MT, mr, mh, gc, a, grid, smem, coop, st);
    return narrow ? launch_mt<int16_t, true, false>(MT, mr, mh, gc, a, grid, smem, coop, st)
                  : launch_mt<int16_t, false, false>(MT, mr, mh, gc, a, grid, smem, coop, st);
}

}  // namespace

bool rec_mma_plan(int H, int Hpad, int B, int sms, int smem_optin, int n_table, RecMmaPlan *out) {
    if (Hpad > 512) return false;                  // the R slice of 128 units must fit one SM
    const int KBn = Hpad / 128;
    const int MT = (H > 128 && H <= 256) ? 2 : 1;
    const int P = (H + 128 * MT - 1) / (128 * MT);
    if (P > sms) return false;
    const int groups_max = std::max(1, sms / P);
    int NB = ((B + groups_max - 1) / groups_max + 15) / 16 * 16;
    const int nb_cap = MT == 2 ? 64 : 128;         // 3*MT*NB accumulator columns <= 512
    NB = std::min(NB, nb_cap);
    while (NB > 16 && smem_layout(MT, KBn, NB, n_table).total + 1024 > (size_t)smem_optin) NB -= 16;
    const size_t smem = smem_layout(MT, KBn, NB, n_table).total + 1024;
    if (smem > (size_t)smem_optin) return false;
    uint32_t cols = 32;
    while ((int)cols < 3 * MT * NB) cols <<= 1;
    out->MT = MT;
    out->P = P;
    out->NB = NB;
    out->G = (B + NB - 1) / NB;
    out->smem = smem;
    out->tmem_cols = (int)cols;
    // groups that cannot be co-resident run as further launches over the remaining batch rows
    out->groups_per_launch = P > 1 ? std::min(out->G, groups_max) : out->G;
    return true;
}

int rec_mma_launch(RecMmaState &s, const RecMmaPlan &pl, RecMmaArgs a, const GateConsts &gc_host,
                   const int8_t *r8, long long r_rows_alloc,
                   long long h_rows_alloc, bool h_unsigned, int ih_bytes, bool narrow, bool fused, bool have_coop,
                   cudaStream_t stream, std::string *err) {
    if (!s.valid || s.r8 != r8 || s.h8 != a.h8 || s.r_rows != r_rows_alloc || s.h_rows != h_rows_alloc ||
        s.Hpad != a.Hpad || s.NB != pl.NB) {
        if (!make_map_u8_sw128(reinterpret_cast<CUtensorMap *>(s.map_r), r8, (uint64_t)r_rows_alloc, (uint64_t)a.Hpad, 128) ||
            !make_map_u8_sw128(reinterpret_cast<CUtensorMap *>(s.map_h), a.h8, (uint64_t)h_rows_alloc, (uint64_t)a.Hpad, (uint32_t)pl.NB)) {
            if (err) *err = "cuTensorMapEncodeTiled failed";
            return QGRU_ERR_CUDA;
        }
        s.valid = true;
        s.r8 = r8;
        s.h8 = a.h8;
        s.r_rows = r_rows_alloc;
        s.h_rows = h_rows_alloc;
        s.Hpad = a.Hpad;
        s.NB = pl.NB;
    }
    if (pl.P > 1 && !have_coop) {
        if (err) *err = "device lacks cooperative launch";
        return QGRU_ERR_UNSUPPORTED;
    }
    const CUtensorMap &mr = *reinterpret_cast<const CUtensorMap *>(s.map_r);
    const CUtensorMap &mh = *reinterpret_cast<const CUtensorMap *>(s.map_h);
    a.P = pl.P;
    a.NB = pl.NB;
    a.h_unsigned = h_unsigned ? 1 : 0;
    a.tmem_cols = (uint32_t)pl.tmem_cols;
    // Groups that cannot all be resident at once run as consecutive launches over batch ranges.
    for (int g0 = 0; g0 < pl.G; g0 += pl.groups_per_launch) {
        const int groups = std::min(pl.groups_per_launch, pl.G - g0);
        a.b_off = g0 * pl.NB;
        a.b_cnt = std::min(a.B - a.b_off, groups * pl.NB);
        const int grid = groups * pl.P;
        const cudaError_t e = launch_any(fused, narrow, ih_bytes, pl.MT, mr, mh, gc_host, a, grid, pl.smem,
                                         pl.P > 1, stream);
        if (e != cudaSuccess) {
            if (err) *err = std::string("recurrence (tcgen05) launch: ") + cudaGetErrorString(e);
            return QGRU_ERR_CUDA;
        }
        ++s.launches;
    }
    return QGRU_OK;
}

}  // namespace qgru
