// qgru_gemm_tc.cu - the input projection W*x + bw for all timesteps as one int8 tensor-core
// GEMM (tcgen05.mma kind::i8, TMA-fed, int32 accumulators in tensor memory) with the
// zero-point / bias correction and the requantization fused into its epilogue.  Replaces the
// reference's quantizedGemmBiasFused launch of ComputeLinearX
// (src/gru_forward_gpu_quant.cu:110-180, 527-562), which multiplies int32 operands on CUDA
// cores with 64-bit accumulation.
//
// Persistent kernel, one CTA per SM looping over tiles of 128 output channels (TMEM lanes) x 128
// tokens (TMEM columns); K streamed in 128-byte slabs through a 4-stage shared-memory ring that
// runs ahead across tiles; four accumulators in tensor memory (all 512 columns) so that the MMAs
// run up to three tiles ahead of the epilogue.  Warp roles: warp 0 issues the TMA loads, warp 1
// owns tensor memory and issues the MMAs, warps 2-17 run the epilogue (one TMEM lane = one
// output channel per thread, so each thread keeps its channel's constants in registers and a
// warp's stores cover 32 consecutive channels of a token).
#include <cuda.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <mutex>

#include "qgru_gemm_tc.cuh"
#include "qgru_device.cuh"
#include "qgru_tc.cuh"

#ifdef QGRU_STAMPS
// development builds only: per CTA, cycles spent waiting in each role of the GEMM kernel
__device__ long long g_gemm_dbg[160 * 8];
extern "C" __attribute__((visibility("default"))) int qgru_debug_read_gemm(long long *out) {
    return cudaMemcpyFromSymbol(out, g_gemm_dbg, sizeof(g_gemm_dbg)) == cudaSuccess ? 0 : 2;
}
#define WAITED(slot, call)                                   \
    [&] {                                                    \
        const long long t0_ = clock64();                     \
        const bool r_ = (call);                              \
        dbg_acc[slot] += clock64() - t0_;                    \
        return r_;                                           \
    }()
#else
#define WAITED(slot, call) (call)
#endif

namespace qgru {

EncodeTiledFn get_encode_tiled() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
        else
            cudaGetLastError();
    });
    return fn;
}

bool make_map_u8_sw128(CUtensorMap *map, const void *base, uint64_t rows, uint64_t row_bytes,
                       uint32_t box_rows) {
    EncodeTiledFn enc = get_encode_tiled();
    if (!enc) return false;
    const cuuint64_t dims[2] = {row_bytes, rows};
    const cuuint64_t strides[1] = {row_bytes};
    const cuuint32_t box[2] = {128, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    return enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(base), dims, strides, box, estr,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

namespace {

constexpr int GM = 128;      // channels per tile
constexpr int GN = 128;      // tokens per tile
constexpr int KB = 128;      // K bytes per stage
constexpr int STAGES = 4;
constexpr int STAGES_A = 8;    // W-stationary form: ring of x slabs (16 KB each)
constexpr int NACC = 4;        // accumulator buffers in tensor memory (NACC * GN = 512 columns: all of it)
constexpr int EPI_WARPS = 16;                      // four warps per TMEM lane quadrant
constexpr int GEMM_THREADS = 64 + 32 * EPI_WARPS;
constexpr int STAGE_BYTES = (GM + GN) * KB;
constexpr long long WAIT_BUDGET = 2000000000ll;  // ~1 s of SM clocks
constexpr int PRE_TAB_MAX = 3 * 1024;              // pre-rescale table entries kept in shared memory
constexpr size_t GEMM_SMEM = (size_t)STAGES * STAGE_BYTES + 1024 + 256 + PRE_TAB_MAX * 4;

// Fast: every scale of the epilogue has the shift-free form and the sums fit 32 bits, so the
// epilogue is branch-free (Rescale::mq, checked by the caller).
// AStat ("A stationary", option gemm_order=w_stationary only): a CTA works on one tile of 128
// channels for the whole launch and keeps that slice of W (all K slabs, K <= 1024) in TENSOR memory,
// 32 columns per 128-byte K slab, staged once through the ring's slots; only token tiles stream
// through the ring and the MMAs read their A operand from tensor memory.  It halves the operand
// bytes that cross shared memory, and measures SLOWER than the streaming form at every K (0.31
// against 0.28 ms at K = 1024, 0.16 against 0.14 at K = 256): shared-memory bandwidth is not what
// holds the streaming form's MMA rate (about 155 cycles per 128 x 128 x 32 MMA in the kernel, 68
// for the same instruction stream issued from resident operands), and the fixed channel tile per
// CTA costs balance.  Grid = m_tiles * groups CTAs; the accumulators take the columns W leaves
// (two buffers at K = 1024, three below).
// Tie = false (with Fast): the requantization rounds half up, which equals the reference's
// round-half-even because no channel can meet an exact tie in its accumulator range (checked
// when the weights are set: rescale_can_tie).
template <bool XUnsigned, typename IhT, bool Fast, bool AStat, bool Tie>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
k_gemm_wx_tc(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
             IhT *__restrict__ ih, long long N, int C, int Kpad, LinearConsts lc, PreScale ps,
             int *abort_flag, int x_row0) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char *tiles = reinterpret_cast<unsigned char *>(
        (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    // AStat: the ring holds STAGES_A x slabs of GN*KB bytes (they also stage W on its way to tensor
    // memory); else the ring holds a W slab and an x slab per stage
    constexpr int NST = AStat ? STAGES_A : STAGES;            // ring stages
    const size_t tile_bytes = AStat ? (size_t)STAGES_A * GN * KB : (size_t)STAGES * STAGE_BYTES;
    unsigned char *ring = tiles;
    uint64_t *bars = reinterpret_cast<uint64_t *>(tiles + tile_bytes);
    uint64_t *full = bars, *empty = bars + NST;
    uint64_t *acc_full = bars + 2 * NST, *acc_empty = bars + 2 * NST + NACC;
    uint64_t *a_full = bars + 2 * NST + 2 * NACC;        // AStat: a pass of W slabs has landed in the slots
    uint64_t *a_ready = a_full + 1;                      // AStat: the epilogue threads have copied that pass
    uint64_t *w_done = a_full + 2;                       // AStat: all of W sits in tensor memory
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(a_full + 3);
    int *failed = reinterpret_cast<int *>(tmem_slot + 1);
    int32_t *pre_tab = reinterpret_cast<int32_t *>(tiles + tile_bytes + 256);
    const bool use_tab = ps.enabled && ps.table != nullptr && 3 * ps.table_n <= PRE_TAB_MAX;
    if (use_tab)
        for (int i = threadIdx.x; i < 3 * ps.table_n; i += blockDim.x) pre_tab[i] = ps.table[i];

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int num_kb = Kpad / KB;
    const int m_tiles = (C + GM - 1) / GM;
    const long long n_tiles = (N + GN - 1) / GN;
    const long long total = (long long)m_tiles * n_tiles;   // consecutive tiles share the token tile
    const int groups = AStat ? (int)gridDim.x / m_tiles : 1;
    // accumulator buffers: all 512 columns in the streaming form; beside W in the stationary form
    const int nacc = AStat ? (num_kb > 4 ? 2 : 3) : NACC;
    const uint32_t w_col = (uint32_t)(nacc * GN);          // first tensor-memory column of W
    // the `local`-th tile of this CTA: false when there is none
    auto tile_of = [&](long long local, int &m0, long long &n0) -> bool {
        if (AStat) {
            const long long n = (long long)(blockIdx.x / m_tiles) + local * groups;
            if (n >= n_tiles || (int)blockIdx.x >= m_tiles * groups) return false;
            m0 = (int)(blockIdx.x % m_tiles) * GM;
            n0 = n * GN;
        } else {
            const long long tile = blockIdx.x + local * gridDim.x;
            if (tile >= total) return false;
            m0 = (int)(tile % m_tiles) * GM;
            n0 = (tile / m_tiles) * GN;
        }
        return true;
    };

    if (threadIdx.x == 0) {
        for (int s = 0; s < NST; ++s) {
            tc::mbar_init(&full[s], 1);
            tc::mbar_init(&empty[s], 1);
        }
        for (int b = 0; b < NACC; ++b) {
            tc::mbar_init(&acc_full[b], 1);
            tc::mbar_init(&acc_empty[b], EPI_WARPS);
        }
        tc::mbar_init(a_full, 1);
        tc::mbar_init(a_ready, 32 * EPI_WARPS);
        tc::mbar_init(w_done, 1);
        *failed = 0;
        tc::fence_barrier_init();
        tc::tma_prefetch_desc(&map_w);
        tc::tma_prefetch_desc(&map_x);
    }
    if (warp == 1) tc::tmem_alloc(tmem_slot, 512);   // several accumulators: the MMAs run ahead of the epilogue
    tc::tc_fence_before_sync();
    __syncthreads();
    tc::tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            long long it = 0;   // k-slab counter across tiles: ring position and phase
            bool ok = true;
            int m0;
            long long n0;
#ifdef QGRU_STAMPS
            long long dbg_acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#endif
            if (AStat) {
                // this CTA's slice of W, once: through the ring's slots into tensor memory, a pass of up
                // to STAGES_A slabs at a time (every CTA takes part, with or without tiles of its own,
                // so that the barriers below see the same sequence everywhere)
                m0 = (int)(blockIdx.x % m_tiles) * GM;
                int pass = 0;
                for (int done = 0; done < num_kb && ok; ++pass) {
                    const int cnt = min(STAGES_A, num_kb - done);
                    tc::mbar_expect_tx(a_full, (uint32_t)(cnt * GM * KB));
                    for (int i = 0; i < cnt; ++i)
                        tc::tma_load_2d(ring + (size_t)i * GM * KB, &map_w, a_full, (done + i) * KB, m0);
                    ok = tc::mbar_wait(a_ready, (uint32_t)(pass & 1), WAIT_BUDGET);
                    done += cnt;
                }
                tc::mbar_arrive(w_done);
            }
            for (long long local = 0; ok && tile_of(local, m0, n0); ++local) {
                for (int kb = 0; kb < num_kb; ++kb, ++it) {
                    const int s = (int)(it % NST);
                    const uint32_t ph = (uint32_t)((it / NST) & 1);
                    if (!WAITED(0, tc::mbar_wait(&empty[s], ph ^ 1, WAIT_BUDGET))) { ok = false; break; }
                    if (AStat) {
                        tc::mbar_expect_tx(&full[s], GN * KB);
                        tc::tma_load_2d(ring + (size_t)s * GN * KB, &map_x, &full[s], kb * KB, (int)n0 + x_row0);
                    } else {
                        unsigned char *a = tiles + (size_t)s * STAGE_BYTES;
                        tc::mbar_expect_tx(&full[s], STAGE_BYTES);
                        tc::tma_load_2d(a, &map_w, &full[s], kb * KB, m0);
                        tc::tma_load_2d(a + GM * KB, &map_x, &full[s], kb * KB, (int)n0 + x_row0);
                    }
                }
            }
            if (!ok) atomicExch(failed, 1);
#ifdef QGRU_STAMPS
            if (blockIdx.x < 160) g_gemm_dbg[blockIdx.x * 8 + 0] = dbg_acc[0];
#endif
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t idesc = tc::idesc_i8(GM, GN, true, !XUnsigned);
            bool ok = true;
            int m0;
            long long n0;
#ifdef QGRU_STAMPS
            long long dbg_acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
            const long long t_start = clock64();
#endif
            if (AStat) {
                ok = tc::mbar_wait(w_done, 0, WAIT_BUDGET);
                tc::tc_fence_after_sync();
            }
            // The loop below is this thread's whole instruction stream and it shares its scheduler
            // with four busy epilogue warps: ring position, barrier addresses and descriptor low words
            // advance by one add each, nothing is recomputed per slab.
            const uint32_t full0 = tc::smem_u32(full), empty0 = tc::smem_u32(empty);
            const uint32_t ring_lo0 = tc::smem_desc_sw128_lo(tc::smem_u32(ring));
            constexpr uint32_t SLOT_LO = (uint32_t)((AStat ? GN * KB : STAGE_BYTES) >> 4);   // descriptor units per ring slot
            constexpr uint32_t B_LO = AStat ? 0u : (uint32_t)((GM * KB) >> 4);               // x slab behind the W slab
            int s = 0;
            uint32_t ph = 0, slot_lo = ring_lo0;
            int buf = 0;
            uint32_t acc_ph = 1;   // parity to wait for on acc_empty: buffers start out free
            for (long long local = 0; ok && tile_of(local, m0, n0); ++local) {
                if (!WAITED(2, tc::mbar_wait(&acc_empty[buf], acc_ph, WAIT_BUDGET))) { ok = false; break; }
                tc::tc_fence_after_sync();
                const uint32_t d_col = tmem_base + (uint32_t)(buf * GN);
                for (int kb = 0; kb < num_kb; ++kb) {
                    // (TMA's writes are ordered before the MMAs by the barrier alone; the tcgen05 fence
                    // belongs after the accumulator hand-over above, not here)
                    if (!WAITED(1, tc::mbar_wait_addr(full0 + 8u * (uint32_t)s, ph, WAIT_BUDGET))) { ok = false; break; }
                    if (AStat) {
                        const uint32_t a_col = tmem_base + w_col + (uint32_t)(kb * 32);
                        tc::mma_i8_ts_lo(d_col, a_col, slot_lo, idesc, (uint32_t)kb);
                        tc::mma_i8_ts_lo(d_col, a_col + 8, slot_lo + 2, idesc, 1u);
                        tc::mma_i8_ts_lo(d_col, a_col + 16, slot_lo + 4, idesc, 1u);
                        tc::mma_i8_ts_lo(d_col, a_col + 24, slot_lo + 6, idesc, 1u);
                    } else {
                        tc::mma_i8_lo(d_col, slot_lo, slot_lo + B_LO, idesc, (uint32_t)kb);
                        tc::mma_i8_lo(d_col, slot_lo + 2, slot_lo + B_LO + 2, idesc, 1u);
                        tc::mma_i8_lo(d_col, slot_lo + 4, slot_lo + B_LO + 4, idesc, 1u);
                        tc::mma_i8_lo(d_col, slot_lo + 6, slot_lo + B_LO + 6, idesc, 1u);
                    }
                    static_assert(KB / 32 == 4, "four MMAs of K = 32 per slab");
                    tc::mma_commit_addr(empty0 + 8u * (uint32_t)s);
                    slot_lo += SLOT_LO;
                    if (++s == NST) {
                        s = 0;
                        ph ^= 1u;
                        slot_lo = ring_lo0;
                    }
                }
                if (ok) tc::mma_commit(&acc_full[buf]);
                if (++buf == nacc) {
                    buf = 0;
                    acc_ph ^= 1u;
                }
            }
            if (!ok) atomicExch(failed, 1);
#ifdef QGRU_STAMPS
            if (blockIdx.x < 160) {
                g_gemm_dbg[blockIdx.x * 8 + 1] = dbg_acc[1];
                g_gemm_dbg[blockIdx.x * 8 + 2] = dbg_acc[2];
                g_gemm_dbg[blockIdx.x * 8 + 3] = clock64() - t_start;
            }
#endif
        }
    } else {
        const int q = warp & 3;                     // TMEM lane quadrant of this warp
#ifdef QGRU_STAMPS
        long long dbg_acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        const long long t_start = clock64();
#endif
        const int part = (warp - 2) >> 2;           // which share of the token columns
        constexpr int COLS = GN / (EPI_WARPS / 4);
        long long local = 0;
        bool ok = true;
        // per-channel constants of a tile's rows: loaded one tile ahead, so that their global-memory
        // latency is not paid at the start of every tile
        struct ChanConsts {
            int64_t corr;
            Rescale rs;
            FastLin fl;
            float fs_off, fs_bias, fs_ratio;   // float-storage forward (lc.fs set)
        };
        auto load_consts = [&](long long lcl) {
            ChanConsts c;
            int tm0 = 0;
            long long tn0 = 0;
            const bool have = tile_of(lcl, tm0, tn0);
            const int m = tm0 + q * 32 + lane;
            const bool m_ok = have && m < C;
            c.corr = m_ok ? lc.corr[m] : 0;
            c.rs = m_ok ? lc.rs[m] : Rescale{1, 1, 0, 0, 0, 0, 0, 0};
            c.fl = m_ok ? lc.fl[m] : FastLin{0, 0, 0, 0, 0, 0};
            const bool fs_ok = m_ok && lc.fs != nullptr;
            c.fs_off = fs_ok ? lc.fs[m] : 0.f;
            c.fs_bias = fs_ok ? lc.fs[lc.fs_C + m] : 0.f;
            c.fs_ratio = fs_ok ? lc.fs[2 * lc.fs_C + m] : 0.f;
            return c;
        };
        if (AStat) {
            // W on its way to tensor memory: this thread owns channel row (32 q + lane) of every slab, eight
            // 16-byte chunks un-swizzled on the way, 32 columns per slab
            const int u = q * 32 + lane;
            int pass = 0;
            for (int done = 0; done < num_kb && ok; ++pass) {
                const int cnt = min(STAGES_A, num_kb - done);
                ok = tc::mbar_wait(a_full, (uint32_t)(pass & 1), WAIT_BUDGET);
                for (int i = part; i < cnt && ok; i += EPI_WARPS / 4) {
                    const unsigned char *row = ring + (size_t)i * GM * KB + (size_t)(u >> 3) * 1024 + (size_t)(u & 7) * 128;
                    uint32_t w[32];
#pragma unroll
                    for (int c = 0; c < 8; ++c) {
                        const uint4 v = *reinterpret_cast<const uint4 *>(row + ((c ^ (u & 7)) << 4));
                        w[4 * c + 0] = v.x;
                        w[4 * c + 1] = v.y;
                        w[4 * c + 2] = v.z;
                        w[4 * c + 3] = v.w;
                    }
                    tc::tmem_st32(tmem_base + ((uint32_t)(q * 32) << 16) + w_col + (uint32_t)((done + i) * 32), w);
                }
                tc::tmem_st_wait();
                tc::tc_fence_before_sync();
                tc::mbar_arrive(a_ready);
                done += cnt;
            }
        }
        ChanConsts cur = load_consts(0);
        int m0;
        long long n0;
        for (; ok && tile_of(local, m0, n0); ++local) {
            const int buf = (int)(local % nacc);
            const int m = m0 + q * 32 + lane;
            const bool m_ok = m < C;
            const ChanConsts nxt = AStat ? cur : load_consts(local + 1);
            const int64_t corr = cur.corr;
            const Rescale rs = cur.rs;
            const FastLin fl = cur.fl;
            // fused-cell mode: the channel's gate decides the second rescale (to its input scale)
            const int gate = (ps.enabled && m_ok) ? m / ps.H : 0;
            const Rescale pre_rs = ps.to[gate];
            const int32_t pre_zp = ps.zp_in[gate];
            const int32_t c32 = (int32_t)corr;
            ok = WAITED(4, tc::mbar_wait(&acc_full[buf], (uint32_t)((local / nacc) & 1), WAIT_BUDGET));
            if (!ok) break;
            tc::tc_fence_after_sync();
            IhT *out = ih + m;
            // this warp's COLS accumulator columns: both halves are fetched before anything is
            // computed, and the buffer goes back to the MMA warp as soon as they have arrived
            static_assert(COLS == 32, "two 16-column loads per warp and tile");
            int32_t vv[2][16];
            tc::tmem_ld16(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * GN + part * COLS), vv[0]);
            tc::tmem_ld16(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * GN + part * COLS + 16), vv[1]);
#ifdef QGRU_STAMPS
            const long long t_ld = clock64();
#endif
            tc::tmem_ld_wait();
#ifdef QGRU_STAMPS
            dbg_acc[5] += clock64() - t_ld;
#endif
            tc::tc_fence_before_sync();
            if (lane == 0) tc::mbar_arrive(&acc_empty[buf]);
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const int c0 = part * COLS + 16 * half;
                const int32_t (&v)[16] = vv[half];
                int32_t y[16];
                if constexpr (Fast) {
                    // all 16 values first, stores afterwards: the chains interleave
                    if (use_tab) {
                        // zero point, clamp and table offset folded into one add and a max/min pair
                        const uint32_t tb = tc::smem_u32(pre_tab);
                        const int32_t t_c = gate * ps.table_n + lc.zp_out - ps.lo;
                        const int32_t t_lo = gate * ps.table_n + lc.lo - ps.lo, t_hi = t_lo + (lc.hi - lc.lo);
#pragma unroll
                        for (int i = 0; i < 16; ++i)
                            y[i] = lds_i32(tb + 4u * (uint32_t)min(max(lin_round<Tie>(v[i], fl) + t_c, t_lo), t_hi));
                    } else if (ps.enabled) {
#pragma unroll
                        for (int i = 0; i < 16; ++i)
                            y[i] = mul_round_hi(linear_epilogue_fast<Tie>(v[i], fl, lc.zp_out, lc.lo, lc.hi) - ps.zp_ih, pre_rs) + pre_zp;
                    } else {
#pragma unroll
                        for (int i = 0; i < 16; ++i) y[i] = linear_epilogue_fast<Tie>(v[i], fl, lc.zp_out, lc.lo, lc.hi);
                    }
                } else if (lc.fs != nullptr) {
                    // float-storage forward: the reference's float requantization of the exact sum
#pragma unroll
                    for (int i = 0; i < 16; ++i)
                        y[i] = (int32_t)fs_linear(v[i], cur.fs_off, cur.fs_bias, cur.fs_ratio, (float)lc.zp_out,
                                                  (float)lc.lo, (float)lc.hi);
                } else {
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        int32_t t = lc.fits32 ? linear_epilogue32(v[i], c32, rs, lc.zp_out, lc.lo, lc.hi)
                                              : linear_epilogue(v[i], corr, rs, lc.zp_out, lc.lo, lc.hi);
                        if (use_tab) t = pre_tab[gate * ps.table_n + (t - ps.lo)];
                        else if (ps.enabled) t = (int32_t)rescale32(t - ps.zp_ih, pre_rs) + pre_zp;
                        y[i] = t;
                    }
                }
                // token n of channel m lives at ih[n * C + m]: one pointer walked by C elements
                IhT *po = out + (n0 + c0) * C;
                if (m_ok && n0 + c0 + 16 <= N) {
#pragma unroll
                    for (int i = 0; i < 16; ++i, po += C) *po = (IhT)y[i];
                } else if (m_ok) {
#pragma unroll
                    for (int i = 0; i < 16; ++i, po += C)
                        if (n0 + c0 + i < N) *po = (IhT)y[i];
                }
            }
            cur = nxt;
        }
        if (!ok && lane == 0) atomicExch(failed, 1);
#ifdef QGRU_STAMPS
        if (warp == 2 && lane == 0 && blockIdx.x < 160) {
            g_gemm_dbg[blockIdx.x * 8 + 4] = dbg_acc[4];
            g_gemm_dbg[blockIdx.x * 8 + 5] = dbg_acc[5];
            g_gemm_dbg[blockIdx.x * 8 + 6] = clock64() - t_start;
            g_gemm_dbg[blockIdx.x * 8 + 7] = local;
        }
#endif
    }
    tc::tc_fence_before_sync();
    __syncthreads();
    if (threadIdx.x == 0 && *failed) atomicOr(abort_flag, 2);
    if (warp == 1) tc::tmem_dealloc(tmem_base, 512);
}

constexpr size_t SMEM_LIMIT = 227 * 1024;   // opt-in shared memory per CTA on sm_100

size_t astat_smem(int) { return (size_t)STAGES_A * GN * KB + 1024 + 256 + PRE_TAB_MAX * 4; }

template <bool XU, typename IhT, bool Fast, bool Tie>
cudaError_t launch_f(const CUtensorMap &mw, const CUtensorMap &mx, void *ih, long long N, int C, int Kpad,
                     LinearConsts lc, PreScale ps, int *abort_flag, int sms, int order, int x_row0, cudaStream_t st) {
    const int m_tiles = (C + GM - 1) / GM;
    const long long n_tiles = (N + GN - 1) / GN;
    // W-stationary form (W in tensor memory): on request only (option gemm_order=w_stationary), it is
    // the slower of the two; needs K <= 1024 and a channel tile per CTA
    const bool fits = Kpad <= 1024 && m_tiles <= sms;
    const bool astat = fits && order == 2;
    if (astat) {
        auto kern = k_gemm_wx_tc<XU, IhT, Fast, true, Tie>;
        const size_t smem = astat_smem(Kpad);
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
        const long long groups = std::max<long long>(1, std::min<long long>(sms / m_tiles, n_tiles));
        kern<<<(unsigned)(m_tiles * groups), GEMM_THREADS, smem, st>>>(mw, mx, (IhT *)ih, N, C, Kpad, lc, ps, abort_flag, x_row0);
        return cudaGetLastError();
    }
    auto kern = k_gemm_wx_tc<XU, IhT, Fast, false, Tie>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)GEMM_SMEM);
    if (e != cudaSuccess) return e;
    const long long tiles = (long long)m_tiles * n_tiles;
    const unsigned grid = (unsigned)std::min<long long>(tiles, sms);   // persistent: one CTA per SM
    kern<<<grid, GEMM_THREADS, GEMM_SMEM, st>>>(mw, mx, (IhT *)ih, N, C, Kpad, lc, ps, abort_flag, x_row0);
    return cudaGetLastError();
}

template <bool XU, typename IhT>
cudaError_t launch(const CUtensorMap &mw, const CUtensorMap &mx, void *ih, long long N, int C, int Kpad,
                   LinearConsts lc, PreScale ps, bool fast, bool notie, int *abort_flag, int sms, int order,
                   int x_row0, cudaStream_t st) {
    if (fast && notie) return launch_f<XU, IhT, true, false>(mw, mx, ih, N, C, Kpad, lc, ps, abort_flag, sms, order, x_row0, st);
    return fast ? launch_f<XU, IhT, true, true>(mw, mx, ih, N, C, Kpad, lc, ps, abort_flag, sms, order, x_row0, st)
                : launch_f<XU, IhT, false, true>(mw, mx, ih, N, C, Kpad, lc, ps, abort_flag, sms, order, x_row0, st);
}

}  // namespace

int tc_gemm_launch(TcGemmState &s, const uint8_t *x8, long long x_rows_alloc, const int8_t *w8,
                   long long w_rows_alloc, void *ih, long long N, int C, int Kpad, bool x_unsigned,
                   int ih_bytes, LinearConsts lc, PreScale ps, bool fast, bool notie, int *abort_flag, int sms,
                   cudaStream_t stream, std::string *err, long long x_row0) {
    // (token tiles that reach past the last allocated row read the tensor map's zero fill)
    if (Kpad % KB != 0 || x_row0 < 0 || x_row0 + N > x_rows_alloc || x_rows_alloc >= 0x7fffffffll ||
        (x_row0 == 0 && x_rows_alloc < (N + GN - 1) / GN * GN) || w_rows_alloc < (C + GM - 1) / GM * GM) {
        if (err) *err = "tcgen05 GEMM needs K padded to 128 and operand rows padded to the tile";
        return QGRU_ERR_UNSUPPORTED;
    }
    if (!s.valid || s.x8 != x8 || s.w8 != w8 || s.x_rows != x_rows_alloc || s.w_rows != w_rows_alloc ||
        s.Kpad != Kpad) {
        static_assert(sizeof(CUtensorMap) <= sizeof(s.map_w), "tensor map storage too small");
        if (!make_map_u8_sw128(reinterpret_cast<CUtensorMap *>(s.map_w), w8, (uint64_t)w_rows_alloc, (uint64_t)Kpad, GM) ||
            !make_map_u8_sw128(reinterpret_cast<CUtensorMap *>(s.map_x), x8, (uint64_t)x_rows_alloc, (uint64_t)Kpad, GN)) {
            if (err) *err = "cuTensorMapEncodeTiled failed";
            return QGRU_ERR_CUDA;
        }
        s.valid = true;
        s.x8 = x8;
        s.w8 = w8;
        s.x_rows = x_rows_alloc;
        s.w_rows = w_rows_alloc;
        s.Kpad = Kpad;
    }
    const CUtensorMap &mw = *reinterpret_cast<const CUtensorMap *>(s.map_w);
    const CUtensorMap &mx = *reinterpret_cast<const CUtensorMap *>(s.map_x);
    // the branch-free epilogue applies the second rescale from the table, or needs its shift-free form
    const bool tab = ps.enabled && ps.table != nullptr && 3 * ps.table_n <= PRE_TAB_MAX;
    fast = fast && (!ps.enabled || tab || (ps.to[0].mq != 0 && ps.to[1].mq != 0 && ps.to[2].mq != 0));
    cudaError_t e;
    if (ih_bytes == 1)
        e = x_unsigned ? launch<true, int8_t>(mw, mx, ih, N, C, Kpad, lc, ps, fast, notie, abort_flag, sms, s.order, (int)x_row0, stream)
                       : launch<false, int8_t>(mw, mx, ih, N, C, Kpad, lc, ps, fast, notie, abort_flag, sms, s.order, (int)x_row0, stream);
    else if (ih_bytes == 2)
        e = x_unsigned ? launch<true, int16_t>(mw, mx, ih, N, C, Kpad, lc, ps, fast, notie, abort_flag, sms, s.order, (int)x_row0, stream)
                       : launch<false, int16_t>(mw, mx, ih, N, C, Kpad, lc, ps, fast, notie, abort_flag, sms, s.order, (int)x_row0, stream);
    else
        e = x_unsigned ? launch<true, int32_t>(mw, mx, ih, N, C, Kpad, lc, ps, fast, notie, abort_flag, sms, s.order, (int)x_row0, stream)
                       : launch<false, int32_t>(mw, mx, ih, N, C, Kpad, lc, ps, fast, notie, abort_flag, sms, s.order, (int)x_row0, stream);
    if (e != cudaSuccess) {
        if (err) *err = std::string("tcgen05 GEMM launch: ") + cudaGetErrorString(e);
        return QGRU_ERR_CUDA;
    }
    return QGRU_OK;
}

}  // namespace qgru
