// qgru_rec_c64.cu - the cluster recurrence with 64 hidden units per CTA: the low-latency form
// for steps that are short on batch rows per SM.
//
// Why another split.  A tcgen05.mma kind::i8 with few batch columns (N <= 48) costs about 44
// SM cycles whatever its M or N (measured: qgru_probe_mma_i8), so the length of a step's MMA
// chain is its instruction count, and the cells of a step issue at about 150 instructions each.
// With 128 units per CTA (qgru_rec_cluster.cu) a step is 48 MMAs and 4 cells per thread at 16
// batch rows.  Here a CTA owns 64 units: the update and reset rows of its units share ONE
// 128-row A tile, the new-gate rows sit in the lower half of each 32-row quadrant of a second
// tile (upper halves zero), so a step is 32 MMAs per K = 512 and 2 cells per thread - both
// halves of the step shrink, twice as many SMs share a direction's rows, and two sub-groups per
// CTA overlap the MMAs of one with the cells of the other.
//
// Row order of the A tiles, chosen so that the three gate sums of a unit meet inside one warp:
//   tile ZR, TMEM lane 32 q + l      (l < 16): update-gate row of unit 16 q + l
//            TMEM lane 32 q + 16 + l          : reset-gate row of the same unit
//   tile N,  TMEM lane 32 q + l      (l < 16): new-gate row of unit 16 q + l;  lanes 32 q + 16 + l: zeros
// A warp reads its quadrant's 32 lanes: lanes l and l + 16 of the warp form a pair that owns one
// unit.  Both run the same gate code on four batch columns - one on the update gate, the other
// on the reset gate, each with its own table offsets - then swap what the partner needs with
// three shuffle pairs and each finishes two of the four cells (new gate and state update).
//
// MMA issue.  One thread issues a dependent chain of these MMAs at one per 53-80 cycles, but the
// tensor pipe takes MMAs from several threads side by side (four issuing warps reach its full
// rate: qgru_probe_mma_i8_ex).  So the step's MMAs are dealt to four issuing warps, one per
// (tile, K half), each accumulating into columns of its own; the cells add the two K halves.
//
// Everything else is the cluster kernel's scheme: R resident in tensor memory for all T steps,
// h_t exchanged between the P (<= 8) CTAs of a cluster through distributed shared memory with
// st.async counted on the receivers' mbarriers, double-buffered state tiles, bounded waits.
// Only the branch-free tabulated cell (every scale of the step in shift-free form) runs here;
// every other configuration stays on qgru_rec_cluster.cu.  Replaces, like that kernel, the
// reference's two launches per step (src/gru_forward_gpu_quant.cu:565-668, 817-828).
#include <cuda.h>
#include <cuda_runtime.h>

#include "qgru_cluster.cuh"
#include "qgru_device.cuh"
#include "qgru_rec_mma.cuh"
#include "qgru_tc.cuh"

#ifdef QGRU_STAMPS
#define STAMP(cond, slot) do { if (a.dbg && blockIdx.x < 2 && (cond)) a.dbg[(((size_t)blockIdx.x * a.T + s) * 2 + g) * 32 + (slot)] = clock64(); } while (0)
#else
#define STAMP(cond, slot) do { } while (0)
#endif

namespace qgru {
using namespace clu;
namespace {

constexpr long long WAIT_BUDGET = 2000000000ll;  // ~1 s of SM clocks
constexpr int EPW = 4;                           // epilogue warps per TMEM lane quadrant
constexpr int EPI_THREADS = 32 * 4 * EPW;
constexpr int ISSUERS = 4;                       // warp 0 and the three warps after the epilogue warps
constexpr int REC_THREADS = 32 * ISSUERS + EPI_THREADS;
constexpr int UT = 64;                           // hidden units per CTA
constexpr int MAX_NG = 2;

struct Smem64 {
    size_t r_tiles, h_tile, bars, tables, total;
};

__host__ __device__ inline Smem64 smem64_layout(int KBn, int NB, int NG, int n_table) {
    Smem64 s;
    s.r_tiles = 0;                                        // 2 * KBn tiles of 16 KB: staging on the way to tensor memory
    s.h_tile = (size_t)2 * KBn * 16384;
    s.bars = s.h_tile + (size_t)NG * 2 * KBn * NB * 128;  // two state buffers per sub-group
    s.tables = s.bars + 256;
    s.total = s.tables + (((size_t)n_table * 4 + 15) & ~size_t(15));
    return s;
}

__device__ __forceinline__ int32_t lookup(uint32_t tab, int32_t v, int32_t c, int32_t lo, int32_t hi) {
    return lds_i32(tab + 4u * (uint32_t)min(max(v + c, lo), hi));
}

// Tie = false: the rescales round half up, equal to round-half-even where no operand can be an
// exact tie (rescale_can_tie, checked on the host).
template <typename IhT, bool Tie>
__global__ void __launch_bounds__(REC_THREADS, 1)
k_recurrence_c64(const __grid_constant__ CUtensorMap map_r, const __grid_constant__ CUtensorMap map_h,
                 const __grid_constant__ GateConsts gc, RecMmaArgs a) {
    extern __shared__ unsigned char smem_raw[];
    // every CTA of the cluster computes the same offsets (see qgru_rec_cluster.cu)
    const uint32_t raw = tc::smem_u32(smem_raw);
    unsigned char *base = smem_raw + (((raw + 1023u) & ~1023u) - raw);
    const int KBn = a.Hpad >> 7;
    const int NG = a.NG;
    const Smem64 L = smem64_layout(KBn, a.NB, NG, a.n_table);
    unsigned char *r_tiles = base + L.r_tiles;
    unsigned char *h_tile = base + L.h_tile;                  // [NG][2 buffers][KBn slabs][NB rows][128 bytes]
    const uint32_t h_buf_bytes = (uint32_t)(KBn * a.NB * 128);
    uint64_t *bars = reinterpret_cast<uint64_t *>(base + L.bars);
    uint64_t *r_full = bars, *h_full = bars + 1, *r_ready = bars + 2;
    uint64_t *h_ready = bars + 3;                    // [NG][2]
    uint64_t *mma_done = bars + 3 + 2 * MAX_NG;      // [NG][2]: tile ZR / tile N accumulated
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 3 + 4 * MAX_NG);
    int32_t *tables = reinterpret_cast<int32_t *>(base + L.tables);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, tid = threadIdx.x;
    const int grp = blockIdx.x / a.P;
    const int p = (int)cluster_rank();
    const int j0 = p * UT;
    const int b0 = a.b_off + grp * NG * a.NB;
    const uint32_t tmem_cols = a.tmem_cols;
    const int n_tiles = 2 * KBn;

    for (int i = tid; i < a.n_table; i += blockDim.x) tables[i] = a.tables[i];
    if (tid == 0) {
        tc::mbar_init(r_full, 1);
        tc::mbar_init(h_full, 1);
        for (int g = 0; g < 2 * NG; ++g) tc::mbar_init(&mma_done[g], (uint32_t)a.k_parts);   // one commit per K part
        for (int g = 0; g < 2 * NG; ++g) tc::mbar_init(&h_ready[g], 4 * EPW + 1);
        tc::mbar_init(r_ready, EPI_THREADS);
        tc::fence_barrier_init();
        tc::tma_prefetch_desc(&map_r);
        tc::tma_prefetch_desc(&map_h);
    }
    if (warp == 0) tc::tmem_alloc(tmem_slot, tmem_cols);
    tc::tc_fence_before_sync();
    __syncthreads();
    tc::tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    cluster_arrive();   // no CTA may receive a peer's block before its barriers are initialised
    cluster_wait();

    if (warp == 0 || warp > 4 * EPW) {
        // ------------------------------------------------------------------ issuing warps
        // issuer cw multiplies tile (cw & 1: ZR / N) over K part (cw >> 1); issuer 0 also loads R and the
        // initial state and announces the peers' bytes on the state barriers
        const int cw = warp == 0 ? 0 : warp - 4 * EPW;
        const int ts = cw & 1, part = cw >> 1;
        if (lane == 0 && part < a.k_parts) {
            bool ok = true;
            if (cw == 0) {
                // The two tile sets of this CTA's R slice, K-slab by K-slab, in boxes of 16 rows (one run of
                // consecutive units of one gate); rows past 3H of the packed R are zeros and fill the unused
                // halves of tile N.
                const int zero_row = a.C + 128;
                tc::mbar_expect_tx(r_full, (uint32_t)n_tiles * 16384u);
                for (int kb = 0; kb < KBn; ++kb) {
                    unsigned char *zr = r_tiles + (size_t)kb * 16384, *nn = r_tiles + (size_t)(KBn + kb) * 16384;
                    for (int q = 0; q < 4; ++q) {
                        tc::tma_load_2d(zr + (size_t)(2 * q) * 2048, &map_r, r_full, kb * 128, 0 * a.H + j0 + 16 * q);
                        tc::tma_load_2d(zr + (size_t)(2 * q + 1) * 2048, &map_r, r_full, kb * 128, 1 * a.H + j0 + 16 * q);
                        tc::tma_load_2d(nn + (size_t)(2 * q) * 2048, &map_r, r_full, kb * 128, 2 * a.H + j0 + 16 * q);
                        tc::tma_load_2d(nn + (size_t)(2 * q + 1) * 2048, &map_r, r_full, kb * 128, zero_row);
                    }
                }
                // the initial state (written by the preceding kernel) into buffer 0 of every sub-group
                tc::mbar_expect_tx(h_full, (uint32_t)NG * h_buf_bytes);
                for (int g = 0; g < NG; ++g)
                    for (int kb = 0; kb < KBn; ++kb)
                        tc::tma_load_2d(h_tile + (size_t)(2 * g) * h_buf_bytes + (size_t)kb * a.NB * 128, &map_h, h_full,
                                        kb * 128, b0 + g * a.NB);
            }
            ok = tc::mbar_wait(r_ready, 0, WAIT_BUDGET);   // the epilogue threads have moved the tiles to tensor memory
            ok = ok && tc::mbar_wait(h_full, 0, WAIT_BUDGET);
            tc::tc_fence_after_sync();
            const uint32_t idesc = tc::idesc_i8(128, a.NB, true, !a.h_unsigned);
            const uint32_t h_lo0 = (tc::smem_u32(h_tile) & 0x3FFFFu) >> 4;
            const uint32_t desc_hi = (uint32_t)(tc::smem_desc_sw128(0) >> 32);
            const uint32_t desc_lo = (uint32_t)tc::smem_desc_sw128(0);
            const uint64_t dhi = (uint64_t)desc_hi << 32;
            const uint32_t ra = tmem_base + (uint32_t)(a.r_tmem_col + ts * KBn * 32);
            const uint32_t blk_bytes = (uint32_t)(a.NB * UT);            // what one peer sends per sub-group and step
            const int kb0 = part == 0 ? 0 : (KBn + 1) / 2;               // this issuer's K-slabs: [kb0, kb1)
            const int kb1 = (a.k_parts == 1 || part == 1) ? KBn : (KBn + 1) / 2;
            for (int s = 0; s < a.T && ok; ++s) {
                for (int g = 0; g < NG; ++g) {
                    const uint32_t buf = (uint32_t)(2 * g + (s & 1));
                    if (s > 0) {
                        if (cw == 0) tc::mbar_expect_tx(&h_ready[buf], (uint32_t)(a.P - 1) * blk_bytes);
                        if (!tc::mbar_wait(&h_ready[buf], (uint32_t)(((s - 1) >> 1) & 1), WAIT_BUDGET)) { ok = false; break; }
                        fence_proxy_async_cta();   // the MMAs read these stores through the async proxy
                    }
                    tc::tc_fence_after_sync();
                    STAMP(true, 2 * cw);
                    const uint32_t hbuf = h_lo0 + ((buf * h_buf_bytes) >> 4);
                    const uint32_t d = tmem_base + (uint32_t)(((2 * g + ts) * a.k_parts + part) * a.NB);
#pragma unroll
                    for (int kb = 0; kb < 4; ++kb)
                        if (kb >= kb0 && kb < kb1) {
#pragma unroll
                            for (int ks = 0; ks < 4; ++ks)
                                tc::mma_i8_ts(d, ra + (uint32_t)(kb * 32 + ks * 8),
                                              dhi | (desc_lo | (hbuf + (uint32_t)(kb * a.NB * 8 + 2 * ks))), idesc,
                                              (kb != kb0 || ks != 0) ? 1u : 0u);
                        }
                    tc::mma_commit(&mma_done[2 * g + ts]);
                    STAMP(true, 2 * cw + 1);
                }
            }
            if (!ok) atomicOr(a.abort_flag, 1);
        }
    } else {
        // ---------------------------------------------------------------- epilogue warps (1 .. 16)
        const int q = warp & 3;                      // TMEM lane quadrant this warp may read
        const int rank = (warp - 1) >> 2;            // 0..EPW-1 among the warps of that quadrant
        const int half = lane >> 4;                  // 0: this lane holds update-gate rows, 1: reset-gate rows
        const int ul = 16 * q + (lane & 15);         // unit within the CTA's 64, shared with lane ^ 16
        const int j = j0 + ul;
        const bool j_ok = j < a.H;
        const size_t BH = (size_t)a.B * a.H;
        const IhT *ihp = reinterpret_cast<const IhT *>(a.ih);
        const int nchunks = a.NB / 4;
        const uint32_t tab = tc::smem_u32(tables);
        const uint32_t h_bits = a.h_unsigned ? 9u : 8u;
        const FastLin fl_g = j_ok ? a.lc.fl[half * a.H + j] : FastLin{0, 0, 0, 0, 0, 0};
        const FastLin fl_n = j_ok ? a.lc.fl[2 * a.H + j] : FastLin{0, 0, 0, 0, 0, 0};
        // table index arithmetic of this lane's gate (fused_gate_fast with the gate chosen per lane)
        const int32_t hc_c = gc.fi_c[3 + half], hc_lo = gc.fi_lo[3 + half], hc_hi = gc.fi_hi[3 + half];
        const int32_t gt_c = gc.fi_c[half], gt_lo = gc.fi_lo[half], gt_hi = gc.fi_hi[half];
        // state exchange: lane t & 15 assembles the word (row (t & 15) >> 2 of the chunk, units 4 (t & 3) .. + 3 of
        // this warp's 16) from byte `x_bi` of four lanes of the half that finished that row; lanes 0-15 send it
        // to the even-ranked peers, lanes 16-31 to the odd-ranked ones
        const int x_rr = (lane & 15) >> 2, x_w = lane & 3;
        const int x_src = 16 * (x_rr >> 1) + 4 * x_w;
        const uint32_t x_sel = (uint32_t)(x_rr & 1) | ((uint32_t)(4 + (x_rr & 1)) << 4);
        const uint32_t tile_u32 = tc::smem_u32(h_tile);
        const uint32_t bar_u32 = tc::smem_u32(h_ready);
        bool ok = tc::mbar_wait(r_full, 0, WAIT_BUDGET);
        // Move the staged tiles into tensor memory: this thread owns row (32 q + lane) of every tile,
        // eight 16-byte chunks un-swizzled on the way, 32 columns per tile.
        {
            const int u = q * 32 + lane;
            for (int i = rank; i < n_tiles && ok; i += EPW) {
                const unsigned char *row = r_tiles + (size_t)i * 16384 + (size_t)(u >> 3) * 1024 + (size_t)(u & 7) * 128;
                uint32_t w[32];
#pragma unroll
                for (int c = 0; c < 8; ++c) {
                    const uint4 v = *reinterpret_cast<const uint4 *>(row + ((c ^ (u & 7)) << 4));
                    w[4 * c + 0] = v.x;
                    w[4 * c + 1] = v.y;
                    w[4 * c + 2] = v.z;
                    w[4 * c + 3] = v.w;
                }
                tc::tmem_st32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(a.r_tmem_col + i * 32), w);
            }
            tc::tmem_st_wait();
            tc::tc_fence_before_sync();
            tc::mbar_arrive(r_ready);
        }
        ok = tc::mbar_wait(h_full, 0, WAIT_BUDGET) && ok;
        // The W*x+bw values of a chunk come from HBM (a microsecond away under load) and a warp issues in
        // order, so they are fetched one chunk AHEAD: while the warp works on a chunk, the six values of
        // its next chunk (next sub-group or next step) are already in flight into registers.
        struct Pre { int32_t g[4], n[2]; };
        auto fetch = [&](int s_, int g_, int c_, Pre &pr) {
            const int t_ = a.reverse ? (a.T - 1 - s_) : s_;
            const int bg = b0 + g_ * a.NB;
            const int nb_ = max(0, min(a.NB, a.b_off + a.b_cnt - bg));
            const int c0_ = 4 * c_, f0_ = c0_ + 2 * half;
            const IhT *rowp = ihp + ((size_t)t_ * a.B + bg) * a.C + j;
#pragma unroll
            for (int i = 0; i < 4; ++i)
                pr.g[i] = ld_ih_pred(rowp + (size_t)(c0_ + i) * a.C + half * a.H, c0_ + i < nb_ && j_ok);
#pragma unroll
            for (int k = 0; k < 2; ++k)
                pr.n[k] = ld_ih_pred(rowp + (size_t)(f0_ + k) * a.C + 2 * a.H, f0_ + k < nb_ && j_ok);
        };
        Pre cur, nxt;
        fetch(0, 0, rank, cur);
        for (int s = 0; s < a.T; ++s) {
            const long long out_slot = a.reverse ? (a.T - 1 - s) : (s + 1);
            const uint32_t par = (uint32_t)(s & 1);
            for (int g = 0; g < NG; ++g) {
                const int bg0 = b0 + g * a.NB;
                const int nb = max(0, min(a.NB, a.b_off + a.b_cnt - bg0));
                const unsigned char *h_cur = h_tile + (size_t)(2 * g + (s & 1)) * h_buf_bytes;
                uint64_t *md = &mma_done[2 * g];
                const uint32_t nbuf = (uint32_t)(2 * g + ((s + 1) & 1));
                const uint32_t bar_nx = bar_u32 + 8u * nbuf;
                bool waited = false;
                int32_t hn_last[2] = {0, 0};
                int f_last = -1;
                for (int c = rank; c < nchunks && ok; c += EPW) {
                    const int c0 = 4 * c;
                    const int f0 = c0 + 2 * half;      // the two batch columns this lane finishes
                    // the next chunk's W*x+bw values start their way now
                    {
                        int s2 = s, g2 = g, c2 = c + EPW;
                        if (c2 >= nchunks) {
                            c2 = rank;
                            if (++g2 == NG) {
                                g2 = 0;
                                ++s2;
                            }
                        }
                        if (s2 < a.T) fetch(s2, g2, c2, nxt);
                    }
                    STAMP((warp % 15) == 1 && lane == 0, 13 + 8 * (warp / 15));
                    int32_t hold[2];
#pragma unroll
                    for (int k = 0; k < 2; ++k) {
                        const bool v_ok = f0 + k < nb && j_ok;
                        const uint8_t hb = v_ok ? h_cur[sw128_offset(f0 + k, j, a.NB)] : (uint8_t)0;
                        hold[k] = state_byte(hb, h_bits);
                    }
                    STAMP((warp % 15) == 1 && lane == 0, 14 + 8 * (warp / 15));
                    const int32_t(&ihg)[4] = cur.g;
                    const int32_t(&ihn)[2] = cur.n;
                    const uint32_t ta0 = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(2 * g * a.k_parts * a.NB + c0);
                    // update gate (lanes 0-15) and reset gate (lanes 16-31) of four batch columns
                    if (!waited) {
                        ok = tc::mbar_wait(&md[0], par, WAIT_BUDGET);
                        if (!ok) break;
                        tc::tc_fence_after_sync();
                    }
                    STAMP((warp % 15) == 1 && lane == 0 && !waited, 8 + 8 * (warp / 15));
                    int32_t acc[4], gd[4];
                    tc::tmem_ld4(ta0, acc);
                    if (a.k_parts == 2) {   // the other K half
                        int32_t hi[4];
                        tc::tmem_ld4(ta0 + (uint32_t)a.NB, hi);
                        tc::tmem_ld_wait();
#pragma unroll
                        for (int i = 0; i < 4; ++i) acc[i] += hi[i];
                    }
                    tc::tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 4; ++i)
                        gd[i] = lookup(tab, ihg[i] + lookup(tab, lin_round<Tie>(acc[i], fl_g), hc_c, hc_lo, hc_hi), gt_c, gt_lo, gt_hi);
                    // the partner finishes the other two columns: it gets this lane's gate value of those
                    const int32_t rc0 = __shfl_xor_sync(0xffffffffu, half ? gd[0] : gd[2], 16);
                    const int32_t rc1 = __shfl_xor_sync(0xffffffffu, half ? gd[1] : gd[3], 16);
                    const int32_t zd0 = half ? rc0 : gd[0], zd1 = half ? rc1 : gd[1];
                    const int32_t rd0 = half ? gd[2] : rc0, rd1 = half ? gd[3] : rc1;
                    // new gate: its sums sit in lanes 0-15; lanes 16-31 receive those of their two columns
                    if (!waited) {
                        ok = tc::mbar_wait(&md[1], par, WAIT_BUDGET);
                        if (!ok) break;
                        tc::tc_fence_after_sync();
                        waited = true;
                    }
                    STAMP((warp % 15) == 1 && lane == 0, 9 + 8 * (warp / 15));
                    tc::tmem_ld4(ta0 + (uint32_t)(a.k_parts * a.NB), acc);
                    if (a.k_parts == 2) {
                        int32_t hi[4];
                        tc::tmem_ld4(ta0 + (uint32_t)(3 * a.NB), hi);
                        tc::tmem_ld_wait();
#pragma unroll
                        for (int i = 0; i < 4; ++i) acc[i] += hi[i];
                    }
                    tc::tmem_ld_wait();
                    const int32_t s2 = __shfl_xor_sync(0xffffffffu, acc[2], 16);
                    const int32_t s3 = __shfl_xor_sync(0xffffffffu, acc[3], 16);
                    const int32_t an0 = half ? s2 : acc[0], an1 = half ? s3 : acc[1];
                    int32_t hn[2];
                    hn[0] = fused_finish_fast<Tie>(gc, tab, ihn[0], lin_round<Tie>(an0, fl_n), zd0, rd0, hold[0]);
                    hn[1] = fused_finish_fast<Tie>(gc, tab, ihn[1], lin_round<Tie>(an1, fl_n), zd1, rd1, hold[1]);
                    // h_t[b][j] = element (row b, K index j) of the next B tile: gather the bytes of four
                    // consecutive units of one row into a word, store it into this CTA's tile and send it
                    // to the peers' (absent rows and units travel too: the peers count on every byte)
                    if (s + 1 < a.T) {
                        const uint32_t pk = ((uint32_t)hn[0] & 0xffu) | (((uint32_t)hn[1] & 0xffu) << 8);
                        const uint32_t v0 = __shfl_sync(0xffffffffu, pk, x_src + 0);
                        const uint32_t v1 = __shfl_sync(0xffffffffu, pk, x_src + 1);
                        const uint32_t v2 = __shfl_sync(0xffffffffu, pk, x_src + 2);
                        const uint32_t v3 = __shfl_sync(0xffffffffu, pk, x_src + 3);
                        const uint32_t word = __byte_perm(__byte_perm(v0, v1, x_sel), __byte_perm(v2, v3, x_sel), 0x5410);
                        const uint32_t at = tile_u32 + nbuf * h_buf_bytes + sw128_offset(c0 + x_rr, j0 + 16 * q + 4 * x_w, a.NB);
                        if (half == 0) sts_u32(at, word);
                        for (int r = half; r < a.P; r += 2)
                            if (r != p) st_async_u32(map_to_rank(at, (uint32_t)r), word, map_to_rank(bar_nx, (uint32_t)r));
                    }
                    const bool last = c + EPW >= nchunks;
                    if (!last) {
#pragma unroll
                        for (int k = 0; k < 2; ++k)
                            if (f0 + k < nb && j_ok) {
                                const size_t o = (size_t)out_slot * BH + (size_t)(bg0 + f0 + k) * a.H + j;
                                if (a.hq_out) a.hq_out[o] = hn[k];
                                if (a.hf_out) a.hf_out[o] = (float)(hn[k] - gc.zp_h) * gc.h_scale;
                                if (a.h8_out) a.h8_out[o] = (uint8_t)hn[k];
                            }
                    } else {
                        hn_last[0] = hn[0];
                        hn_last[1] = hn[1];
                        f_last = f0;
                    }
                    cur = nxt;
                }
                if (ok && !waited) {
                    // a warp without a chunk still waits for this step's MMAs: it must not arrive twice
                    // within one phase of the tile barrier
                    ok = tc::mbar_wait(&md[1], par, WAIT_BUDGET);
                    tc::tc_fence_after_sync();
                }
                fence_proxy_async_cta();   // this warp's own words, for the MMAs' async-proxy reads
                tc::tc_fence_before_sync();
                __syncwarp();
                STAMP((warp % 15) == 1 && lane == 0, 10 + 8 * (warp / 15));
                if (lane == 0 && s + 1 < a.T) tc::mbar_arrive(&h_ready[nbuf]);
                STAMP((warp % 15) == 1 && lane == 0, 11 + 8 * (warp / 15));
                // outputs of the warp's last chunk leave after the arrive: nothing in the next step waits for them
                if (f_last >= 0) {
#pragma unroll
                    for (int k = 0; k < 2; ++k)
                        if (f_last + k < nb && j_ok) {
                            const size_t o = (size_t)out_slot * BH + (size_t)(bg0 + f_last + k) * a.H + j;
                            if (a.hq_out) a.hq_out[o] = hn_last[k];
                            if (a.hf_out) a.hf_out[o] = (float)(hn_last[k] - gc.zp_h) * gc.h_scale;
                            if (a.h8_out) a.h8_out[o] = (uint8_t)hn_last[k];
                        }
                }
                STAMP((warp % 15) == 1 && lane == 0, 12 + 8 * (warp / 15));
            }
        }
        if (!ok && lane == 0) atomicOr(a.abort_flag, 1);
    }
    tc::tc_fence_before_sync();
    __syncthreads();
    // nobody leaves while a peer's store into its shared memory may be in flight
    cluster_arrive();
    cluster_wait();
    if (warp == 0) tc::tmem_dealloc(tmem_base, tmem_cols);
}

template <typename IhT, bool Tie>
cudaError_t launch64(const CUtensorMap &mr, const CUtensorMap &mh, const GateConsts &gc, RecMmaArgs &a, int grid,
                     size_t smem, cudaStream_t st) {
    auto kern = k_recurrence_c64<IhT, Tie>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(REC_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)a.P;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kern, mr, mh, gc, a);
}

}  // namespace

// 64 units per CTA: H <= 512 (clusters of up to 8), two sub-groups of NB rows per CTA.
// `force`: take it whenever it fits; otherwise only where a cluster ends up with few rows (the
// latency-bound regime it was written for).
bool rec_c64_plan(int H, int Hpad, int B, int sms, int smem_optin, int n_table, bool force, RecMmaPlan *out) {
    if (Hpad > 512) return false;
    const int KBn = Hpad / 128;
    const int P = (H + UT - 1) / UT;
    if (P > 8 || P > sms) return false;
    const int groups_max = std::max(1, sms / P);
    const int NG = 2;
    int RC = ((B + groups_max - 1) / groups_max + 31) / 32 * 32;   // rows per cluster: two sub-groups of 16 x
    RC = std::max(RC, 32);
    if (!force && (RC > 64 || P < 3)) return false;
    int NB = RC / NG;
    if (NB > 48) return false;                                      // beyond 48 columns an MMA gets slower: no point
    const size_t smem = smem64_layout(KBn, NB, NG, n_table).total + 1024;
    if (smem > (size_t)smem_optin) return false;
    // two K halves per tile, each with an issuing warp and accumulator columns of its own, where K has
    // two slabs and tensor memory has the room
    int k_parts = KBn >= 2 ? 2 : 1;
    if ((NG * 2 * k_parts * NB + 31) / 32 * 32 + 2 * KBn * 32 > 512) k_parts = 1;
    const int acc_cols = (NG * 2 * k_parts * NB + 31) / 32 * 32;
    uint32_t cols = 32;
    while ((int)cols < acc_cols + 2 * KBn * 32) cols <<= 1;
    if (cols > 512) return false;
    out->MT = 1;
    out->P = P;
    out->NB = NB;
    out->NG = NG;
    out->G = (B + NB * NG - 1) / (NB * NG);
    out->smem = smem;
    out->tmem_cols = (int)cols;
    out->r_tmem_col = acc_cols;
    out->tmem_tiles = 2 * KBn;
    out->r_slots = 2 * KBn;
    out->k_parts = k_parts;
    out->groups_per_launch = out->G;
    return true;
}

int rec_c64_launch(RecMmaState &s, const RecMmaPlan &pl, RecMmaArgs a, const GateConsts &gc_host, const int8_t *r8,
                   long long r_rows_alloc, long long h_rows_alloc, bool h_unsigned, int ih_bytes, bool notie,
                   cudaStream_t stream, std::string *err) {
    if (r_rows_alloc < a.C + 144) {
        if (err) *err = "packed R lacks the zero rows the 64-unit recurrence reads";
        return QGRU_ERR_UNSUPPORTED;
    }
    if (!s.valid || s.r8 != r8 || s.h8 != a.h8 || s.r_rows != r_rows_alloc || s.h_rows != h_rows_alloc ||
        s.Hpad != a.Hpad || s.NB != pl.NB) {
        if (!make_map_u8_sw128(reinterpret_cast<CUtensorMap *>(s.map_r), r8, (uint64_t)r_rows_alloc, (uint64_t)a.Hpad, 16) ||
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
    const CUtensorMap &mr = *reinterpret_cast<const CUtensorMap *>(s.map_r);
    const CUtensorMap &mh = *reinterpret_cast<const CUtensorMap *>(s.map_h);
    a.P = pl.P;
    a.NB = pl.NB;
    a.NG = pl.NG;
    a.h_unsigned = h_unsigned ? 1 : 0;
    a.tmem_cols = (uint32_t)pl.tmem_cols;
    a.r_tmem_col = pl.r_tmem_col;
    a.tmem_tiles = pl.tmem_tiles;
    a.r_slots = pl.r_slots;
    a.k_parts = pl.k_parts;
    a.b_off = 0;
    a.b_cnt = a.B;
    const int grid = pl.G * pl.P;
    const cudaError_t e =
        notie ? (ih_bytes == 2 ? launch64<int16_t, false>(mr, mh, gc_host, a, grid, pl.smem, stream)
                               : launch64<int32_t, false>(mr, mh, gc_host, a, grid, pl.smem, stream))
              : (ih_bytes == 2 ? launch64<int16_t, true>(mr, mh, gc_host, a, grid, pl.smem, stream)
                               : launch64<int32_t, true>(mr, mh, gc_host, a, grid, pl.smem, stream));
    if (e != cudaSuccess) {
        if (err) *err = std::string("recurrence (64-unit cluster) launch: ") + cudaGetErrorString(e);
        cudaGetLastError();
        return QGRU_ERR_CUDA;
    }
    ++s.launches;
    return QGRU_OK;
}

}  // namespace qgru
