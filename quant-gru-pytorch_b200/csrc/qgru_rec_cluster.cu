// qgru_rec_cluster.cu - the tensor-core recurrence with the state exchanged through distributed
// shared memory.
//
// Same work split as k_recurrence_mma (qgru_rec_mma.cu): a CTA owns 128*MT hidden units of one
// group of NB batch rows and keeps its slice of R in shared memory for all T steps.  Here the P
// CTAs of a group form one thread-block cluster and h_t never leaves the SMs.  The 128 units of
// CTA p are exactly K-slab p of the B-operand tile (NB rows x 128 bytes, 128-byte swizzle), a
// contiguous NB*128-byte block.  Each epilogue warp transposes its 4 rows x 32 units of 8-bit h_t
// through shuffles into one 32-bit word per lane, stores the word into its OWN tile and sends
// it to the same place of every peer's tile with st.async, a store that counts its bytes on the
// peer's mbarrier when it lands.  A CTA starts the MMAs of a step when its 16 warps have arrived
// and the P-1 peer blocks have landed: no relay through one thread, no cluster-wide barrier,
// no fence on the sending side, no global-memory round trip.  Only the outputs go to global
// memory.
//
// The tile is double buffered: step s multiplies buffer s&1 while the blocks of h_{s+1} land in
// buffer (s+1)&1.  A peer can never be more than one step ahead (its MMAs of step s+1 need this
// CTA's block of h_{s+1}), which is what makes two buffers enough.  Step 0's state is loaded
// from global memory by TMA.
//
// A CTA may own NG independent sub-groups of NB batch rows each (NG = 2: "A" and "B").  Each has
// its own accumulators, state tiles and barriers; the control thread issues the MMAs of A then
// B, the epilogue warps work on A then B, so that B's MMAs run on the tensor pipe while the
// warps are busy with A's cells and A's next MMAs while they are busy with B's: the two halves
// of a step, which are serial for one group (exchange -> MMAs -> cells), overlap.
//
// Three warps issue the MMAs, one per gate.  A single thread issues a chain of these small MMAs at
// one per 53-80 cycles, while the tensor pipe takes MMAs from several threads side by side
// (qgru_probe_mma_i8_ex): the 48 MMAs of a step at H = 512 take 1700 cycles instead of 3900 (about
// 115 bytes of R per cycle; the same 48 MMAs from three issuers take 850 cycles in the probe, and
// six issuers, one per gate and K half, were measured no faster here).  Each issuer commits
// once per step: a commit holds its thread until the MMAs before it are done, so a thread that
// commits gate by gate serialises the gates (measured; the form with one issuer per K half and
// accumulator columns of its own, k_parts = 2, is kept for experiments).  The reset and new
// gates' issuers start a little after the update gate's, so that the update gate, which the cells
// need first, gets the head of the stream.
#include <cuda.h>
#include <cuda_runtime.h>

#include "qgru_cluster.cuh"
#include "qgru_device.cuh"
#include "qgru_rec_mma.cuh"
#include "qgru_tc.cuh"

#ifdef QGRU_STAMPS
#define STAMP(cond, slot) do { if (a.dbg && blockIdx.x == 0 && (cond)) a.dbg[((size_t)s * 2 + g) * 8 + (slot)] = clock64(); } while (0)
#else
#define STAMP(cond, slot) do { } while (0)
#endif

namespace qgru {
using namespace clu;
namespace {

constexpr long long WAIT_BUDGET = 2000000000ll;  // ~1 s of SM clocks
constexpr int EPW = 4;                           // epilogue warps per TMEM lane quadrant
constexpr int EPI_THREADS = 32 * 4 * EPW;
constexpr int ISSUERS = 3;                       // warp 0 and the two warps after the epilogue warps
constexpr int REC_THREADS = 32 * ISSUERS + EPI_THREADS;
constexpr int CH = 4;                            // batch columns per chunk

}  // namespace

struct ClusterSmem {
    size_t r_tiles, h_tile, bars, tables, h_priv, total;
};

// r_slots: 16 KB tile slots for R (staging on the way to tensor memory, then home of the tiles
// that stay in shared memory)
__host__ __device__ inline ClusterSmem cluster_smem_layout(int r_slots, int KBn, int NB, int NG, int n_table) {
    ClusterSmem s;
    s.r_tiles = 0;
    s.h_tile = (size_t)r_slots * 16384;
    s.bars = s.h_tile + (size_t)NG * 2 * KBn * NB * 128;   // two state buffers per sub-group
    s.tables = s.bars + 256;
    s.h_priv = s.tables + (((size_t)n_table * 4 + 15) & ~size_t(15));
    // warps with several chunks of cells per step keep the state of their own cells here, one word
    // (four row bytes of the thread's unit) per chunk and thread: [chunks per warp][EPI_THREADS]
    const int chunks = NB / CH;
    s.total = s.h_priv + ((NG == 1 && chunks > EPW) ? (size_t)((chunks + EPW - 1) / EPW) * EPI_THREADS * 4 : 0);
    return s;
}


namespace {

// MMA issue for wide hidden sizes (512 < H <= 1024): the tiles of a gate come partly from tensor
// memory, partly from their shared-memory slots.  Rolled loops (the fully unrolled form of these
// 96 MMAs measured slower) in a function of its own, so that its registers do not weigh on the
// kernel's common path.
__device__ __noinline__ void issue_wide(int MT, int KBn, int NB, int tmem_tiles, uint32_t tmem_base, uint32_t r_t0,
                                        uint32_t r_lo0, uint32_t hb0, uint32_t desc_lo, uint64_t dhi, uint32_t idesc,
                                        uint64_t *mma_done, int KP, int part, int kb0, int kb1, int gate_lo, int gate_hi) {
    for (int g = gate_lo; g < gate_hi; ++g) {
        for (int mt = 0; mt < MT; ++mt) {
            const uint32_t d = tmem_base + (uint32_t)(((mt * 3 + g) * KP + part) * NB);
            for (int kb = kb0; kb < kb1; ++kb) {
                const int tile = (mt * 3 + g) * KBn + kb;
                const uint32_t bd = hb0 + (uint32_t)(kb * NB * 8);
                if (tile < tmem_tiles) {
                    const uint32_t ra = r_t0 + (uint32_t)(tile * 32);
#pragma unroll
                    for (int ks = 0; ks < 4; ++ks)
                        tc::mma_i8_ts(d, ra + (uint32_t)(ks * 8), dhi | (bd + 2 * ks), idesc, (kb != kb0 || ks != 0) ? 1u : 0u);
                } else {
                    const uint32_t rb = desc_lo | (r_lo0 + (uint32_t)((tile - tmem_tiles) * 1024));
#pragma unroll
                    for (int ks = 0; ks < 4; ++ks)
                        tc::mma_i8(d, dhi | (rb + (uint32_t)(2 * ks)), dhi | (bd + 2 * ks), idesc, (kb != kb0 || ks != 0) ? 1u : 0u);
                }
            }
        }
        tc::mma_commit(&mma_done[g]);
    }
}

constexpr int MAX_NG = 2;                        // sub-groups of batch rows per CTA

// Cell variants: Fused = false: the generic datapath (Narrow picks its 32-bit rescales);
// Fused = true: the tabulated cell, where Narrow = true selects the branch-free form that needs
// every scale of the step in shift-free form and 32-bit linear sums.
// Floor = true is a measurement aid: the same launch, barriers, state exchange and output stores
// with the MMAs and the cell left out (h_t = h_{t-1}); its duration is the synchronisation floor
// the real kernel's time per step is quoted against.
// Tie = false (branch-free tabulated cell only): the rescales round half up, which equals the
// reference's round-half-even because none of them can meet an exact tie (rescale_can_tie).
template <typename IhT, bool Narrow, bool Fused, int MT, bool Floor, bool Tie, bool Priv>
__global__ void __launch_bounds__(REC_THREADS, 1)
k_recurrence_cluster(const __grid_constant__ CUtensorMap map_r, const __grid_constant__ CUtensorMap map_h,
                     const __grid_constant__ GateConsts gc, RecMmaArgs a) {
    extern __shared__ unsigned char smem_raw[];
    // every CTA of the cluster must compute the same offsets: the dynamic shared window starts at
    // the same shared address in all of them, so the aligned base is the same too
    const uint32_t raw = tc::smem_u32(smem_raw);
    unsigned char *base = smem_raw + (((raw + 1023u) & ~1023u) - raw);
    const int KBn = a.Hpad >> 7;
    const int NG = a.NG;
    const ClusterSmem L = cluster_smem_layout(a.r_slots, KBn, a.NB, NG, a.n_table);
    unsigned char *r_tiles = base + L.r_tiles;
    unsigned char *h_tile = base + L.h_tile;                  // [NG][2 buffers][KBn slabs][NB rows][128 bytes]
    const uint32_t h_buf_bytes = (uint32_t)(KBn * a.NB * 128);
    uint64_t *bars = reinterpret_cast<uint64_t *>(base + L.bars);
    uint64_t *r_full = bars, *h_full = bars + 1, *r_ready = bars + 2;
    uint64_t *h_ready = bars + 3;                    // [NG][2]: the tile buffer holds h_t of every CTA of the cluster
    uint64_t *mma_done = bars + 3 + 2 * MAX_NG;      // [NG][3]: the rows of gate z / r / n are accumulated
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 3 + 5 * MAX_NG);
    int32_t *tables = reinterpret_cast<int32_t *>(base + L.tables);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, tid = threadIdx.x;
    const int grp = blockIdx.x / a.P;
    const int p = (int)cluster_rank();               // == blockIdx.x % P: clusters are P consecutive CTAs
    const int j0 = p * 128 * MT;
    const int b0 = a.b_off + grp * NG * a.NB;        // first batch row of the cluster; sub-group g starts NB * g later
    const uint32_t tmem_cols = a.tmem_cols;
    const int KP = a.k_parts;                                      // K halves with accumulators of their own
    const uint32_t acc_cols_g = (uint32_t)(MT * 3 * KP * a.NB);   // accumulator columns of one sub-group

    for (int i = tid; i < a.n_table; i += blockDim.x) tables[i] = a.tables[i];
    if (tid == 0) {
        tc::mbar_init(r_full, 1);
        tc::mbar_init(h_full, 1);
        for (int g = 0; g < 3 * NG; ++g) tc::mbar_init(&mma_done[g], (uint32_t)KP);   // one commit per K half
        // per phase: one arrival per epilogue warp, one by the control thread (which also announces
        // the bytes the peers send)
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
    // no CTA may receive a peer's block before its barriers are initialised
    cluster_arrive();
    cluster_wait();

    if (warp == 0 || warp > 4 * EPW) {
        // ------------------------------------------------------------------ issuing warps
        // k_parts == 1: issuer w multiplies the rows of gate w.  k_parts == 2: issuers 0 and 1 multiply one
        // half of K each, for every gate.  Issuer 0 also loads R and the initial state and announces the
        // peers' bytes on the state barriers.
        const int iw = warp == 0 ? 0 : warp - 4 * EPW;
        const int part = KP == 2 ? iw : 0;
        const int gate_lo = KP == 2 ? 0 : iw, gate_hi = KP == 2 ? 3 : iw + 1;
        bool ok = true;
        uint32_t idesc = 0, r_lo0 = 0, h_lo0 = 0, desc_hi = 0, desc_lo = 0;
        if (lane == 0 && (KP == 1 || iw < 2)) {
            if (iw == 0) {
                // R slice: tiles [0, tmem_tiles) go to tensor memory through the slots, one pass of up to
                // r_slots tiles at a time (the epilogue threads copy a pass and hand the slots back);
                // the remaining tiles are then loaded into the slots to stay.
                const int n_tiles = MT * 3 * KBn;
                auto load_tiles = [&](int first, int cnt) {
                    tc::mbar_expect_tx(r_full, (uint32_t)cnt * 16384u);
                    for (int i = 0; i < cnt; ++i) {
                        const int t = first + i, mt = t / (3 * KBn), g = (t / KBn) % 3, kb = t % KBn;
                        tc::tma_load_2d(r_tiles + (size_t)i * 16384, &map_r, r_full, kb * 128, g * a.H + j0 + mt * 128);
                    }
                };
                int pass = 0;
                for (int done = 0; done < a.tmem_tiles && ok; ++pass) {
                    const int cnt = min(a.r_slots, a.tmem_tiles - done);
                    load_tiles(done, cnt);
                    ok = tc::mbar_wait(r_ready, (uint32_t)(pass & 1), WAIT_BUDGET);   // copied: slots free again
                    done += cnt;
                }
                if (ok && n_tiles > a.tmem_tiles) {
                    load_tiles(a.tmem_tiles, n_tiles - a.tmem_tiles);
                    ok = tc::mbar_wait(r_full, (uint32_t)(pass & 1), WAIT_BUDGET);
                }
                // the initial state (written by the preceding kernel) into buffer 0 of every sub-group; it
                // is requested after R is in place, so its arrival tells the other issuer that too
                tc::mbar_expect_tx(h_full, (uint32_t)NG * h_buf_bytes);
                for (int g = 0; g < NG; ++g)
                    for (int kb = 0; kb < KBn; ++kb)
                        tc::tma_load_2d(h_tile + (size_t)(2 * g) * h_buf_bytes + (size_t)kb * a.NB * 128, &map_h, h_full,
                                        kb * 128, b0 + g * a.NB);
            }
            ok = ok && tc::mbar_wait(h_full, 0, WAIT_BUDGET);
            tc::tc_fence_after_sync();
            idesc = tc::idesc_i8(128, a.NB, true, !a.h_unsigned);
            r_lo0 = (tc::smem_u32(r_tiles) & 0x3FFFFu) >> 4;
            h_lo0 = (tc::smem_u32(h_tile) & 0x3FFFFu) >> 4;
            desc_hi = (uint32_t)(tc::smem_desc_sw128(0) >> 32);
            desc_lo = (uint32_t)tc::smem_desc_sw128(0);
            if (!ok) atomicOr(a.abort_flag, 1);
            const uint32_t blk_bytes = (uint32_t)(a.NB * 128);           // one K-slab of the tile
            const int kb0 = part == 0 ? 0 : (KBn + 1) / 2;               // this issuer's K-slabs: [kb0, kb1)
            const int kb1 = (KP == 1 || part == 1) ? KBn : (KBn + 1) / 2;
            for (int s = 0; s < a.T && ok; ++s) {
                for (int g = 0; g < NG; ++g) {
                    const uint32_t buf = (uint32_t)(2 * g + (s & 1));
                    if (s > 0) {
                        // h_s in buffer s & 1: the 16 warps of this CTA have stored their words and the
                        // (P-1) * NB * 128 bytes of the peers have landed
                        if (iw == 0) tc::mbar_expect_tx(&h_ready[buf], (uint32_t)(a.P - 1) * blk_bytes);
                        if (!tc::mbar_wait(&h_ready[buf], (uint32_t)(((s - 1) >> 1) & 1), WAIT_BUDGET)) { ok = false; break; }
                        fence_proxy_async_cta();   // the MMAs read these stores through the async proxy
                    }
                    tc::tc_fence_after_sync();
                    STAMP(iw == 0, 0);
                    uint64_t *md = &mma_done[3 * g];
                    if constexpr (Floor) {
                        for (int k = gate_lo; k < gate_hi; ++k) tc::mma_commit(&md[k]);
                        continue;
                    }
                    if (KP == 1 && iw > 0 && a.issue_delay > 0) {
                        // the update gate's MMAs get a head start on the tensor pipe (bounded: a fixed number of cycles)
                        const long long until = clock64() + (long long)iw * a.issue_delay;
                        while (clock64() < until) {
                        }
                    }
                    const uint32_t hbuf = h_lo0 + ((buf * h_buf_bytes) >> 4);
                    const uint32_t acc0 = tmem_base + (uint32_t)g * acc_cols_g;
                    const uint64_t dhi = (uint64_t)desc_hi << 32;
                    const uint32_t r_t0 = tmem_base + (uint32_t)a.r_tmem_col;
                    if (KBn <= 4 && (a.tmem_tiles == 0 || a.tmem_tiles == MT * 3 * KBn)) {
                        // the common shapes (H <= 512, R in one place): fully unrolled, one independent add per MMA
                        uint32_t bdl[4][4];   // low descriptor words of the state tile: K-slab kb, 32-byte step ks
#pragma unroll
                        for (int kb = 0; kb < 4; ++kb)
#pragma unroll
                            for (int ks = 0; ks < 4; ++ks) bdl[kb][ks] = desc_lo | (hbuf + (uint32_t)(kb * a.NB * 8 + 2 * ks));
#pragma unroll
                        for (int gate = 0; gate < 3; ++gate) {
                            if (gate < gate_lo || gate >= gate_hi) continue;
                            if (a.tmem_tiles > 0) {   // A operand from tensor memory
#pragma unroll
                                for (int mt = 0; mt < MT; ++mt) {
                                    const uint32_t d = acc0 + (uint32_t)(((mt * 3 + gate) * KP + part) * a.NB);
                                    const uint32_t ra = r_t0 + (uint32_t)((mt * 3 + gate) * KBn * 32);
#pragma unroll
                                    for (int kb = 0; kb < 4; ++kb)
                                        if (kb >= kb0 && kb < kb1) {
#pragma unroll
                                            for (int ks = 0; ks < 4; ++ks)
                                                tc::mma_i8_ts(d, ra + (uint32_t)(kb * 32 + ks * 8), dhi | bdl[kb][ks], idesc,
                                                              (kb != kb0 || ks != 0) ? 1u : 0u);
                                        }
                                }
                            } else {
#pragma unroll
                                for (int mt = 0; mt < MT; ++mt) {
                                    const uint32_t d = acc0 + (uint32_t)(((mt * 3 + gate) * KP + part) * a.NB);
                                    const uint32_t rb = desc_lo | (r_lo0 + (uint32_t)((mt * 3 + gate) * KBn * 1024));
#pragma unroll
                                    for (int kb = 0; kb < 4; ++kb)
                                        if (kb >= kb0 && kb < kb1) {
#pragma unroll
                                            for (int ks = 0; ks < 4; ++ks)
                                                tc::mma_i8(d, dhi | (rb + (uint32_t)(kb * 1024 + 2 * ks)), dhi | bdl[kb][ks], idesc,
                                                           (kb != kb0 || ks != 0) ? 1u : 0u);
                                        }
                                }
                            }
                            tc::mma_commit(&md[gate]);
                        }
                    } else {
                        issue_wide(MT, KBn, a.NB, a.tmem_tiles, acc0, r_t0, r_lo0, desc_lo | hbuf, desc_lo, dhi, idesc, md, KP,
                                   part, kb0, kb1, gate_lo, gate_hi);
                    }
                    STAMP(iw == 0, 1);
                }
            }
            if (!ok) atomicOr(a.abort_flag, 1);
        }
    } else {
        // ---------------------------------------------------------------- epilogue warps (1 .. 16)
        const int q = warp & 3;                      // TMEM lane quadrant this warp may read
        const int rank = (warp - 1) >> 2;            // 0..EPW-1 among the warps of that quadrant
        const int u = q * 32 + lane;                 // unit within a 128-unit tile = TMEM lane
        const size_t BH = (size_t)a.B * a.H;
        const IhT *ihp = reinterpret_cast<const IhT *>(a.ih);
        const int nchunks = a.NB / CH;
        const uint32_t tab = tc::smem_u32(tables);          // fused-cell tables, shared-window address
        const uint32_t h_bits = a.h_unsigned ? 9u : 8u;     // state bytes: zero- or sign-extended
        // Exchange: after the shuffle transposition lane t holds the word (row t >> 3 of the chunk,
        // units 4 * (t & 7) .. + 3 of this warp's 32); source lanes, byte selector and the peers'
        // tile / barrier addresses are fixed for the whole launch.
        static_assert(CH == 4, "the exchange packs four row bytes per lane");
        const int x_row = lane >> 3, x_word = lane & 7;
        const uint32_t x_sel = (uint32_t)x_row | ((uint32_t)(4 + x_row) << 4);
        const uint32_t tile_u32 = tc::smem_u32(h_tile);
        const uint32_t bar_u32 = tc::smem_u32(h_ready);
        int64_t corr[MT][3];
        Rescale rs[MT][3];
        FastLin fl[MT][3];
        bool j_ok[MT];
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
            const int j = j0 + mt * 128 + u;
            j_ok[mt] = j < a.H;
#pragma unroll
            for (int g = 0; g < 3; ++g) {
                corr[mt][g] = j_ok[mt] ? a.lc.corr[g * a.H + j] : 0;
                rs[mt][g] = j_ok[mt] ? a.lc.rs[g * a.H + j] : Rescale{1, 1, 0, 0, 0, 0, 0, 0};
                fl[mt][g] = j_ok[mt] ? a.lc.fl[g * a.H + j] : FastLin{0, 0, 0, 0, 0, 0};
            }
        }
        // float-storage forward: offset, bias term and scale ratio of this thread's three R*h rows
        float fsk[MT][3][3];
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int g = 0; g < 3; ++g)
#pragma unroll
                for (int k = 0; k < 3; ++k)
                    fsk[mt][g][k] = (a.fs_on && j_ok[mt]) ? a.fs_chan[(size_t)k * a.C + g * a.H + j0 + mt * 128 + u] : 0.f;
        bool ok = true;
        {
            // Move tiles [0, tmem_tiles) of the R slice from their TMA-written slots into tensor
            // memory, where the MMA reads its A operand without touching shared memory.  This thread
            // owns row u of every 128-row tile: eight 16-byte chunks per 128-byte row, un-swizzled
            // on the way (chunk c of row u lies at chunk c ^ (u & 7)), written to 32 columns of TMEM
            // lane u.  One pass per refill of the slots.
            int pass = 0;
            for (int done = 0; done < a.tmem_tiles && ok; ++pass) {
                const int cnt = min(a.r_slots, a.tmem_tiles - done);
                ok = tc::mbar_wait(r_full, (uint32_t)(pass & 1), WAIT_BUDGET);
                for (int i = rank; i < cnt && ok; i += EPW) {
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
                    tc::tmem_st32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(a.r_tmem_col + (done + i) * 32), w);
                }
                tc::tmem_st_wait();
                tc::tc_fence_before_sync();
                tc::mbar_arrive(r_ready);
                done += cnt;
            }
        }
        // the TMA-written initial state must be complete before h_{t-1} is read from the tile
        ok = tc::mbar_wait(h_full, 0, WAIT_BUDGET) && ok;
        // A warp with one chunk per step (NB <= 4 * EPW rows, one sub-group) computes the same cells every
        // step, so h_{t-1} of its cells is what it produced a step ago: kept in registers, not read back
        // from the state tile (one byte load with its swizzled address per cell).
        const bool keep_h = NG == 1 && nchunks <= EPW;
        // With several chunks per step the same holds per chunk, and the four bytes go through a private
        // word of shared memory per chunk and thread instead: one conflict-free 32-bit load and four
        // byte extracts against four byte loads at swizzled addresses of the state tile.
        // (an instance of its own, template Priv: the one-chunk-per-warp instances carry none of this)
        const bool priv_h = Priv && MT == 1 && NG == 1 && nchunks > EPW;
        uint32_t *h_priv = reinterpret_cast<uint32_t *>(base + L.h_priv) + (tid - 32);
        // byte extract of row i: zero-extended (unsigned state) or with the sign replicated
        const uint32_t priv_sel = a.h_unsigned ? 0x4440u : 0x8880u;
        int32_t h_keep[MT][CH];
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int i = 0; i < CH; ++i) h_keep[mt][i] = 0;
        // the CH cells of a chunk to whichever outputs the caller asked for: the choice is made once
        // per chunk, not per cell; `base` is the element offset of (time slot, first row of the sub-group)
        auto store_outputs = [&](const int32_t(&v)[MT][CH], int c0, int nb, size_t base) {
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
                if (!j_ok[mt]) continue;
                const uint32_t oj = (uint32_t)(c0 * a.H + j0 + mt * 128 + u);
                if (a.hf_out) {
                    float *o = a.hf_out + base;
#pragma unroll
                    for (int i = 0; i < CH; ++i)
                        if (c0 + i < nb) o[oj + (uint32_t)(i * a.H)] = (float)(v[mt][i] - gc.zp_h) * gc.h_scale;
                }
                if (a.hq_out) {
                    int32_t *o = a.hq_out + base;
#pragma unroll
                    for (int i = 0; i < CH; ++i)
                        if (c0 + i < nb) o[oj + (uint32_t)(i * a.H)] = v[mt][i];
                }
                if (a.h8_out) {
                    uint8_t *o = a.h8_out + base;
#pragma unroll
                    for (int i = 0; i < CH; ++i)
                        if (c0 + i < nb) o[oj + (uint32_t)(i * a.H)] = (uint8_t)v[mt][i];
                }
            }
        };
        for (int s = 0; s < a.T; ++s) {
            const int t = a.reverse ? (a.T - 1 - s) : s;
            const long long out_slot = a.reverse ? (a.T - 1 - s) : (s + 1);
            const uint32_t par = (uint32_t)(s & 1);
            for (int g = 0; g < NG; ++g) {
            const int bg0 = b0 + g * a.NB;                                   // first batch row of this sub-group
            const int nb = max(0, min(a.NB, a.b_off + a.b_cnt - bg0));     // its rows that exist
            const unsigned char *h_cur = h_tile + (size_t)(2 * g + (s & 1)) * h_buf_bytes;
            // this step's rows of W*x+bw and of the outputs: one warp-uniform base each, 32-bit offsets
            // per cell (a sub-group's rows of one step span far less than 2^32 elements)
            const IhT *ih_s = ihp + ((size_t)t * a.B + bg0) * a.C;
            const size_t out_base = (size_t)out_slot * BH + (size_t)bg0 * a.H;
            const bool from_regs = keep_h && s > 0;
            const bool from_priv = priv_h && s > 0;
            int kc = 0;   // ordinal of the chunk among this warp's chunks
            uint64_t *md = &mma_done[3 * g];
            bool waited = false;
            int32_t hn_last[MT][CH];   // the warp's last chunk: its outputs go to global memory after the arrive
            int c_last = -1;
            for (int c = rank; c < nchunks && ok; c += EPW) {
                const int c0 = c * CH;
                // operands that do not depend on this step's MMA: issued first
                int32_t ihv[MT][CH][3];
                int32_t hold[MT][CH];
                const uint32_t priv_word = from_priv ? h_priv[kc * EPI_THREADS] : 0u;
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
                    const int j = j0 + mt * 128 + u;
#pragma unroll
                    for (int i = 0; i < CH; ++i) {
                        const int b = c0 + i;
                        const bool v_ok = b < nb && j_ok[mt];
                        const uint32_t off = (uint32_t)(b * a.C + j);
#pragma unroll
                        for (int k = 0; k < 3; ++k)
                            ihv[mt][i][k] = (v_ok && !Floor) ? (int32_t)ih_s[off + (uint32_t)(k * a.H)] : 0;
                        if (from_regs) {
                            hold[mt][i] = h_keep[mt][i];
                        } else if (from_priv) {
                            // (prmt with four-bit selectors: 8 | i replicates the sign of byte i)
                            asm("prmt.b32 %0, %1, %2, %3;" : "=r"(hold[mt][i]) : "r"(priv_word), "r"(0u), "r"(priv_sel + 0x1111u * (uint32_t)i));
                        } else {
                            const uint8_t hb = v_ok ? h_cur[sw128_offset(b, j, a.NB)] : (uint8_t)0;
                            hold[mt][i] = state_byte(hb, h_bits);
                        }
                    }
                }
                // All CH cells of a tile are computed before anything is stored: a byte store into
                // the state tile may alias the tables as far as the compiler knows, so a store
                // between two cells would keep the second cell's table reads behind it and serialise
                // the dependency chains.  Inputs of absent rows/units are zeros and every table index
                // is clamped, so every lane computes; only the stores are guarded.
                int32_t hn[MT][CH];
                const uint32_t ta0 = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)g * acc_cols_g + (uint32_t)c0;
                // the sums of one gate for this thread's CH cells: the K halves are added here
                auto ld_gate = [&](int gate, int32_t(&acc)[MT][CH]) {
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt) tc::tmem_ld4(ta0 + (uint32_t)(((mt * 3 + gate) * KP) * a.NB), acc[mt]);
                    if (KP == 2) {
                        int32_t hi[MT][CH];
#pragma unroll
                        for (int mt = 0; mt < MT; ++mt) tc::tmem_ld4(ta0 + (uint32_t)(((mt * 3 + gate) * KP + 1) * a.NB), hi[mt]);
                        tc::tmem_ld_wait();
#pragma unroll
                        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                            for (int i = 0; i < CH; ++i) acc[mt][i] += hi[mt][i];
                    } else {
                        tc::tmem_ld_wait();
                    }
                };
                if constexpr (Floor) {
                    if (!waited) {
                        ok = tc::mbar_wait(&md[2], par, WAIT_BUDGET);
                        if (!ok) break;
                        tc::tc_fence_after_sync();
                        waited = true;
                        STAMP(warp == 1 && lane == 0, 2);
                    }
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                        for (int i = 0; i < CH; ++i) hn[mt][i] = hold[mt][i];
                } else if constexpr (Fused && Narrow) {
                    int32_t acc[MT][CH], zd[MT][CH], rd[MT][CH];
                    // update gate
                    if (!waited) {
                        ok = tc::mbar_wait(&md[0], par, WAIT_BUDGET);
                        if (!ok) break;
                        tc::tc_fence_after_sync();
                        STAMP(warp == 1 && lane == 0, 2);
                    }
                    ld_gate(0, acc);
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                        for (int i = 0; i < CH; ++i)
                            zd[mt][i] = fused_gate_fast(gc, tab, ACT_Z, ihv[mt][i][0], lin_round<Tie>(acc[mt][i], fl[mt][0]));
                    // reset gate
                    if (!waited) {
                        ok = tc::mbar_wait(&md[1], par, WAIT_BUDGET);
                        if (!ok) break;
                        tc::tc_fence_after_sync();
                    }
                    ld_gate(1, acc);
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                        for (int i = 0; i < CH; ++i)
                            rd[mt][i] = fused_gate_fast(gc, tab, ACT_R, ihv[mt][i][1], lin_round<Tie>(acc[mt][i], fl[mt][1]));
                    // new gate and the state update
                    if (!waited) {
                        ok = tc::mbar_wait(&md[2], par, WAIT_BUDGET);
                        if (!ok) break;
                        tc::tc_fence_after_sync();
                        waited = true;
                    }
                    ld_gate(2, acc);
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                        for (int i = 0; i < CH; ++i)
                            hn[mt][i] = fused_finish_fast<Tie>(gc, tab, ihv[mt][i][2], lin_round<Tie>(acc[mt][i], fl[mt][2]),
                                                          zd[mt][i], rd[mt][i], hold[mt][i]);
                } else if (!Fused && !Narrow && a.fs_on) {
                    // float-storage forward: float requantization of the exact sums, real sigmoid /
                    // tanh (PointwiseOperationsFP of the reference), gate by gate as the MMAs of
                    // each gate's rows complete
                    int32_t acc[MT][CH];
                    float ug[MT][CH], rg[MT][CH];
                    if (!waited) {
                        ok = tc::mbar_wait(&md[0], par, WAIT_BUDGET);
                        if (!ok) break;
                        tc::tc_fence_after_sync();
                    }
                    ld_gate(0, acc);
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                        for (int i = 0; i < CH; ++i)
                            ug[mt][i] = fs_sigmoid_gate_tab(a.fs, tab, 0, (float)ihv[mt][i][0],
                                                            fs_linear(acc[mt][i], fsk[mt][0][0], fsk[mt][0][1], fsk[mt][0][2],
                                                                      a.fs.zp_hh, a.fs.hh_lo, a.fs.hh_hi));
                    if (!waited) {
                        ok = tc::mbar_wait(&md[1], par, WAIT_BUDGET);
                        if (!ok) break;
                        tc::tc_fence_after_sync();
                    }
                    ld_gate(1, acc);
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                        for (int i = 0; i < CH; ++i)
                            rg[mt][i] = fs_sigmoid_gate_tab(a.fs, tab, 1, (float)ihv[mt][i][1],
                                                            fs_linear(acc[mt][i], fsk[mt][1][0], fsk[mt][1][1], fsk[mt][1][2],
                                                                      a.fs.zp_hh, a.fs.hh_lo, a.fs.hh_hi));
                    if (!waited) {
                        ok = tc::mbar_wait(&md[2], par, WAIT_BUDGET);
                        if (!ok) break;
                        tc::tc_fence_after_sync();
                        waited = true;
                    }
                    ld_gate(2, acc);
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                        for (int i = 0; i < CH; ++i)
                            hn[mt][i] = (int32_t)fs_finish_tab(a.fs, tab, ug[mt][i], rg[mt][i], (float)ihv[mt][i][2],
                                                           fs_linear(acc[mt][i], fsk[mt][2][0], fsk[mt][2][1], fsk[mt][2][2],
                                                                     a.fs.zp_hh, a.fs.hh_lo, a.fs.hh_hi),
                                                           (float)hold[mt][i]);
                } else {
                    if (!waited) {
                        ok = tc::mbar_wait(&md[0], par, WAIT_BUDGET) && tc::mbar_wait(&md[1], par, WAIT_BUDGET) &&
                             tc::mbar_wait(&md[2], par, WAIT_BUDGET);
                        if (!ok) break;
                        tc::tc_fence_after_sync();
                        waited = true;
                    }
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt) {
                        int32_t az[CH], ar[CH], an[CH];
                        const uint32_t ta = ta0 + (uint32_t)(mt * 3 * KP * a.NB);
                        tc::tmem_ld4(ta, az);
                        tc::tmem_ld4(ta + KP * a.NB, ar);
                        tc::tmem_ld4(ta + 2 * KP * a.NB, an);
                        if (KP == 2) {
                            int32_t bz[CH], br_[CH], bn[CH];
                            tc::tmem_ld4(ta + a.NB, bz);
                            tc::tmem_ld4(ta + 3 * a.NB, br_);
                            tc::tmem_ld4(ta + 5 * a.NB, bn);
                            tc::tmem_ld_wait();
#pragma unroll
                            for (int i = 0; i < CH; ++i) {
                                az[i] += bz[i];
                                ar[i] += br_[i];
                                an[i] += bn[i];
                            }
                        }
                        tc::tmem_ld_wait();
#pragma unroll
                        for (int i = 0; i < CH; ++i) {
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
                            if constexpr (Fused)
                                hn[mt][i] = gru_cell_fused(gc, tables, ihv[mt][i][0], ihv[mt][i][1], ihv[mt][i][2], hh_z,
                                                           hh_r, hh_n, hold[mt][i]);
                            else
                                hn[mt][i] = gru_cell<Narrow>(gc, tables, ihv[mt][i][0], ihv[mt][i][1], ihv[mt][i][2], hh_z,
                                                             hh_r, hh_n, hold[mt][i]);
                        }
                    }
                }
                // h_t[b][j] = element (row b, K index j) of the next B tile.  Pack the CH row bytes of
                // this lane's unit, gather byte x_row of the four lanes 4 * x_word .. + 3, store the
                // word into this CTA's tile and send it to every peer's.  Absent rows and units send
                // their (clamped) values too: they land in padding rows, or multiply zero columns of
                // R, and the peers count on the full number of bytes.
                const bool last = c + EPW >= nchunks;
                const uint32_t nbuf = (uint32_t)(2 * g + ((s + 1) & 1));
                const uint32_t bar_nx = bar_u32 + 8u * nbuf;
                // (nothing reads the state after the last step, and no store may be on its way to a
                // peer when the kernel ends)
#pragma unroll
                for (int mt = 0; mt < MT && s + 1 < a.T; ++mt) {
                    const uint32_t packed = ((uint32_t)hn[mt][0] & 0xffu) | (((uint32_t)hn[mt][1] & 0xffu) << 8) |
                                            (((uint32_t)hn[mt][2] & 0xffu) << 16) | ((uint32_t)hn[mt][3] << 24);
                    if (priv_h) h_priv[kc * EPI_THREADS] = packed;
                    const uint32_t v0 = __shfl_sync(0xffffffffu, packed, 4 * x_word + 0);
                    const uint32_t v1 = __shfl_sync(0xffffffffu, packed, 4 * x_word + 1);
                    const uint32_t v2 = __shfl_sync(0xffffffffu, packed, 4 * x_word + 2);
                    const uint32_t v3 = __shfl_sync(0xffffffffu, packed, 4 * x_word + 3);
                    const uint32_t word = __byte_perm(__byte_perm(v0, v1, x_sel), __byte_perm(v2, v3, x_sel), 0x5410);
                    const uint32_t at = tile_u32 + nbuf * h_buf_bytes +
                                        sw128_offset(c0 + x_row, j0 + mt * 128 + q * 32 + 4 * x_word, a.NB);
                    sts_u32(at, word);
                    for (int r = 0; r < a.P; ++r)
                        if (r != p) st_async_u32(map_to_rank(at, (uint32_t)r), word, map_to_rank(bar_nx, (uint32_t)r));
                }
                if (!last) store_outputs(hn, c0, nb, out_base);
                if (a.write_final && s + 1 == a.T) {
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                        for (int i = 0; i < CH; ++i)
                            if (c0 + i < nb && j_ok[mt])
                                a.h8[(size_t)(bg0 + c0 + i) * a.Hpad + j0 + mt * 128 + u] = (uint8_t)hn[mt][i];
                }
#pragma unroll
                for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                    for (int i = 0; i < CH; ++i) {
                        hn_last[mt][i] = hn[mt][i];
                        h_keep[mt][i] = hn[mt][i];
                    }
                if (last) c_last = c;
                ++kc;
            }
            if (ok && !waited) {
                // A warp without a chunk still waits for this step's MMAs: it must not arrive twice
                // within one phase of the tile barrier.
                ok = tc::mbar_wait(&md[2], par, WAIT_BUDGET);
                tc::tc_fence_after_sync();
            }
            // this warp's own words are ordered for the async proxy (the MMAs read them), then one
            // lane arrives for the warp on this CTA's barrier of the buffer just written
            fence_proxy_async_cta();
            tc::tc_fence_before_sync();
            __syncwarp();
            STAMP(warp == 1 && lane == 0, 4);
            if (lane == 0 && s + 1 < a.T) tc::mbar_arrive(&h_ready[2 * g + ((s + 1) & 1)]);
            // Outputs of the last chunk leave for global memory after the arrive: nothing in the next
            // step waits for them, so they overlap the exchange and the next MMAs.
            if (c_last >= 0) store_outputs(hn_last, c_last * CH, nb, out_base);
            }   // sub-groups
        }
        if (!ok && lane == 0) atomicOr(a.abort_flag, 1);
    }
    tc::tc_fence_before_sync();
    __syncthreads();
    // nobody leaves while a peer's copy into, or out of, its shared memory may be in flight
    cluster_arrive();
    cluster_wait();
    if (warp == 0) tc::tmem_dealloc(tmem_base, tmem_cols);
}

template <typename IhT, bool Narrow, bool Fused, int MT, bool Floor, bool Tie = true, bool Priv = false>
cudaError_t launch_one(const CUtensorMap &mr, const CUtensorMap &mh, const GateConsts &gc, RecMmaArgs &a,
                       int grid, size_t smem, cudaStream_t st) {
    auto kern = k_recurrence_cluster<IhT, Narrow, Fused, MT, Floor, Tie, Priv>;
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

template <typename IhT, bool Narrow, bool Fused>
cudaError_t launch_mt(int MT, const CUtensorMap &mr, const CUtensorMap &mh, const GateConsts &gc,
                      RecMmaArgs &a, int grid, size_t smem, cudaStream_t st) {
    return MT == 2 ? launch_one<IhT, Narrow, Fused, 2, false>(mr, mh, gc, a, grid, smem, st)
                   : launch_one<IhT, Narrow, Fused, 1, false>(mr, mh, gc, a, grid, smem, st);
}

template <typename IhT>
cudaError_t launch_notie(int MT, const CUtensorMap &mr, const CUtensorMap &mh, const GateConsts &gc, RecMmaArgs &a,
                         int grid, size_t smem, cudaStream_t st) {
    return MT == 2 ? launch_one<IhT, true, true, 2, false, false>(mr, mh, gc, a, grid, smem, st)
                   : launch_one<IhT, true, true, 1, false, false>(mr, mh, gc, a, grid, smem, st);
}

cudaError_t launch_any(bool fused, bool narrow, int ih_bytes, int MT, bool floor, bool notie, const CUtensorMap &mr,
                       const CUtensorMap &mh, const GateConsts &gc, RecMmaArgs &a, int grid, size_t smem,
                       cudaStream_t st) {
    if (floor)   // the synchronisation-floor measurement exists for the one form the benchmark's headline runs
        return (fused && narrow && ih_bytes == 2 && MT == 1)
                   ? launch_one<int16_t, true, true, 1, true>(mr, mh, gc, a, grid, smem, st)
                   : cudaErrorNotSupported;
    // several chunks of cells per warp and step: the instance that keeps the state of a warp's own cells
    // in private words of shared memory (branch-free fused cell, one tile per CTA, one sub-group)
    if (fused && narrow && MT == 1 && a.NG == 1 && a.NB / CH > EPW) {
        if (notie)
            return ih_bytes == 2 ? launch_one<int16_t, true, true, 1, false, false, true>(mr, mh, gc, a, grid, smem, st)
                                 : launch_one<int32_t, true, true, 1, false, false, true>(mr, mh, gc, a, grid, smem, st);
        return ih_bytes == 2 ? launch_one<int16_t, true, true, 1, false, true, true>(mr, mh, gc, a, grid, smem, st)
                             : launch_one<int32_t, true, true, 1, false, true, true>(mr, mh, gc, a, grid, smem, st);
    }
    if (fused && narrow && notie)
        return ih_bytes == 2 ? launch_notie<int16_t>(MT, mr, mh, gc, a, grid, smem, st)
                             : launch_notie<int32_t>(MT, mr, mh, gc, a, grid, smem, st);
    if (fused && narrow)   // for the fused cell `narrow` carries "every scale is shift-free"
        return ih_bytes == 2 ? launch_mt<int16_t, true, true>(MT, mr, mh, gc, a, grid, smem, st)
                             : launch_mt<int32_t, true, true>(MT, mr, mh, gc, a, grid, smem, st);
    if (fused)
        return ih_bytes == 2 ? launch_mt<int16_t, false, true>(MT, mr, mh, gc, a, grid, smem, st)
                             : launch_mt<int32_t, false, true>(MT, mr, mh, gc, a, grid, smem, st);
    if (ih_bytes == 1)
        return narrow ? launch_mt<int8_t, true, false>(MT, mr, mh, gc, a, grid, smem, st)
                      : launch_mt<int8_t, false, false>(MT, mr, mh, gc, a, grid, smem, st);
    return narrow ? launch_mt<int16_t, true, false>(MT, mr, mh, gc, a, grid, smem, st)
                  : launch_mt<int16_t, false, false>(MT, mr, mh, gc, a, grid, smem, st);
}

}  // namespace

bool rec_cluster_plan(int H, int Hpad, int B, int sms, int smem_optin, int n_table, int r_where,
                      int mt_opt, int ng_opt, int kp_opt, RecMmaPlan *out) {
    if (Hpad > 1024) return false;                 // K-slab loops are unrolled to 8
    const int KBn = Hpad / 128;
    // One 128-unit tile per CTA.  Two tiles per CTA for 128 < H <= 256 (one CTA per group, no
    // exchange) exist as an option (mt_opt 2) but measured 2.4x slower per step: twice the
    // epilogue per thread under the same register limit.
    const int MT = (mt_opt == 2 && H > 128 && H <= 256) ? 2 : 1;
    const int P = (H + 128 * MT - 1) / (128 * MT);  // cluster size: 1..8 (the portable maximum)
    if (P > 8 || P > sms) return false;
    const int groups_max = std::max(1, sms / P);
    // Rows per cluster, then sub-groups per CTA (ng_opt: 0 auto = 1, 1, 2).  Two sub-groups let the
    // MMAs of one overlap the cells of the other; measured no faster so far (the warps' own
    // instruction latencies between two chunks fill the time), so only on request.
    int RC = ((B + groups_max - 1) / groups_max + 15) / 16 * 16;
    int NG = ng_opt == 2 ? 2 : 1;
    if (NG == 2) RC = std::max(RC, 32);
    int NB = (RC / NG + 15) / 16 * 16;
    const int nb_cap = (MT == 2 ? 64 : 128) / NG;  // 3 * MT * NB * NG accumulator columns <= 512
    NB = std::min(NB, nb_cap);
    const int n_tiles = MT * 3 * KBn;
    // Where the R slice lives: as many 128x128 tiles as fit beside the accumulators go to tensor
    // memory (32 columns each; r_where: 0 auto, 1 none, 2 at least one), the rest stays in
    // shared-memory slots; the slots also stage the tensor-memory tiles, up to 12 per pass.
    for (;; NB -= 16) {
        // two K halves with accumulators of their own where K has two slabs and the whole slice of R still
        // fits tensor memory beside them
        int KP = (kp_opt == 2 && KBn >= 2) ? 2 : 1;
        if ((3 * MT * NB * NG * KP + 31) / 32 * 32 + n_tiles * 32 > 512 && (3 * MT * NB * NG + 31) / 32 * 32 + n_tiles * 32 <= 512)
            KP = 1;
        if (3 * MT * NB * NG * KP > 384) KP = 1;
        const int acc_cols = (3 * MT * NB * NG * KP + 31) / 32 * 32;
        int tmem_tiles = r_where == 1 ? 0 : std::max(0, std::min(n_tiles, (512 - acc_cols) / 32));
        // a slice that does not fit tensor memory as a whole but fits shared memory stays there as
        // a whole: the split form needs a slower, rolled MMA issue loop
        if (tmem_tiles < n_tiles && r_where != 2 &&
            cluster_smem_layout(n_tiles, KBn, NB, NG, n_table).total + 1024 <= (size_t)smem_optin)
            tmem_tiles = 0;
        const int resident = n_tiles - tmem_tiles;
        for (int stage = std::min(std::max(tmem_tiles, 1), 12); stage >= 1; --stage) {
            const int r_slots = std::max(resident, stage);
            const size_t smem = cluster_smem_layout(r_slots, KBn, NB, NG, n_table).total + 1024;
            if (smem > (size_t)smem_optin || (r_where == 2 && tmem_tiles == 0)) continue;
            uint32_t cols = 32;
            while ((int)cols < acc_cols + tmem_tiles * 32) cols <<= 1;
            out->MT = MT;
            out->P = P;
            out->NB = NB;
            out->NG = NG;
            out->G = (B + NB * NG - 1) / (NB * NG);
            out->smem = smem;
            out->tmem_cols = (int)cols;
            out->r_tmem_col = tmem_tiles > 0 ? acc_cols : 0;
            out->tmem_tiles = tmem_tiles;
            out->r_slots = r_slots;
            out->k_parts = KP;
            out->groups_per_launch = out->G;       // clusters are scheduled as SMs free up
            return true;
        }
        if (NB <= 16) return false;
    }
}

int rec_cluster_launch(RecMmaState &s, const RecMmaPlan &pl, RecMmaArgs a, const GateConsts &gc_host,
                       const int8_t *r8, long long r_rows_alloc, long long h_rows_alloc, bool h_unsigned,
                       int ih_bytes, bool narrow, bool fused, bool floor, bool notie, cudaStream_t stream,
                       std::string *err) {
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
    const cudaError_t e = launch_any(fused, narrow, ih_bytes, pl.MT, floor, notie, mr, mh, gc_host, a, pl.G * pl.P, pl.smem, stream);
    if (e == cudaErrorNotSupported && floor) {
        if (err) *err = "the synchronisation-floor probe exists for the fused shift-free cell with 16-bit W*x+bw only";
        return QGRU_ERR_UNSUPPORTED;
    }
    if (e != cudaSuccess) {
        if (err) *err = std::string("recurrence (cluster) launch: ") + cudaGetErrorString(e);
        cudaGetLastError();
        return QGRU_ERR_CUDA;
    }
    ++s.launches;
    return QGRU_OK;
}

}  // namespace qgru
