// qgru_kernels.cuh - device code of the integer GRU forward: boundary quantize kernels,
// the SIMT input-projection GEMM, the persistent recurrence kernel and the generic
// (any bit width) fallback kernels.  Include from ONE translation unit only (it defines
// non-template __global__ functions).  Written for sm_100a; one CTA per SM is assumed for the
// persistent kernel (it claims most of the 227 KB of shared memory).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "qgru_device.cuh"
#include "qgru_internal.h"

namespace qgru {

// --------------------------------------------------------- boundary kernels (a12, a13)

// quantize(float, FixedPointScale, zp, bw) (include/quantize_ops_helper.h:528-533): IEEE
// division by the decoded 16-bit-mantissa scale, round half to even, add zp in float.
__device__ __forceinline__ int32_t quantize_one(float x, float scale, int32_t zp, int32_t lo,
                                                int32_t hi) {
    const float q = rintf(__fdiv_rn(x, scale)) + (float)zp;
    return clampi((int32_t)q, lo, hi);
}

// fp32 activations -> 8-bit rows padded to Kpad (zeros), optionally also int32 containers.
// One thread per group of 4 padded columns.
__global__ void k_quantize_rows_f32(const float *__restrict__ x, uint8_t *__restrict__ out8,
                                    int32_t *__restrict__ out32, long long rows, int K, int Kpad,
                                    float scale, int32_t zp, int32_t lo, int32_t hi) {
    const int kw = Kpad >> 2;
    const long long total = rows * kw;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const long long row = i / kw;
        const int k0 = (int)(i - row * kw) * 4;
        unsigned packed = 0;
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int k = k0 + u;
            int32_t q = 0;
            if (k < K) {
                q = quantize_one(x[row * K + k], scale, zp, lo, hi);
                if (out32) out32[row * K + k] = q;
            }
            packed |= ((unsigned)q & 0xffu) << (8 * u);
        }
        if (out8) reinterpret_cast<unsigned *>(out8)[i] = packed;
    }
}

// int32 containers -> 8-bit rows padded to Kpad.  Values outside [lo, hi] (they would have
// been clamped by the reference's quantize step) raise bit 0 of *err.
__global__ void k_narrow_rows_i32(const int32_t *__restrict__ x, uint8_t *__restrict__ out8,
                                  long long rows, int K, int Kpad, int32_t lo, int32_t hi,
                                  int *err) {
    const int kw = Kpad >> 2;
    const long long total = rows * kw;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const long long row = i / kw;
        const int k0 = (int)(i - row * kw) * 4;
        unsigned packed = 0;
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int k = k0 + u;
            int32_t q = 0;
            if (k < K) {
                q = x[row * K + k];
                if (q < lo || q > hi) atomicOr(err, 1);
            }
            packed |= ((unsigned)q & 0xffu) << (8 * u);
        }
        reinterpret_cast<unsigned *>(out8)[i] = packed;
    }
}

// fp32 -> int32 containers (generic path and x_q_out).
__global__ void k_quantize_f32_i32(const float *__restrict__ x, int32_t *__restrict__ out,
                                   long long n, float scale, int32_t zp, int32_t lo, int32_t hi) {
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n;
         i += (long long)gridDim.x * blockDim.x)
        out[i] = quantize_one(x[i], scale, zp, lo, hi);
}

// Per-channel weight quantize, zp = 0 (quantificationPerChannelBitwidth,
// src/quantize_ops.cu:313; channel = idx % C).
__global__ void k_quantize_weights(const float *__restrict__ w, int32_t *__restrict__ out,
                                   long long n, int C, const float *__restrict__ scales, int32_t lo,
                                   int32_t hi) {
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n;
         i += (long long)gridDim.x * blockDim.x)
        out[i] = quantize_one(w[i], scales[i % C], 0, lo, hi);
}

// dequantize (include/quantize_ops_helper.h:504-508).
__global__ void k_dequantize(const int32_t *__restrict__ q, float *__restrict__ out, long long n,
                             float scale, int32_t zp) {
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n;
         i += (long long)gridDim.x * blockDim.x)
        out[i] = (float)(q[i] - zp) * scale;
}

// Weight repack: int32 [K][C] (haste layout) -> int8 [C][Kpad] (K contiguous, zero padded)
// plus the column sums used by the zero-point correction.  One CTA per channel.
__global__ void k_pack_weights(const int32_t *__restrict__ wq, int8_t *__restrict__ w8,
                               int32_t *__restrict__ wsum, int K, int Kpad, int C, int *err) {
    const int m = blockIdx.x;
    int local = 0;
    for (int k = threadIdx.x; k < Kpad; k += blockDim.x) {
        int32_t v = 0;
        if (k < K) {
            v = wq[(size_t)k * C + m];
            local += v;
            if (v < -128 || v > 127) atomicOr(err, 2);
        }
        if (w8) w8[(size_t)m * Kpad + k] = (int8_t)v;
    }
    __shared__ int red[32];
    for (int o = 16; o > 0; o >>= 1) local += __shfl_xor_sync(0xffffffffu, local, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = local;
    __syncthreads();
    if (threadIdx.x == 0) {
        int s = 0;
        for (int i = 0; i < (int)((blockDim.x + 31) >> 5); ++i) s += red[i];
        wsum[m] = s;
    }
}

// corr[m] = rescale(bias_q[m], bias_rs[m]) - zp_in * sum_k W_q[k][m]
__global__ void k_channel_consts(const int32_t *__restrict__ bias_q,
                                 const Rescale *__restrict__ bias_rs,
                                 const int32_t *__restrict__ wsum, int32_t zp_in,
                                 int64_t *__restrict__ corr, const Rescale *__restrict__ rs,
                                 FastLin *__restrict__ fl, int C, long long acc_bound, int *flags,
                                 int flag_bit) {
    const int m = blockIdx.x * blockDim.x + threadIdx.x;
    if (m >= C) return;
    const int64_t c = rescale64((int64_t)bias_q[m], bias_rs[m]) - (int64_t)zp_in * (int64_t)wsum[m];
    corr[m] = c;
    fl[m] = make_fast_lin(rs[m], c);
    // acc + corr must stay inside int32 for the one-multiply epilogue
    const int64_t mag = c < 0 ? -c : c;
    if (mag + acc_bound >= 0x7fffffffll) atomicOr(flags, flag_bit);
    // can this channel's requantization meet an exact tie anywhere in its accumulator range?
    if (rescale_can_tie(rs[m].mult, rs[m].shift, c - acc_bound, c + acc_bound)) atomicOr(flags, flag_bit << 2);
}

// ------------------------------------------------ input projection, SIMT dp4a form (a1)

// ih[n][m] = epilogue( sum_k W8[m][k] * x8[n][k] ), n < N tokens, m < C channels.
// 64x64 output tile per CTA, 256 threads, 4x4 outputs per thread, K staged in 64-byte slabs.
// Raw: store the int32 sums themselves (no zero-point compensation, bias or requantization).
template <bool XUnsigned, typename IhT, bool Raw = false>
__global__ void __launch_bounds__(256)
k_gemm_wx_simt(const uint8_t *__restrict__ x8, const int8_t *__restrict__ w8, IhT *__restrict__ ih,
               long long N, int C, int Kpad, LinearConsts lc) {
    __shared__ unsigned xs[64][17];
    __shared__ unsigned ws[64][17];
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const long long n0 = (long long)blockIdx.x * 64;
    const int m0 = blockIdx.y * 64;
    int acc[4][4] = {};
    for (int k0 = 0; k0 < Kpad; k0 += 64) {
        for (int i = threadIdx.x; i < 64 * 16; i += 256) {
            const int r = i >> 4, c = i & 15;
            const int kb = k0 + c * 4;
            unsigned xv = 0, wv = 0;
            if (kb < Kpad) {
                if (n0 + r < N) xv = *reinterpret_cast<const unsigned *>(x8 + (n0 + r) * Kpad + kb);
                if (m0 + r < C) wv = *reinterpret_cast<const unsigned *>(w8 + (size_t)(m0 + r) * Kpad + kb);
            }
            xs[r][c] = xv;
            ws[r][c] = wv;
        }
        __syncthreads();
#pragma unroll
        for (int c = 0; c < 16; ++c) {
            unsigned xv[4];
            int wv[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) xv[i] = xs[ty * 4 + i][c];
#pragma unroll
            for (int j = 0; j < 4; ++j) wv[j] = (int)ws[tx + 16 * j][c];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = dp4a_w<XUnsigned>(wv[j], xv[i], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const long long n = n0 + ty * 4 + i;
        if (n >= N) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int m = m0 + tx + 16 * j;
            if (m >= C) continue;
            if constexpr (Raw) ih[n * C + m] = (IhT)acc[i][j];
            else if (lc.fs != nullptr)
                ih[n * C + m] = (IhT)(int32_t)fs_linear(acc[i][j], lc.fs[m], lc.fs[lc.fs_C + m], lc.fs[2 * lc.fs_C + m],
                                                        (float)lc.zp_out, (float)lc.lo, (float)lc.hi);
            else ih[n * C + m] = (IhT)linear_epilogue(acc[i][j], lc.corr[m], lc.rs[m], lc.zp_out, lc.lo, lc.hi);
        }
    }
}

// ------------------------------------------------------------ h slot 0 / state init

// Writes the initial state: the 8-bit state buffer (padded rows), and slot `slot` of the
// int32 / float outputs (quantGRUForwardInt32's h_q[0] fill, src/gru_interface.cc:568-574;
// the float entry point dequantizes that slot like every other, :704).
__global__ void k_init_state(const int32_t *__restrict__ h0_q, const float *__restrict__ h0_f,
                             uint8_t *__restrict__ h8, int32_t *__restrict__ hq_out,
                             float *__restrict__ hf_out, uint8_t *__restrict__ h8_out, int B, int H, int Hpad,
                             long long slot,
                             float scale, int32_t zp, int32_t lo, int32_t hi, int *err) {
    const long long total = (long long)B * Hpad;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const int b = (int)(i / Hpad), j = (int)(i % Hpad);
        int32_t q = 0;
        if (j < H) {
            if (h0_q) {
                q = h0_q[(size_t)b * H + j];
                if (q < lo || q > hi) atomicOr(err, 1);
            } else if (h0_f) {
                q = quantize_one(h0_f[(size_t)b * H + j], scale, zp, lo, hi);
            } else {
                q = zp;
            }
            const long long o = slot * B * H + (long long)b * H + j;
            if (hq_out) hq_out[o] = q;
            if (hf_out) hf_out[o] = (float)(q - zp) * scale;
            if (h8_out) h8_out[o] = (uint8_t)q;
        }
        if (h8) h8[i] = (uint8_t)q;
    }
}

// ------------------------------------------------ persistent recurrence, dp4a form (a2+a3)

struct RecArgs {
    int T, B, H, Hpad, C;
    int Hs;        // hidden units per CTA (multiple of 32)
    int Bt;        // batch rows per group
    int P;         // CTAs per group (slices of the hidden dimension)
    int reverse;
    const int8_t *r8;      // [3H][Hpad]
    const void *ih;        // [T*B][3H] int8 or int16
    uint8_t *h8;           // [2][B][Hpad] ping-pong state
    int32_t *hq_out;       // [(T+1)][B][H] or null
    float *hf_out;         // [(T+1)][B][H] or null
    uint8_t *h8_out = nullptr;   // [(T+1)][B][H] or null: the quantized state in its 8-bit container
    LinearConsts lc;       // R*h + br epilogue
    const GateConsts *gc;  // device copy
    const int32_t *tables; // activation tables, gc->table_off indexes into it
    int n_table;           // ints in tables
    unsigned *bar;         // one counter per group, 32 words apart
    int *abort_flag;       // set when a barrier wait ran out; every CTA then leaves
    unsigned spin_limit;
    int withhold_arrive = 0;   // failure-path test: CTA 0 skips its arrival after step 0, so its group's wait runs out
    // float-storage forward (k_recurrence_gemv with Cell 3): the float cell of the reference's
    // quantGRUForwardFP; fs_chan = [3][C] offset, bias term, scale ratio of R*h + br per channel
    const float *fs_chan = nullptr;
    FsConsts fs{};
};

// One CTA owns Hs hidden units (all three gates) of one group of Bt batch rows and keeps its
// slice of R in shared memory for all T steps.  Per step: fetch h_{t-1} of the group's rows,
// R*h with dp4a, requantize, gates, write h_t.  Groups never interact; the P CTAs of a group
// meet once per step at a counter in global memory (bounded spin).
template <bool HUnsigned, typename IhT, bool Narrow>
__global__ void __launch_bounds__(256, 1) k_recurrence_dp4a(RecArgs a) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int kw = a.Hpad >> 2;  // words per row
    // layout: GateConsts | tables | corr[3*Hs] i64 | rs[3*Hs] | Rs[3][kw][Hs] words | hs[Bt][kw] words
    GateConsts *gc = reinterpret_cast<GateConsts *>(smem_raw);
    size_t off = (sizeof(GateConsts) + 15) & ~size_t(15);
    int32_t *tables = reinterpret_cast<int32_t *>(smem_raw + off);
    off += ((size_t)a.n_table * 4 + 15) & ~size_t(15);
    int64_t *corr = reinterpret_cast<int64_t *>(smem_raw + off);
    off += (size_t)3 * a.Hs * 8;
    Rescale *rs = reinterpret_cast<Rescale *>(smem_raw + off);
    off += (size_t)3 * a.Hs * sizeof(Rescale);
    unsigned *Rs = reinterpret_cast<unsigned *>(smem_raw + off);
    off += (size_t)3 * kw * a.Hs * 4;
    unsigned *hs = reinterpret_cast<unsigned *>(smem_raw + off);

    const int grp = blockIdx.x / a.P, p = blockIdx.x % a.P;
    const int j0 = p * a.Hs, b0 = grp * a.Bt;
    const int nb = min(a.Bt, a.B - b0);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

    for (int i = tid; i < (int)(sizeof(GateConsts) / 4); i += 256)
        reinterpret_cast<int *>(gc)[i] = reinterpret_cast<const int *>(a.gc)[i];
    for (int i = tid; i < a.n_table; i += 256) tables[i] = a.tables[i];
    for (int i = tid; i < 3 * a.Hs; i += 256) {
        const int g = i / a.Hs, jl = i % a.Hs, j = j0 + jl;
        const bool ok = j < a.H;
        corr[i] = ok ? a.lc.corr[g * a.H + j] : 0;
        rs[i] = ok ? a.lc.rs[g * a.H + j] : Rescale{1, 1, 0, 0, 0, 0, 0, 0};
    }
    {
        const unsigned *r8w = reinterpret_cast<const unsigned *>(a.r8);
        const int total = 3 * a.Hs * kw;
        for (int i = tid; i < total; i += 256) {
            const int k4 = i % kw, gj = i / kw;
            const int g = gj / a.Hs, jl = gj % a.Hs, j = j0 + jl;
            Rs[(g * kw + k4) * a.Hs + jl] = (j < a.H) ? r8w[(size_t)(g * a.H + j) * kw + k4] : 0u;
        }
    }
    __syncthreads();

    const int JW = a.Hs >> 5;        // warps along the hidden dimension
    const int BW = 8 / JW;           // warps along the batch dimension
    const int wj = warp % JW, wb = warp / JW;
    const int jl = wj * 32 + lane, j = j0 + jl;
    const bool j_ok = j < a.H;
    constexpr int NB = 4;
    const size_t BH = (size_t)a.B * a.H;
    const IhT *ihp = reinterpret_cast<const IhT *>(a.ih);
    unsigned *bar = a.bar + grp * 32;
    bool dead = false;

    for (int s = 0; s < a.T; ++s) {
        const int t = a.reverse ? (a.T - 1 - s) : s;                  // x / ih time index
        const long long out_slot = a.reverse ? (a.T - 1 - s) : (s + 1);
        const uint8_t *h_cur = a.h8 + (size_t)(s & 1) * a.B * a.Hpad;
        uint8_t *h_nxt = a.h8 + (size_t)((s + 1) & 1) * a.B * a.Hpad;

        if (a.P > 1 && s > 0) {
            if (tid == 0) {
                const unsigned want = (unsigned)a.P * (unsigned)s;
                unsigned it = 0;
                while (ld_acquire(bar) < want) {
                    if (++it > a.spin_limit || (it % 1024 == 0 && *(volatile int *)a.abort_flag)) {
                        atomicOr(a.abort_flag, 1);
                        break;
                    }
                }
            }
            __syncthreads();
            if (tid == 0 && *(volatile int *)a.abort_flag) dead = true;
            if (__syncthreads_or(dead)) break;
        }

        // h_{t-1} rows of this group -> shared (L2 loads: other CTAs wrote them)
        {
            const uint4 *src = reinterpret_cast<const uint4 *>(h_cur + (size_t)b0 * a.Hpad);
            uint4 *dst = reinterpret_cast<uint4 *>(hs);
            const int total = nb * (a.Hpad >> 4);
            for (int i = tid; i < total; i += 256) dst[i] = __ldcg(src + i);
        }
        __syncthreads();

        for (int bb = wb * NB; bb < nb; bb += BW * NB) {
            int acc[NB][3];
#pragma unroll
            for (int u = 0; u < NB; ++u) acc[u][0] = acc[u][1] = acc[u][2] = 0;
            // ih loads are issued first so they fly under the dot products
            int32_t ihv[NB][3];
#pragma unroll
            for (int u = 0; u < NB; ++u) {
                const int b = bb + u;
#pragma unroll
                for (int g = 0; g < 3; ++g)
                    ihv[u][g] = (b < nb && j_ok)
                                    ? (int32_t)ihp[((size_t)t * a.B + b0 + b) * a.C + g * a.H + j]
                                    : 0;
            }
            for (int k4 = 0; k4 < kw; k4 += 4) {
                uint4 hv[NB];
#pragma unroll
                for (int u = 0; u < NB; ++u) {
                    const int b = min(bb + u, nb - 1);
                    hv[u] = *reinterpret_cast<const uint4 *>(hs + (size_t)b * kw + k4);
                }
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const int wz = (int)Rs[(0 * kw + k4 + q) * a.Hs + jl];
                    const int wr = (int)Rs[(1 * kw + k4 + q) * a.Hs + jl];
                    const int wn = (int)Rs[(2 * kw + k4 + q) * a.Hs + jl];
#pragma unroll
                    for (int u = 0; u < NB; ++u) {
                        const unsigned h4 = q == 0 ? hv[u].x : q == 1 ? hv[u].y : q == 2 ? hv[u].z : hv[u].w;
                        acc[u][0] = dp4a_w<HUnsigned>(wz, h4, acc[u][0]);
                        acc[u][1] = dp4a_w<HUnsigned>(wr, h4, acc[u][1]);
                        acc[u][2] = dp4a_w<HUnsigned>(wn, h4, acc[u][2]);
                    }
                }
            }
#pragma unroll
            for (int u = 0; u < NB; ++u) {
                const int b = bb + u;
                if (b >= nb || !j_ok) continue;
                int32_t hh[3];
#pragma unroll
                for (int g = 0; g < 3; ++g)
                    hh[g] = linear_epilogue(acc[u][g], corr[g * a.Hs + jl], rs[g * a.Hs + jl],
                                            a.lc.zp_out, a.lc.lo, a.lc.hi);
                const uint8_t hb = reinterpret_cast<const uint8_t *>(hs)[(size_t)b * a.Hpad + j];
                const int32_t h_old = HUnsigned ? (int32_t)hb : (int32_t)(int8_t)hb;
                const int32_t hn = gru_cell<Narrow>(*gc, tables, ihv[u][0], ihv[u][1], ihv[u][2],
                                                    hh[0], hh[1], hh[2], h_old);
                h_nxt[(size_t)(b0 + b) * a.Hpad + j] = (uint8_t)hn;
                const size_t o = (size_t)out_slot * BH + (size_t)(b0 + b) * a.H + j;
                if (a.hq_out) a.hq_out[o] = hn;
                if (a.hf_out) a.hf_out[o] = (float)(hn - gc->zp_h) * gc->h_scale;
                if (a.h8_out) a.h8_out[o] = (uint8_t)hn;
            }
        }
        __syncthreads();
        if (a.P > 1 && tid == 0 && !(a.withhold_arrive && blockIdx.x == 0 && s == 0)) {
            __threadfence();
            atomicAdd(bar, 1u);
        }
    }
}

// ------------------------------------------- persistent recurrence, small batch (GEMV form)

// One CTA per batch row, the whole R (3H x Hpad int8, H <= 256) in shared memory for all T
// steps: rows never interact, so there is no inter-CTA synchronisation at all and the step is
// as short as one matrix-vector product plus one cell.  A quad of threads owns one hidden unit:
// each lane takes a quarter of K for the unit's three gate rows (dp4a), two shuffles add the
// partial sums, lane 0 of the quad requantizes and runs the cell.  R is stored in the order the
// threads read it ([16-byte chunk][gate][thread]), so every 128-bit load is conflict-free.
// The state h_t stays in shared memory (two buffers, one __syncthreads per step).
// Cell: 0 generic datapath, 1 its 32-bit ("narrow") rescales, 2 the tabulated branch-free cell
// (W*x+bw arrives pre-rescaled from the GEMM; every scale in shift-free form), 3 the float cell
// of the float-storage forward (W*x+bw arrives requantized by the GEMM's float epilogue).
template <bool HUnsigned, typename IhT, int Cell>
__global__ void __launch_bounds__(1024, 1) k_recurrence_gemv(const __grid_constant__ GateConsts gc, RecArgs a) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int NT = blockDim.x;             // 4 * units (units rounded up to 32)
    const int Kq = a.Hpad >> 2;            // K bytes per lane of a quad
    const int nch = Kq >> 4;               // 16-byte chunks per lane and gate row (2 or 4)
    // layout: tables | hs[2][Hs] | Rq[nch * 3][NT] uint4.  The four K-quarters of a state buffer
    // are 16 bytes further apart than their length, so that the four 16-byte segments a warp
    // reads at once fall into different banks.
    const int Qs = Kq + 16, Hs = 4 * Qs;
    int32_t *tables = reinterpret_cast<int32_t *>(smem_raw);
    size_t off = ((size_t)a.n_table * 4 + 15) & ~size_t(15);
    unsigned char *hs = smem_raw + off;
    off += (size_t)2 * Hs;
    uint4 *Rq = reinterpret_cast<uint4 *>(smem_raw + off);

    const int tid = threadIdx.x, qd = tid & 3, j = tid >> 2;
    const int b = blockIdx.x;
    const bool j_ok = j < a.H;

    for (int i = tid; i < a.n_table; i += NT) tables[i] = a.tables[i];
    for (int i = tid; i < a.Hpad; i += NT) {
        const int at = (i / Kq) * Qs + (i % Kq);
        hs[at] = a.h8[(size_t)b * a.Hpad + i];      // initial state of this row (buffer 0 of h8)
        hs[Hs + at] = 0;
    }
    const int j_at = (j / Kq) * Qs + (j % Kq);      // where unit j's byte sits in a state buffer
    for (int g = 0; g < 3; ++g)
        for (int c = 0; c < nch; ++c) {
            uint4 w = make_uint4(0u, 0u, 0u, 0u);
            if (j_ok) w = *reinterpret_cast<const uint4 *>(a.r8 + (size_t)(g * a.H + j) * a.Hpad + qd * Kq + 16 * c);
            Rq[(size_t)(c * 3 + g) * NT + tid] = w;
        }
    // per-unit constants of the R*h + br epilogue (used by lane 0 of the quad)
    int64_t corr[3] = {0, 0, 0};
    Rescale rs[3];
    FastLin fl[3];
    bool fast = a.lc.fits32 != 0;
#pragma unroll
    for (int g = 0; g < 3; ++g) {
        rs[g] = Rescale{1, 1, 0, 0, 0, 0, 0, 0};
        fl[g] = FastLin{0, 0, 0, 0, 0, 0};
        if (j_ok) {
            corr[g] = a.lc.corr[g * a.H + j];
            rs[g] = a.lc.rs[g * a.H + j];
            fl[g] = a.lc.fl[g * a.H + j];
        }
        fast = fast && fl[g].mq != 0;
    }
    float fsk[3][3] = {};
    if constexpr (Cell == 3) {
#pragma unroll
        for (int g = 0; g < 3; ++g)
#pragma unroll
            for (int k = 0; k < 3; ++k) fsk[g][k] = j_ok ? a.fs_chan[(size_t)k * a.C + g * a.H + j] : 0.f;
    }
    __syncthreads();

    const size_t BH = (size_t)a.B * a.H;
    const IhT *ihp = reinterpret_cast<const IhT *>(a.ih);
    const uint32_t tab = (uint32_t)__cvta_generic_to_shared(tables);
    const bool worker = qd == 0 && j_ok;
    // W*x + bw of this row: loaded one step ahead, so the cell never waits for global memory
    auto load_ih = [&](int s, int32_t (&v)[3]) {
        const int t = a.reverse ? (a.T - 1 - s) : s;
        const IhT *src = ihp + ((size_t)t * a.B + b) * a.C + j;
        v[0] = (int32_t)src[0];
        v[1] = (int32_t)src[a.H];
        v[2] = (int32_t)src[2 * a.H];
    };
    int32_t ihv[3] = {0, 0, 0};
    if (worker) load_ih(0, ihv);
    for (int s = 0; s < a.T; ++s) {
        const long long out_slot = a.reverse ? (a.T - 1 - s) : (s + 1);
        const unsigned char *h_cur = hs + (size_t)(s & 1) * Hs;
        unsigned char *h_nxt = hs + (size_t)((s + 1) & 1) * Hs;
        int32_t ihn[3] = {0, 0, 0};
        if (worker && s + 1 < a.T) load_ih(s + 1, ihn);
        int acc[3] = {0, 0, 0};
        const uint4 *hq4 = reinterpret_cast<const uint4 *>(h_cur + qd * Qs);
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            if (c >= nch) break;
            const uint4 hv = hq4[c];
#pragma unroll
            for (int g = 0; g < 3; ++g) {
                const uint4 w = Rq[(size_t)(c * 3 + g) * NT + tid];
                acc[g] = dp4a_w<HUnsigned>((int)w.x, hv.x, acc[g]);
                acc[g] = dp4a_w<HUnsigned>((int)w.y, hv.y, acc[g]);
                acc[g] = dp4a_w<HUnsigned>((int)w.z, hv.z, acc[g]);
                acc[g] = dp4a_w<HUnsigned>((int)w.w, hv.w, acc[g]);
            }
        }
#pragma unroll
        for (int g = 0; g < 3; ++g) {
            acc[g] += __shfl_xor_sync(0xffffffffu, acc[g], 1);
            acc[g] += __shfl_xor_sync(0xffffffffu, acc[g], 2);
        }
        if (worker) {
            const unsigned char hb = h_cur[j_at];
            const int32_t h_old = HUnsigned ? (int32_t)hb : (int32_t)(int8_t)hb;
            int32_t hn;
            if constexpr (Cell == 2) {
                const int32_t z_d = fused_gate_fast(gc, tab, ACT_Z, ihv[0], lin_round(acc[0], fl[0]));
                const int32_t r_d = fused_gate_fast(gc, tab, ACT_R, ihv[1], lin_round(acc[1], fl[1]));
                hn = fused_finish_fast(gc, tab, ihv[2], lin_round(acc[2], fl[2]), z_d, r_d, h_old);
            } else if constexpr (Cell == 3) {
                // (computing the update and the reset gate on two lanes of the quad measured no faster)
                const float fih[3] = {(float)ihv[0], (float)ihv[1], (float)ihv[2]};
                float fhh[3];
#pragma unroll
                for (int g = 0; g < 3; ++g)
                    fhh[g] = fs_linear(acc[g], fsk[g][0], fsk[g][1], fsk[g][2], a.fs.zp_hh, a.fs.hh_lo, a.fs.hh_hi);
                const float u_g = fs_sigmoid_gate_tab(a.fs, tab, 0, fih[0], fhh[0]);
                const float r_g = fs_sigmoid_gate_tab(a.fs, tab, 1, fih[1], fhh[1]);
                hn = (int32_t)fs_finish_tab(a.fs, tab, u_g, r_g, fih[2], fhh[2], (float)h_old);
            } else {
                int32_t hh[3];
#pragma unroll
                for (int g = 0; g < 3; ++g) {
                    if (fast) hh[g] = linear_epilogue_fast(acc[g], fl[g], a.lc.zp_out, a.lc.lo, a.lc.hi);
                    else hh[g] = linear_epilogue(acc[g], corr[g], rs[g], a.lc.zp_out, a.lc.lo, a.lc.hi);
                }
                hn = gru_cell<Cell == 1>(gc, tables, ihv[0], ihv[1], ihv[2], hh[0], hh[1], hh[2], h_old);
            }
            h_nxt[j_at] = (unsigned char)hn;
            const size_t o = (size_t)out_slot * BH + (size_t)b * a.H + j;
            if (a.hq_out) a.hq_out[o] = hn;
            if (a.hf_out) a.hf_out[o] = (float)(hn - gc.zp_h) * gc.h_scale;
            if (a.h8_out) a.h8_out[o] = (uint8_t)hn;
        }
        ihv[0] = ihn[0];
        ihv[1] = ihn[1];
        ihv[2] = ihn[2];
        __syncthreads();
    }
}

// The same with R in REGISTERS (the branch-free cells only): two threads own one hidden unit, each
// half of K for the unit's three gate rows, i.e. 3 * KT bytes of R (KT = Hpad / 2 = 64 or 128) held
// in 48 or 96 registers for all T steps.  A step then reads only the state (a few hundred bytes,
// broadcast) from shared memory instead of all of R (196 KB at H = 256, which at 128 bytes per
// clock is 1536 cycles on its own): KT / 4 * 3 dp4a per thread.  The threads of the upper K half
// are the upper half of the CTA's warps: they hand their three partial sums over through shared
// memory (a named barrier they only arrive on), and the lower half's warps run the cell with every
// lane busy.  The per-unit constants of the R*h + br requantization live in shared memory (the
// registers belong to R).
// Cell: 2 the tabulated integer cell, 3 the float cell of the float-storage forward (as in k_recurrence_gemv).
template <bool HUnsigned, typename IhT, int KT, int Cell = 2>
__global__ void __launch_bounds__(512, 1) k_recurrence_gemv_reg(const __grid_constant__ GateConsts gc, RecArgs a) {
    static_assert(Cell == 2 || Cell == 3, "the branch-free cells only");
    extern __shared__ __align__(16) unsigned char smem_raw[];
    static_assert(KT == 64 || KT == 128, "Hpad = 128 or 256");
    constexpr int QS = KT + 16;            // the two K halves of a state buffer sit 16 bytes further apart than their length
    constexpr int HS = 2 * QS;
    const int NT = blockDim.x;             // 2 * units (units rounded up to 32: whole warps per K half)
    int32_t *tables = reinterpret_cast<int32_t *>(smem_raw);
    size_t off = ((size_t)a.n_table * 4 + 15) & ~size_t(15);
    unsigned char *hs = smem_raw + off;
    off += (size_t)2 * HS;
    int *part = reinterpret_cast<int *>(smem_raw + off);          // [3][units]: the upper K half's partial sums
    off += (size_t)3 * (NT >> 1) * sizeof(int);
    FastLin *fls = reinterpret_cast<FastLin *>(smem_raw + off);   // Cell 2: [3][units]
    float *fsk = reinterpret_cast<float *>(smem_raw + off);       // Cell 3: [3 gates][3 constants][units]

    const int tid = threadIdx.x, units = NT >> 1, half = tid >= units ? 1 : 0, j = tid - half * units;
    const int b = blockIdx.x;
    const bool j_ok = j < a.H;

    for (int i = tid; i < a.n_table; i += NT) tables[i] = a.tables[i];
    for (int i = tid; i < 2 * KT; i += NT) {
        const int at = (i / KT) * QS + (i % KT);
        hs[at] = a.h8[(size_t)b * a.Hpad + i];      // initial state of this row (buffer 0 of h8)
        hs[HS + at] = 0;
    }
    if constexpr (Cell == 2) {
        for (int i = tid; i < 3 * units; i += NT) {
            const int g = i / units, u = i % units;
            fls[i] = u < a.H ? a.lc.fl[g * a.H + u] : FastLin{0, 0, 0, 0, 0, 0};
        }
    } else {
        for (int i = tid; i < 9 * units; i += NT) {
            const int gk = i / units, u = i % units, g = gk / 3, k = gk % 3;
            fsk[i] = u < a.H ? a.fs_chan[(size_t)k * a.C + g * a.H + u] : 0.f;
        }
    }
    const int j_at = (j / KT) * QS + (j % KT);      // where unit j's byte sits in a state buffer
    uint32_t R[3][KT / 4];
#pragma unroll
    for (int g = 0; g < 3; ++g)
#pragma unroll
        for (int c = 0; c < KT / 16; ++c) {
            uint4 w = make_uint4(0u, 0u, 0u, 0u);
            if (j_ok) w = *reinterpret_cast<const uint4 *>(a.r8 + (size_t)(g * a.H + j) * a.Hpad + half * KT + 16 * c);
            R[g][4 * c + 0] = w.x;
            R[g][4 * c + 1] = w.y;
            R[g][4 * c + 2] = w.z;
            R[g][4 * c + 3] = w.w;
        }
    __syncthreads();

    const size_t BH = (size_t)a.B * a.H;
    const IhT *ihp = reinterpret_cast<const IhT *>(a.ih);
    const uint32_t tab = (uint32_t)__cvta_generic_to_shared(tables);
    const bool worker = half == 0 && j_ok;
    // W*x + bw of this row: loaded one step ahead, so the cell never waits for global memory
    auto load_ih = [&](int s, int32_t (&v)[3]) {
        const int t = a.reverse ? (a.T - 1 - s) : s;
        const IhT *src = ihp + ((size_t)t * a.B + b) * a.C + j;
        v[0] = (int32_t)src[0];
        v[1] = (int32_t)src[a.H];
        v[2] = (int32_t)src[2 * a.H];
    };
    int32_t ihv[3] = {0, 0, 0};
    if (worker) load_ih(0, ihv);
    for (int s = 0; s < a.T; ++s) {
        const long long out_slot = a.reverse ? (a.T - 1 - s) : (s + 1);
        const unsigned char *h_cur = hs + (size_t)(s & 1) * HS;
        unsigned char *h_nxt = hs + (size_t)((s + 1) & 1) * HS;
        int32_t ihn[3] = {0, 0, 0};
        if (worker && s + 1 < a.T) load_ih(s + 1, ihn);
        int acc[3] = {0, 0, 0};
        const uint4 *hq4 = reinterpret_cast<const uint4 *>(h_cur + half * QS);
#pragma unroll
        for (int c = 0; c < KT / 16; ++c) {
            const uint4 hv = hq4[c];
#pragma unroll
            for (int g = 0; g < 3; ++g) {
                acc[g] = dp4a_w<HUnsigned>((int)R[g][4 * c + 0], hv.x, acc[g]);
                acc[g] = dp4a_w<HUnsigned>((int)R[g][4 * c + 1], hv.y, acc[g]);
                acc[g] = dp4a_w<HUnsigned>((int)R[g][4 * c + 2], hv.z, acc[g]);
                acc[g] = dp4a_w<HUnsigned>((int)R[g][4 * c + 3], hv.w, acc[g]);
            }
        }
        if (half) {
            // hand the partial sums to the lower half's thread of the same unit; nothing to wait for here
#pragma unroll
            for (int g = 0; g < 3; ++g) part[g * units + j] = acc[g];
            asm volatile("bar.arrive 1, %0;" ::"r"(NT) : "memory");
        } else {
            asm volatile("bar.sync 1, %0;" ::"r"(NT) : "memory");
#pragma unroll
            for (int g = 0; g < 3; ++g) acc[g] += part[g * units + j];
        }
        if (worker) {
            const unsigned char hb = h_cur[j_at];
            const int32_t h_old = HUnsigned ? (int32_t)hb : (int32_t)(int8_t)hb;
            int32_t hn;
            if constexpr (Cell == 2) {
                const int32_t z_d = fused_gate_fast(gc, tab, ACT_Z, ihv[0], lin_round(acc[0], fls[j]));
                const int32_t r_d = fused_gate_fast(gc, tab, ACT_R, ihv[1], lin_round(acc[1], fls[units + j]));
                hn = fused_finish_fast(gc, tab, ihv[2], lin_round(acc[2], fls[2 * units + j]), z_d, r_d, h_old);
            } else {
                const float fih[3] = {(float)ihv[0], (float)ihv[1], (float)ihv[2]};
                float fhh[3];
#pragma unroll
                for (int g = 0; g < 3; ++g)
                    fhh[g] = fs_linear(acc[g], fsk[(g * 3 + 0) * units + j], fsk[(g * 3 + 1) * units + j],
                                       fsk[(g * 3 + 2) * units + j], a.fs.zp_hh, a.fs.hh_lo, a.fs.hh_hi);
                const float u_g = fs_sigmoid_gate_tab(a.fs, tab, 0, fih[0], fhh[0]);
                const float r_g = fs_sigmoid_gate_tab(a.fs, tab, 1, fih[1], fhh[1]);
                hn = (int32_t)fs_finish_tab(a.fs, tab, u_g, r_g, fih[2], fhh[2], (float)h_old);
            }
            h_nxt[j_at] = (unsigned char)hn;
            const size_t o = (size_t)out_slot * BH + (size_t)b * a.H + j;
            if (a.hq_out) a.hq_out[o] = hn;
            if (a.hf_out) a.hf_out[o] = (float)(hn - gc.zp_h) * gc.h_scale;
            if (a.h8_out) a.h8_out[o] = (uint8_t)hn;
        }
        ihv[0] = ihn[0];
        ihv[1] = ihn[1];
        ihv[2] = ihn[2];
        __syncthreads();
    }
}

// --------------------------------------------- generic fallback (any bit width, int32 data)

// out[n][m] = epilogue( sum_k W_q[k][m] * in[n][k] ) with 64-bit accumulation
// (quantizedGemmBiasFused's arithmetic, src/gru_forward_gpu_quant.cu:110-180).
__global__ void k_linear_generic(const int32_t *__restrict__ wq, const int32_t *__restrict__ in,
                                 int32_t *__restrict__ out, long long N, int K, int C,
                                 LinearConsts lc, uint8_t *__restrict__ keep = nullptr) {
    const int m = blockIdx.x * blockDim.x + threadIdx.x;
    const long long n = blockIdx.y;
    if (m >= C || n >= N) return;
    int64_t acc = 0;
    for (int k = 0; k < K; ++k) acc += (int64_t)wq[(size_t)k * C + m] * (int64_t)in[n * K + k];
    out[n * C + m] = linear_epilogue(acc, lc.corr[m], lc.rs[m], lc.zp_out, lc.lo, lc.hi,
                                     keep ? keep + n * C + m : nullptr);
}

// v: optional [B][4H] out of this step: update, reset, new gate outputs and the R*h + br row of
// the new gate (the training buffer of the reference).
__global__ void k_gates_generic(const int32_t *__restrict__ ih, const int32_t *__restrict__ hh,
                                const int32_t *__restrict__ h_in, int32_t *__restrict__ h_out,
                                int32_t *__restrict__ v, int B, int H, const GateConsts *__restrict__ gcp,
                                const int32_t *__restrict__ tables) {
    const int j = blockIdx.x * blockDim.x + threadIdx.x;
    const int b = blockIdx.y;
    if (j >= H || b >= B) return;
    const size_t w = (size_t)b * 3 * H + j;
    int32_t gates[3];
    h_out[(size_t)b * H + j] = gru_cell<false>(*gcp, tables, ih[w], ih[w + H], ih[w + 2 * H], hh[w],
                                               hh[w + H], hh[w + 2 * H], h_in[(size_t)b * H + j], gates);
    if (v) {
        int32_t *vb = v + (size_t)b * 4 * H + j;
        vb[0] = gates[0];
        vb[H] = gates[1];
        vb[2 * H] = gates[2];
        vb[3 * H] = hh[w + 2 * H];
    }
}

// The training form of k_gates_generic: v as above plus the clamp masks of this step (each may be
// null): gate inputs and gate outputs [B][3H], new state [B][H]; 1 = not clamped.
__global__ void k_gates_train(const int32_t *__restrict__ ih, const int32_t *__restrict__ hh,
                              const int32_t *__restrict__ h_in, int32_t *__restrict__ h_out,
                              int32_t *__restrict__ v, uint8_t *__restrict__ m_in,
                              uint8_t *__restrict__ m_out, uint8_t *__restrict__ m_h, int B, int H,
                              const GateConsts *__restrict__ gcp) {
    const int j = blockIdx.x * blockDim.x + threadIdx.x;
    const int b = blockIdx.y;
    if (j >= H || b >= B) return;
    const size_t w = (size_t)b * 3 * H + j;
    int32_t gates[3];
    uint8_t keep[7];
    h_out[(size_t)b * H + j] = gru_cell_train(*gcp, ih[w], ih[w + H], ih[w + 2 * H], hh[w], hh[w + H],
                                              hh[w + 2 * H], h_in[(size_t)b * H + j], gates, keep);
    int32_t *vb = v + (size_t)b * 4 * H + j;
    vb[0] = gates[0];
    vb[H] = gates[1];
    vb[2 * H] = gates[2];
    vb[3 * H] = hh[w + 2 * H];
    if (m_in) { m_in[w] = keep[0]; m_in[w + H] = keep[1]; m_in[w + 2 * H] = keep[2]; }
    if (m_out) { m_out[w] = keep[3]; m_out[w + H] = keep[4]; m_out[w + 2 * H] = keep[5]; }
    if (m_h) m_h[(size_t)b * H + j] = keep[6];
}

}  // namespace qgru
