// Float-storage quantized forward: the reference's quantGRUForwardFP (src/gru_interface.cc:894-995,
// src/gru_forward_gpu_quant_fp.cu), inference mode.  Every tensor holds quantized values, but the
// requantization between operators is float arithmetic (round(x * scale_ratio)) and the gates
// are the real sigmoid / tanh on dequantized inputs - the arithmetic QAT trains against.
//
// The reference stores the quantized values in fp32 and multiplies with cuBLAS SGEMM.  Here the
// operands stay 8 bit: W*x runs on the tcgen05 int8 GEMM of the integer path with the float
// requantization (biasRescaleInline) as its epilogue, so W*x + bw is stored once, clamped, in one
// or two bytes; R*h runs as exact dp4a sums inside one persistent kernel that keeps its slice
// of R in shared memory for all T steps and applies the float cell.  An fp32 sum of integer
// products below 2^24 is exact too, so both sides see the same sums, and every float operation
// after them is PointwiseOperationsFP's, in its order: results agree with the reference bit for
// bit wherever its fp32 sums were exact.
//
// Included at the end of qgru_api.cu (it shares that file's kernels).
#pragma once
#include <cmath>
#include <cstring>
#include <vector>

#include "qgru_handle.h"
#include "qgru_internal.h"
#include "qgru_kernels.cuh"

namespace qgru {

// per-channel float arrays, one block of 4 * C floats on the device
struct FsChannels {
    const float *inv_gemm_x, *inv_bw, *inv_gemm_h, *inv_br;
};

// quantize_f (include/quantize_ops_helper.h:514-519): the zero point is added before rounding.
__device__ __forceinline__ float fs_quantize(float x, float scale, float zp, float lo, float hi) {
    return fs_clamp(rintf(x / scale + zp), lo, hi);
}

// fp32 activations -> 8-bit rows padded to Kpad; optionally the quantized values as floats.
__global__ void k_fs_quantize_rows(const float *__restrict__ x, uint8_t *__restrict__ out8,
                                   float *__restrict__ xq_out, long long rows, int K, int Kpad,
                                   float scale, float zp, float lo, float hi,
                                   uint8_t *__restrict__ keep = nullptr) {
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
            int q = 0;
            if (k < K) {
                const float raw = rintf(x[row * K + k] / scale + zp);
                const float qf = fs_clamp(raw, lo, hi);
                if (xq_out) xq_out[row * K + k] = qf;
                if (keep) keep[row * K + k] = (raw < lo || raw > hi) ? 0 : 1;
                q = (int)qf;
            }
            packed |= ((unsigned)q & 0xffu) << (8 * u);
        }
        reinterpret_cast<unsigned *>(out8)[i] = packed;
    }
}

// Initial state: quantize_f(h0) or the zero point (src/gru_interface.cc:949-961), into the
// 8-bit state rows and, dequantized, into slot `slot` of the output.
__global__ void k_fs_init_state(const float *__restrict__ h0, uint8_t *__restrict__ h8,
                                float *__restrict__ h_out, int B, int H, int Hpad, long long slot,
                                FsConsts fc, uint8_t *__restrict__ keep = nullptr) {
    const long long total = (long long)B * Hpad;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const int b = (int)(i / Hpad), j = (int)(i % Hpad);
        float q = 0.f;
        if (j < H) {
            const float raw = h0 ? rintf(h0[(size_t)b * H + j] / fc.h_scale + fc.zp_h) : fc.zp_h;
            q = fs_clamp(raw, fc.h_lo, fc.h_hi);
            h_out[slot * B * H + (long long)b * H + j] = (q - fc.zp_h) * fc.h_scale;
            if (keep) keep[(size_t)b * H + j] = (raw < fc.h_lo || raw > fc.h_hi) ? 0 : 1;
        }
        h8[i] = (uint8_t)(int)q;
    }
}

// Per-channel constants of the two linear layers, prepared once per parameter set:
// chan[0..2] = offset, bias term, GEMM ratio of W*x; chan[3..5] the same for R*h; each [3H].
__global__ void k_fs_channel_consts(const int32_t *__restrict__ wsum_x, const int32_t *__restrict__ wsum_h,
                                    const int32_t *__restrict__ bw_q, const int32_t *__restrict__ br_q,
                                    FsChannels ch, float zp_x, float zp_h, float *__restrict__ chan, int C) {
    const int m = blockIdx.x * blockDim.x + threadIdx.x;
    if (m >= C) return;
    chan[m] = fs_offset(wsum_x[m], zp_x);
    chan[C + m] = fs_bias_term(bw_q[m], ch.inv_bw[m]);
    chan[2 * C + m] = ch.inv_gemm_x[m];
    chan[3 * C + m] = fs_offset(wsum_h[m], zp_h);
    chan[4 * C + m] = fs_bias_term(br_q[m], ch.inv_br[m]);
    chan[5 * C + m] = ch.inv_gemm_h[m];
}

// Gate outputs over the whole clamped gate-input range, evaluated by the code that evaluates a
// gate directly (fs_activation), so a lookup returns exactly what the evaluation would.
__global__ void k_fs_tables(FsConsts fc, float *__restrict__ tab) {
    const int g = blockIdx.x;
    const int n = (int)(fc.in_hi[g] - fc.in_lo[g]) + 1;
    for (int i = threadIdx.x; i < n; i += blockDim.x)
        tab[fc.tab_off[g] + i] = fs_activation(fc, g, fc.in_lo[g] + (float)i);
}

// PointwiseOperationsFP<false, false> (src/gru_forward_gpu_quant_fp.cu:572-770) as its own launch:
// one thread per (hidden unit, batch row).  Used where the persistent kernel below has no plan.
template <typename IhT>
__global__ void k_fs_cell(const IhT *__restrict__ ih_q, const int32_t *__restrict__ hh_acc,
                          const float *__restrict__ chan, const uint8_t *__restrict__ h8_in,
                          uint8_t *__restrict__ h8_out, float *__restrict__ h_out, int B, int H, int Hpad,
                          FsConsts fc) {
    const int j = blockIdx.x * blockDim.x + threadIdx.x;
    const int b = blockIdx.y;
    if (j >= H || b >= B) return;
    const int C = 3 * H;
    const size_t w = (size_t)b * C + j;
    float ih[3], hh[3];
#pragma unroll
    for (int g = 0; g < 3; ++g) {
        const int m = j + g * H;
        ih[g] = (float)ih_q[w + g * H];     // requantized and clamped by the GEMM's epilogue
        hh[g] = fs_linear(hh_acc[w + g * H], chan[3 * C + m], chan[4 * C + m], chan[5 * C + m], fc.zp_hh,
                          fc.hh_lo, fc.hh_hi);
    }
    const float h_old = (float)state_byte(h8_in[(size_t)b * Hpad + j], fc.h_bits);
    const float h_new = fs_cell(fc, ih, hh, h_old);
    h8_out[(size_t)b * Hpad + j] = (uint8_t)(int)h_new;
    h_out[(size_t)b * H + j] = (h_new - fc.zp_h) * fc.h_scale;
}

// ---- training mode (quantGRUForwardFP with is_training): the per-step kernel also keeps the gate
// buffer v and the clamp masks, 1 = the value was inside its range before the clamp
// (clamp_f<true>, include/quantize_ops_helper.h:416-431).

// Dequantization constants of the four slots of v (dequantificationVFPInplace,
// src/quantize_ops.cu:368-397): update, reset, new gate outputs, R*h + br row of the new gate.
struct FsTrainConsts {
    float scale[4], zp[4];
};

__device__ __forceinline__ float fs_clamp_keep(float v, float lo, float hi, uint8_t &keep) {
    keep = (v < lo || v > hi) ? 0 : 1;
    return fs_clamp(v, lo, hi);
}
// biasRescaleInline<true>
__device__ __forceinline__ float fs_linear_keep(int acc, float off, float bias_term, float inv_gemm,
                                                float zp_out, float lo, float hi, uint8_t &keep) {
    const float val = __fsub_rn((float)acc, off);
    const float combined = __fadd_rn(val, bias_term);
    return fs_clamp_keep(rintf(__fmul_rn(combined, inv_gemm)) + zp_out, lo, hi, keep);
}
// real_sigmoid_f<true> / real_tanh_f<true> on an already clamped gate input
__device__ __forceinline__ float fs_activation_keep(const FsConsts &fc, int g, float in, uint8_t &keep) {
    const float x = (in - fc.zp_in[g]) * fc.s_in[g];
    const float y = g == 2 ? tanhf(x) : fs_sigmoid(x);
    return fs_clamp_keep(rintf(y / fc.s_out[g] + fc.zp_out[g]), fc.out_lo[g], fc.out_hi[g], keep);
}

// PointwiseOperationsFP<true, false> (src/gru_forward_gpu_quant_fp.cu:572-770) for one timestep.
// ih_acc / hh_acc: exact sums of W*x and R*h; masks point at this step's rows, any may be null.
__global__ void k_fs_cell_train(const int32_t *__restrict__ ih_acc, const int32_t *__restrict__ hh_acc,
                                const float *__restrict__ chan, const uint8_t *__restrict__ h8_in,
                                uint8_t *__restrict__ h8_out, float *__restrict__ h_out, float *__restrict__ v,
                                uint8_t *__restrict__ m_ih, uint8_t *__restrict__ m_hh, uint8_t *__restrict__ m_gin,
                                uint8_t *__restrict__ m_gout, uint8_t *__restrict__ m_h, int B, int H, int Hpad,
                                FsConsts fc, FsTrainConsts tc) {
    const int j = blockIdx.x * blockDim.x + threadIdx.x;
    const int b = blockIdx.y;
    if (j >= H || b >= B) return;
    const int C = 3 * H;
    const size_t w = (size_t)b * C + j;
    float ih[3], hh[3];
    uint8_t k_ih[3], k_hh[3], k_in[3], k_out[3], k_h;
#pragma unroll
    for (int g = 0; g < 3; ++g) {
        const int m = j + g * H;
        ih[g] = fs_linear_keep(ih_acc[w + g * H], chan[m], chan[C + m], chan[2 * C + m], fc.zp_ih, fc.ih_lo,
                               fc.ih_hi, k_ih[g]);
        hh[g] = fs_linear_keep(hh_acc[w + g * H], chan[3 * C + m], chan[4 * C + m], chan[5 * C + m], fc.zp_hh,
                               fc.hh_lo, fc.hh_hi, k_hh[g]);
    }
    float gate[2];
#pragma unroll
    for (int g = 0; g < 2; ++g) {
        const float a = rintf((ih[g] - fc.zp_ih) * fc.ih_to[g]);
        const float c = rintf((hh[g] - fc.zp_hh) * fc.hh_to[g]);
        const float in = fs_clamp_keep(a + c + fc.zp_in[g], fc.in_lo[g], fc.in_hi[g], k_in[g]);
        gate[g] = fs_activation_keep(fc, g, in, k_out[g]);
    }
    const float u = gate[0], r = gate[1];
    const float rh = rintf(((r - fc.zp_out[1]) * (hh[2] - fc.zp_hh)) * fc.rh_to_n);
    const float a_n = rintf((ih[2] - fc.zp_ih) * fc.ih_to[2]);
    const float in_n = fs_clamp_keep(a_n + rh + fc.zp_in[2], fc.in_lo[2], fc.in_hi[2], k_in[2]);
    const float n = fs_activation_keep(fc, 2, in_n, k_out[2]);
    const float h_old = (float)state_byte(h8_in[(size_t)b * Hpad + j], fc.h_bits);
    const float n_h = rintf((n - fc.zp_out[2]) * fc.n_to_h) + fc.zp_h;
    const float old_c = (u - fc.zp_out[0]) * (h_old - fc.zp_h);
    const float new_c = ((fc.one_q - u) - fc.zp_out[0]) * (n_h - fc.zp_h);
    const float h_new = fs_clamp_keep(rintf((old_c + new_c) * fc.uh_to_h) + fc.zp_h, fc.h_lo, fc.h_hi, k_h);
    h8_out[(size_t)b * Hpad + j] = (uint8_t)(int)h_new;
    h_out[(size_t)b * H + j] = (h_new - fc.zp_h) * fc.h_scale;
    float *vb = v + (size_t)b * 4 * H + j;
    vb[0] = (u - tc.zp[0]) * tc.scale[0];
    vb[H] = (r - tc.zp[1]) * tc.scale[1];
    vb[2 * H] = (n - tc.zp[2]) * tc.scale[2];
    vb[3 * H] = (hh[2] - tc.zp[3]) * tc.scale[3];
#pragma unroll
    for (int g = 0; g < 3; ++g) {
        if (m_ih) m_ih[w + g * H] = k_ih[g];
        if (m_hh) m_hh[w + g * H] = k_hh[g];
        if (m_gin) m_gin[w + g * H] = k_in[g];
        if (m_gout) m_gout[w + g * H] = k_out[g];
    }
    if (m_h) m_h[(size_t)b * H + j] = k_h;
}

// Clamp masks of the weight quantization (quantificationPerChannelFP<true>, src/quantize_ops.cu:
// 155-175): w [K][C] or [C], per-channel scales.
__global__ void k_fs_weight_mask(const float *__restrict__ w, long long n, int C, const float *__restrict__ scales,
                                 float lo, float hi, uint8_t *__restrict__ keep) {
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n;
         i += (long long)gridDim.x * blockDim.x) {
        const float q = rintf(w[i] / scales[i % C]);
        keep[i] = (q < lo || q > hi) ? 0 : 1;
    }
}

// The whole recurrence in one launch: k_recurrence_dp4a's organisation (a CTA keeps its slice of
// R in shared memory for all T steps, the P CTAs of a group of batch rows meet once per step at
// a counter in global memory, bounded spin) with the float-storage epilogue.  Shared memory:
// chan[3][3*Hs] floats (R*h side) | Rs[3][kw][Hs] words | hs[Bt][kw] words.
struct FsRecArgs {
    FsConsts fc;
    const void *ih_q;        // [T*B][3H] W*x + bw, requantized and clamped (int8 or int16)
    const float *chan;       // [6][3H]
};

template <bool HUnsigned, typename IhT>
__global__ void __launch_bounds__(256, 1) k_fs_recurrence(RecArgs a, FsRecArgs f) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int kw = a.Hpad >> 2;
    float *chan = reinterpret_cast<float *>(smem_raw);
    size_t off = ((size_t)9 * a.Hs * 4 + 15) & ~size_t(15);
    unsigned *Rs = reinterpret_cast<unsigned *>(smem_raw + off);
    off += (size_t)3 * kw * a.Hs * 4;
    unsigned *hs = reinterpret_cast<unsigned *>(smem_raw + off);

    const int grp = blockIdx.x / a.P, p = blockIdx.x % a.P;
    const int j0 = p * a.Hs, b0 = grp * a.Bt;
    const int nb = min(a.Bt, a.B - b0);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const FsConsts &fc = f.fc;

    for (int i = tid; i < 9 * a.Hs; i += 256) {          // the three arrays of the R*h side
        const int q = i / (3 * a.Hs), r = i % (3 * a.Hs);
        const int g = r / a.Hs, j = j0 + r % a.Hs;
        chan[i] = (j < a.H) ? f.chan[(size_t)(3 + q) * a.C + g * a.H + j] : 0.f;
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

    const int JW = a.Hs >> 5;
    const int BW = 8 / JW;
    const int wj = warp % JW, wb = warp / JW;
    const int jl = wj * 32 + lane, j = j0 + jl;
    const bool j_ok = j < a.H;
    constexpr int NB = 4;
    const size_t BH = (size_t)a.B * a.H;
    unsigned *bar = a.bar + grp * 32;
    const IhT *ihp = reinterpret_cast<const IhT *>(f.ih_q);
    bool dead = false;

    for (int s = 0; s < a.T; ++s) {
        const int t = a.reverse ? (a.T - 1 - s) : s;
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
            int32_t ihv[NB][3];
#pragma unroll
            for (int u = 0; u < NB; ++u) {
                const int b = bb + u;
#pragma unroll
                for (int g = 0; g < 3; ++g)
                    ihv[u][g] = (b < nb && j_ok) ? (int32_t)ihp[((size_t)t * a.B + b0 + b) * a.C + g * a.H + j] : 0;
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
                float ih[3], hh[3];
#pragma unroll
                for (int g = 0; g < 3; ++g) {
                    const int c = g * a.Hs + jl;
                    ih[g] = (float)ihv[u][g];
                    hh[g] = fs_linear(acc[u][g], chan[c], chan[3 * a.Hs + c], chan[6 * a.Hs + c], fc.zp_hh,
                                      fc.hh_lo, fc.hh_hi);
                }
                const uint8_t hb = reinterpret_cast<const uint8_t *>(hs)[(size_t)b * a.Hpad + j];
                const float h_old = HUnsigned ? (float)hb : (float)(int8_t)hb;
                const float hn = fs_cell(fc, ih, hh, h_old);
                h_nxt[(size_t)(b0 + b) * a.Hpad + j] = (uint8_t)(int)hn;
                a.hf_out[(size_t)out_slot * BH + (size_t)(b0 + b) * a.H + j] = (hn - fc.zp_h) * fc.h_scale;
            }
        }
        __syncthreads();
        if (a.P > 1 && tid == 0) {
            __threadfence();
            atomicAdd(bar, 1u);
        }
    }
}

namespace {

float op_lo(const qgru_op &o) { return (float)op_qmin(o); }
float op_hi(const qgru_op &o) { return (float)op_qmax(o); }

}  // namespace

// Training mode: what fstorage_forward does after its constants are ready when the caller wants
// the gate buffer v and the clamp masks.  Exact int32 sums of both products (dp4a GEMMs), then
// per step k_fs_cell_train; two launches per step, like the reference.
struct FsTrainArgs {
    const float *W, *R, *bw, *br;   // float master weights (device), for the weight masks; may be null
    float *v;                       // [T,B,4H] dequantized gate buffer
    qgru_train_masks m;
};

int fstorage_train_tail(qgru_handle *h, int T, int B, const float *x, const float *h0, float *h_out,
                        float *xq_out, unsigned flags, cudaStream_t st, const FsConsts &fc, const float *chan,
                        const FsTrainArgs &tr) {
    const qgru_params &p = h->p;
    const int H = h->H, C = h->C, I = h->I;
    const long long N = (long long)T * B;
    const bool pot2 = p.use_pot2 != 0;
    FsTrainConsts tc{};
    const int v_ops[4] = {QGRU_OP_UPDATE_OUT, QGRU_OP_RESET_OUT, QGRU_OP_NEW_OUT, QGRU_OP_HH_LINEAR};
    for (int k = 0; k < 4; ++k) {
        Rescale f;
        if (!to_fixed_scale(p.op[v_ops[k]].scale, pot2, &f)) return fail(h, QGRU_ERR_RANGE, "scale cannot be encoded");
        tc.scale[k] = decode_scale(f);
        tc.zp[k] = (float)p.op[v_ops[k]].zero_point;
    }
    int rc;
    if ((rc = ensure(h, h->x8, (size_t)((N + 127) / 128 * 128) * h->Ipad))) return rc;
    if ((rc = ensure(h, h->h8, (size_t)(2 * B + 256) * h->Hpad))) return rc;
    if ((rc = ensure(h, h->ih32, (size_t)N * C * 4))) return rc;
    if ((rc = ensure(h, h->hh32, (size_t)B * C * 4))) return rc;
    const qgru_op &ox = p.op[QGRU_OP_X];
    const bool rev = flags & QGRU_FLAG_REVERSE;
    const long long init_slot = rev ? T : 0;
    uint8_t *h8 = (uint8_t *)h->h8.p;
    const size_t h8_half = (size_t)B * h->Hpad;
    h->ev = h->ring[h->calls % qgru_handle::kRing];
    h->calls++;
    CK(cudaEventRecord(h->ev[0], st));
    CK(cudaMemsetAsync(h->d_flags, 0, 2 * sizeof(int), st));
    k_fs_quantize_rows<<<grid_for(N * (h->Ipad / 4), 256, h->sm_count), 256, 0, st>>>(
        x, (uint8_t *)h->x8.p, xq_out, N, I, h->Ipad, h->x_scale, fc.zp_x, op_lo(ox), op_hi(ox), tr.m.x);
    CK(cudaMemsetAsync(h8, 0, (size_t)(2 * B + 256) * h->Hpad, st));
    k_fs_init_state<<<grid_for((long long)B * h->Hpad, 256, h->sm_count), 256, 0, st>>>(
        h0, h8, h_out, B, H, h->Hpad, init_slot, fc, tr.m.h0);
    // weight masks: W [I][3H], R [H][3H], bw, br [3H] against their per-channel scales
    const float *wsrc[4] = {tr.W, tr.R, tr.bw, tr.br};
    uint8_t *wmask[4] = {tr.m.W, tr.m.R, tr.m.bw, tr.m.br};
    const long long wn[4] = {(long long)I * C, (long long)H * C, C, C};
    const int wop[4] = {QGRU_OP_W, QGRU_OP_R, QGRU_OP_BW, QGRU_OP_BR};
    for (int k = 0; k < 4; ++k)
        if (wsrc[k] && wmask[k])
            k_fs_weight_mask<<<grid_for(wn[k], 256, h->sm_count), 256, 0, st>>>(
                wsrc[k], wn[k], C, h->d_wscale[k], op_lo(p.op[wop[k]]), op_hi(p.op[wop[k]]), wmask[k]);
    CK(cudaEventRecord(h->ev[1], st));
    {
        dim3 grid((unsigned)((N + 63) / 64), (unsigned)((C + 63) / 64));
        if (h->x_uns)
            k_gemm_wx_simt<true, int32_t, true><<<grid, 256, 0, st>>>((const uint8_t *)h->x8.p, h->d_w8[0],
                                                                    (int32_t *)h->ih32.p, N, C, h->Ipad, LinearConsts{});
        else
            k_gemm_wx_simt<false, int32_t, true><<<grid, 256, 0, st>>>((const uint8_t *)h->x8.p, h->d_w8[0],
                                                                     (int32_t *)h->ih32.p, N, C, h->Ipad, LinearConsts{});
    }
    CK(cudaEventRecord(h->ev[2], st));
    const size_t BH = (size_t)B * H, BC = (size_t)B * C;
    for (int s = 0; s < T; ++s) {
        const int t = rev ? T - 1 - s : s;
        const size_t out_slot = rev ? (size_t)(T - 1 - s) : (size_t)(s + 1);
        const uint8_t *hin = h8 + (size_t)(s & 1) * h8_half;
        uint8_t *hout = h8 + (size_t)((s + 1) & 1) * h8_half;
        dim3 g1((unsigned)((B + 63) / 64), (unsigned)((C + 63) / 64));
        if (h->h_uns)
            k_gemm_wx_simt<true, int32_t, true><<<g1, 256, 0, st>>>(hin, h->d_w8[1], (int32_t *)h->hh32.p, B, C,
                                                                  h->Hpad, LinearConsts{});
        else
            k_gemm_wx_simt<false, int32_t, true><<<g1, 256, 0, st>>>(hin, h->d_w8[1], (int32_t *)h->hh32.p, B, C,
                                                                   h->Hpad, LinearConsts{});
        dim3 g2((H + 127) / 128, B);
        k_fs_cell_train<<<g2, 128, 0, st>>>(
            (const int32_t *)h->ih32.p + (size_t)t * BC, (const int32_t *)h->hh32.p, chan, hin, hout,
            h_out + out_slot * BH, tr.v + (size_t)t * B * 4 * H,
            tr.m.ih_linear ? tr.m.ih_linear + (size_t)t * BC : nullptr,
            tr.m.hh_linear ? tr.m.hh_linear + (size_t)t * BC : nullptr,
            tr.m.gate_input ? tr.m.gate_input + (size_t)t * BC : nullptr,
            tr.m.gate_output ? tr.m.gate_output + (size_t)t * BC : nullptr, tr.m.h ? tr.m.h + (size_t)t * BH : nullptr,
            B, H, h->Hpad, fc, tc);
    }
    h->launches += 4 + 2ull * T;
    CK(cudaGetLastError());
    CK(cudaEventRecord(h->ev[3], st));
    h->timing_valid = true;
    h->plan_text = "path=float_storage_training gemm=simt_dp4a_raw rec=per_step_float_cell_train";
    return QGRU_OK;
}

// Host side of quantGRUForwardFP, inference mode.  x, h0, h_out, xq_out are device pointers.
int fstorage_forward(qgru_handle *h, int T, int B, const float *x, const float *h0, float *h_out,
                     float *xq_out, unsigned flags, cudaStream_t st, const FsTrainArgs *train = nullptr) {
    if (!h->fast)
        return fail(h, QGRU_ERR_UNSUPPORTED,
                    "float-storage forward needs 8-bit W, R, x and h (the operands of the two products)");
    const qgru_params &p = h->p;
    const int H = h->H, C = h->C;
    const long long N = (long long)T * B;
    // ---- constants (setRescaleParam, src/gru_forward_gpu_quant_fp.cu:821-1003): float ratios
    // of the stored scales, computed in the same float operations
    FsConsts fc{};
    const qgru_op &ox = p.op[QGRU_OP_X], &oh = p.op[QGRU_OP_H], &oih = p.op[QGRU_OP_IH_LINEAR],
                  &ohh = p.op[QGRU_OP_HH_LINEAR];
    const int op_in[3] = {QGRU_OP_UPDATE_IN, QGRU_OP_RESET_IN, QGRU_OP_NEW_IN};
    const int op_out[3] = {QGRU_OP_UPDATE_OUT, QGRU_OP_RESET_OUT, QGRU_OP_NEW_OUT};
    fc.zp_x = (float)ox.zero_point;
    fc.zp_h = (float)oh.zero_point;
    fc.zp_ih = (float)oih.zero_point;
    fc.zp_hh = (float)ohh.zero_point;
    for (int g = 0; g < 3; ++g) {
        const qgru_op &i_ = p.op[op_in[g]], &o_ = p.op[op_out[g]];
        fc.zp_in[g] = (float)i_.zero_point;
        fc.zp_out[g] = (float)o_.zero_point;
        fc.s_in[g] = i_.scale;
        fc.s_out[g] = o_.scale;
        fc.ih_to[g] = oih.scale / i_.scale;
        if (g < 2) fc.hh_to[g] = ohh.scale / i_.scale;
        fc.in_lo[g] = op_lo(i_);
        fc.in_hi[g] = op_hi(i_);
        fc.out_lo[g] = op_lo(o_);
        fc.out_hi[g] = op_hi(o_);
    }
    const qgru_op &ou = p.op[QGRU_OP_UPDATE_OUT], &orr = p.op[QGRU_OP_RESET_OUT], &on = p.op[QGRU_OP_NEW_OUT];
    fc.rh_to_n = (orr.scale * ohh.scale) / p.op[QGRU_OP_NEW_IN].scale;
    fc.one_q = rintf(1.0f / ou.scale) + (float)ou.zero_point;
    fc.uh_to_h = (ou.scale * oh.scale) / oh.scale;
    fc.n_to_h = on.scale / oh.scale;
    fc.ih_lo = op_lo(oih); fc.ih_hi = op_hi(oih);
    fc.hh_lo = op_lo(ohh); fc.hh_hi = op_hi(ohh);
    fc.h_lo = op_lo(oh); fc.h_hi = op_hi(oh);
    fc.h_scale = h->h_scale;
    fc.h_bits = h->h_uns ? 9 : 8;

    // gate tables where every gate input has at most 10 bits (3 x 1024 floats of shared memory);
    // option cell=generic keeps the tables out of the kernels (every gate is evaluated)
    bool tab_possible = true;
    int tab_total = 0;
    for (int g = 0; g < 3; ++g) {
        const int n = (int)(fc.in_hi[g] - fc.in_lo[g]) + 1;
        if (n > 1024) tab_possible = false;
        fc.tab_off[g] = tab_total;
        tab_total += n;
    }
    fc.tab_on = (tab_possible && h->opt_cell != 1) ? 1 : 0;
    const int n_tab = fc.tab_on ? tab_total : 0;

    int rc;
    // per-channel constants: 4 x C scale ratios from the host, then 6 x C derived on the device
    // from the packed weights (column sums, quantized biases); then the gate tables
    if ((rc = ensure(h, h->fs_ch, ((size_t)10 * C + 3 * 1024) * sizeof(float)))) return rc;
    float *chp = (float *)h->fs_ch.p;
    float *chan = chp + (size_t)4 * C;
    float *gate_tab = chp + (size_t)10 * C;
    if (!h->fs_ready) {
        std::vector<float> hostc((size_t)4 * C);
        for (int m = 0; m < C; ++m) {
            const float s_wx = h->sc[0][m] * ox.scale;
            hostc[m] = s_wx / oih.scale;                 // inv_div_gemm_x_to_weight_ih_linear
            hostc[C + m] = h->sc[2][m] / s_wx;           // inv_div_bw_to_gemm_x
            const float s_rh = h->sc[1][m] * oh.scale;
            hostc[2 * C + m] = s_rh / ohh.scale;
            hostc[3 * C + m] = h->sc[3][m] / s_rh;
        }
        CK(cudaMemcpyAsync(chp, hostc.data(), hostc.size() * sizeof(float), cudaMemcpyHostToDevice, st));
        CK(cudaStreamSynchronize(st));   // hostc leaves scope
        const FsChannels ch{chp, chp + C, chp + 2 * C, chp + 3 * C};
        k_fs_channel_consts<<<(C + 127) / 128, 128, 0, st>>>(h->d_wsum[0], h->d_wsum[1], h->d_wq[2], h->d_wq[3], ch,
                                                            fc.zp_x, fc.zp_h, chan, C);
        if (tab_possible) k_fs_tables<<<3, 256, 0, st>>>(fc, gate_tab);
        CK(cudaGetLastError());
        h->launches += 2;
        h->fs_ready = true;
    }
    if (train) return fstorage_train_tail(h, T, B, x, h0, h_out, xq_out, flags, st, fc, chan, *train);

    if ((rc = ensure(h, h->x8, (size_t)((N + 127) / 128 * 128) * h->Ipad))) return rc;
    if ((rc = ensure(h, h->h8, (size_t)(2 * B + 256) * h->Hpad))) return rc;
    // W*x + bw requantized and clamped to the width of weight_ih_linear: one or two bytes
    const int ih_bytes = (oih.bits <= 8 && !oih.is_unsigned) ? 1 : 2;
    if (oih.bits > 16 || (oih.bits == 16 && oih.is_unsigned))
        return fail(h, QGRU_ERR_UNSUPPORTED, "float-storage forward stores W*x + bw in at most 16 signed bits");
    if ((rc = ensure(h, h->ih, (size_t)N * C * ih_bytes))) return rc;
    const bool rev = flags & QGRU_FLAG_REVERSE;
    const long long init_slot = rev ? T : 0;
    uint8_t *h8 = (uint8_t *)h->h8.p;
    const size_t h8_half = (size_t)B * h->Hpad;
    const int sms = h->opt_sm_limit > 0 ? std::min(h->opt_sm_limit, h->sm_count) : h->sm_count;

    h->ev = h->ring[h->calls % qgru_handle::kRing];
    h->calls++;
    CK(cudaEventRecord(h->ev[0], st));
    CK(cudaMemsetAsync(h->d_flags, 0, 2 * sizeof(int), st));
    k_fs_quantize_rows<<<grid_for(N * (h->Ipad / 4), 256, h->sm_count), 256, 0, st>>>(
        x, (uint8_t *)h->x8.p, xq_out, N, h->I, h->Ipad, h->x_scale, fc.zp_x, op_lo(ox), op_hi(ox));
    CK(cudaMemsetAsync(h8, 0, (size_t)(2 * B + 256) * h->Hpad, st));
    k_fs_init_state<<<grid_for((long long)B * h->Hpad, 256, h->sm_count), 256, 0, st>>>(
        h0, h8, h_out, B, H, h->Hpad, init_slot, fc);
    CK(cudaEventRecord(h->ev[1], st));
    // the input projection: exact int32 sums on the tensor cores (dp4a form as fallback), float
    // requantization in the epilogue
    LinearConsts lcx = linear_consts(h, 0);
    lcx.fs = chan;
    lcx.fs_C = C;
    bool used_tc = false;
    if (h->opt_gemm != 1) {
        PreScale ps{};
        rc = tc_gemm_launch(h->tc, (const uint8_t *)h->x8.p, (N + 127) / 128 * 128, h->d_w8[0], h->w8_rows[0],
                            h->ih.p, N, C, h->Ipad, h->x_uns, ih_bytes, lcx, ps, false, false, h->d_flags + 1, sms, st,
                            &h->err);
        if (rc == QGRU_OK) used_tc = true;
        else if (rc != QGRU_ERR_UNSUPPORTED || h->opt_gemm == 2) return rc;
    }
    if (!used_tc) {
        dim3 grid((unsigned)((N + 63) / 64), (unsigned)((C + 63) / 64));
        const uint8_t *x8 = (const uint8_t *)h->x8.p;
        if (ih_bytes == 1) {
            if (h->x_uns) k_gemm_wx_simt<true, int8_t><<<grid, 256, 0, st>>>(x8, h->d_w8[0], (int8_t *)h->ih.p, N, C, h->Ipad, lcx);
            else k_gemm_wx_simt<false, int8_t><<<grid, 256, 0, st>>>(x8, h->d_w8[0], (int8_t *)h->ih.p, N, C, h->Ipad, lcx);
        } else {
            if (h->x_uns) k_gemm_wx_simt<true, int16_t><<<grid, 256, 0, st>>>(x8, h->d_w8[0], (int16_t *)h->ih.p, N, C, h->Ipad, lcx);
            else k_gemm_wx_simt<false, int16_t><<<grid, 256, 0, st>>>(x8, h->d_w8[0], (int16_t *)h->ih.p, N, C, h->Ipad, lcx);
        }
        CK(cudaGetLastError());
    }
    CK(cudaEventRecord(h->ev[2], st));
    h->launches += 3;
    char buf[256];
    RecPlan pl;
    RecMmaPlan cp;
    // the tensor-core recurrence of the integer path (one cluster per group of batch rows, h_t
    // exchanged through distributed shared memory) with the float cell as its epilogue
    // (small batches of a narrow layer run faster on the SIMT forms below: measured 0.17 ms against
    // 0.28 ms at H = 128, B = 32 and 4.1 against 4.6 us per step at H = 256, B = 1)
    const bool small = (h->opt_rec == 0 || h->opt_rec == 4) && h->Hpad <= 256 && B <= sms;
    const bool cluster_ok = !small && h->opt_rec != 1 && h->opt_rec != 3 && h->opt_exchange != 1 &&
                            rec_cluster_plan(H, h->Hpad, B, sms, h->smem_optin, n_tab, h->opt_r_where, h->opt_mt, h->opt_ng, h->opt_kp, &cp);
    if (cluster_ok) {
        if (cp.G > h->bar_groups) {
            if ((rc = alloc_dev(h, &h->d_bar, (size_t)cp.G * 32))) return rc;
            h->bar_groups = cp.G;
        }
        CK(cudaMemsetAsync(h->d_bar, 0, (size_t)cp.G * 32 * sizeof(unsigned), st));
        RecMmaArgs a;
        a.T = T; a.B = B; a.H = H; a.Hpad = h->Hpad; a.C = C;
        a.P = cp.P; a.NB = cp.NB; a.b_off = 0; a.b_cnt = B;
        a.reverse = rev ? 1 : 0;
        a.tmem_cols = (uint32_t)cp.tmem_cols;
        a.ih = h->ih.p;
        a.h8 = h8;
        a.hq_out = nullptr;
        a.hf_out = h_out;
        a.lc = linear_consts(h, 1);
        a.tables = (const int32_t *)gate_tab;   // float bit patterns
        a.n_table = n_tab;
        a.bar = h->d_bar;
        a.abort_flag = h->d_flags + 1;
        a.spin_limit = h->spin_limit;
        a.fs_on = 1;
        a.fs_chan = chan + (size_t)3 * C;
        a.fs = fc;
        const unsigned long long before = h->rec_cl.launches;
        rc = rec_cluster_launch(h->rec_cl, cp, a, h->gc_host, h->d_w8[1], h->w8_rows[1], (long long)2 * B + 256,
                                h->h_uns, ih_bytes, false, false, false, false, st, &h->err);
        if (rc) return rc;
        h->launches += h->rec_cl.launches - before;
        snprintf(buf, sizeof(buf), "path=float_storage gemm=%s rec=tcgen05_i8_float_cell exchange=cluster_dsmem NB=%d NG=%d P=%d G=%d smem=%zu tmem_cols=%d ih_bytes=%d gates=%s",
                 used_tc ? "tcgen05_i8" : "simt_dp4a", cp.NB, cp.NG, cp.P, cp.G, cp.smem, cp.tmem_cols, ih_bytes,
                 fc.tab_on ? "tabulated" : "evaluated");
    } else if ((h->opt_rec == 0 || h->opt_rec == 4) && h->Hpad <= 256 && B <= sms &&
               gemv_smem(h, n_tab) <= (size_t)h->smem_optin) {
        // one CTA per batch row, the whole R in shared memory, no synchronisation between CTAs
        RecArgs a{};
        a.T = T; a.B = B; a.H = H; a.Hpad = h->Hpad; a.C = C;
        a.reverse = rev ? 1 : 0;
        a.r8 = h->d_w8[1];
        a.ih = h->ih.p;
        a.h8 = h8;
        a.hf_out = h_out;
        a.lc = linear_consts(h, 1);
        a.gc = h->d_gc;
        a.tables = (const int32_t *)gate_tab;   // float bit patterns
        a.n_table = n_tab;
        a.abort_flag = h->d_flags + 1;
        a.spin_limit = h->spin_limit;
        a.fs_chan = chan + (size_t)3 * C;
        a.fs = fc;
        // R in registers where the form exists (Hpad 128 or 256; option gemv_r=smem: in shared memory)
        const bool in_regs = h->opt_gemv_r != 1 && (h->Hpad == 128 || h->Hpad == 256);
        size_t smem;
        if (in_regs) {
            const size_t units = (size_t)(H + 31) / 32 * 32;
            smem = (((size_t)n_tab * 4 + 15) & ~size_t(15)) + (size_t)2 * 2 * (h->Hpad / 2 + 16) + 3 * units * sizeof(int) +
                   9 * units * sizeof(float);
            auto kern = h->Hpad == 128
                            ? (ih_bytes == 1 ? (h->h_uns ? k_recurrence_gemv_reg<true, int8_t, 64, 3> : k_recurrence_gemv_reg<false, int8_t, 64, 3>)
                                             : (h->h_uns ? k_recurrence_gemv_reg<true, int16_t, 64, 3> : k_recurrence_gemv_reg<false, int16_t, 64, 3>))
                            : (ih_bytes == 1 ? (h->h_uns ? k_recurrence_gemv_reg<true, int8_t, 128, 3> : k_recurrence_gemv_reg<false, int8_t, 128, 3>)
                                             : (h->h_uns ? k_recurrence_gemv_reg<true, int16_t, 128, 3> : k_recurrence_gemv_reg<false, int16_t, 128, 3>));
            CK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            kern<<<B, 2 * (int)units, smem, st>>>(h->gc_host, a);
        } else {
            auto kern = ih_bytes == 1 ? (h->h_uns ? k_recurrence_gemv<true, int8_t, 3> : k_recurrence_gemv<false, int8_t, 3>)
                                      : (h->h_uns ? k_recurrence_gemv<true, int16_t, 3> : k_recurrence_gemv<false, int16_t, 3>);
            smem = gemv_smem(h, n_tab);
            CK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            const int threads = 4 * ((H + 31) / 32 * 32);
            kern<<<B, threads, smem, st>>>(h->gc_host, a);
        }
        CK(cudaGetLastError());
        h->launches++;
        snprintf(buf, sizeof(buf), "path=float_storage gemm=%s rec=gemv_float_cell r_in=%s rows_per_cta=1 ctas=%d smem=%zu ih_bytes=%d gates=%s",
                 used_tc ? "tcgen05_i8" : "simt_dp4a", in_regs ? "registers" : "smem", B, smem, ih_bytes, fc.tab_on ? "tabulated" : "evaluated");
    } else if (h->opt_rec != 3 && plan_recurrence(h, B, &pl)) {
        // the whole recurrence in one launch
        if (pl.G > h->bar_groups) {
            if ((rc = alloc_dev(h, &h->d_bar, (size_t)pl.G * 32))) return rc;
            h->bar_groups = pl.G;
        }
        CK(cudaMemsetAsync(h->d_bar, 0, (size_t)pl.G * 32 * sizeof(unsigned), st));
        RecArgs a{};
        a.T = T; a.B = B; a.H = H; a.Hpad = h->Hpad; a.C = C;
        a.Hs = pl.Hs; a.Bt = pl.Bt; a.P = pl.P;
        a.reverse = rev ? 1 : 0;
        a.r8 = h->d_w8[1];
        a.h8 = h8;
        a.hf_out = h_out;
        a.bar = h->d_bar;
        a.abort_flag = h->d_flags + 1;
        a.spin_limit = h->spin_limit;
        FsRecArgs f{fc, h->ih.p, chan};
        auto kern = ih_bytes == 1 ? (h->h_uns ? k_fs_recurrence<true, int8_t> : k_fs_recurrence<false, int8_t>)
                                  : (h->h_uns ? k_fs_recurrence<true, int16_t> : k_fs_recurrence<false, int16_t>);
        CK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pl.smem));
        const int grid = pl.G * pl.P;
        if (pl.P > 1) {
            if (!h->coop) return fail(h, QGRU_ERR_UNSUPPORTED, "device lacks cooperative launch");
            int per_sm = 0;
            CK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, 256, pl.smem));
            if ((long long)per_sm * h->sm_count < grid)
                return fail(h, QGRU_ERR_UNSUPPORTED, "recurrence grid cannot be co-resident");
            void *args[] = {&a, &f};
            CK(cudaLaunchCooperativeKernel((void *)kern, dim3(grid), dim3(256), args, pl.smem, st));
        } else {
            kern<<<grid, 256, pl.smem, st>>>(a, f);
            CK(cudaGetLastError());
        }
        h->launches++;
        snprintf(buf, sizeof(buf), "path=float_storage gemm=%s rec=dp4a_float_cell Hs=%d Bt=%d P=%d G=%d smem=%zu ih_bytes=%d",
                 used_tc ? "tcgen05_i8" : "simt_dp4a", pl.Hs, pl.Bt, pl.P, pl.G, pl.smem, ih_bytes);
    } else {
        // two launches per step, as the reference
        if ((rc = ensure(h, h->hh32, (size_t)B * C * 4))) return rc;
        const size_t BH = (size_t)B * H;
        for (int s = 0; s < T; ++s) {
            const int t = rev ? T - 1 - s : s;
            const size_t out_slot = rev ? (size_t)(T - 1 - s) : (size_t)(s + 1);
            const uint8_t *hin = h8 + (size_t)(s & 1) * h8_half;
            uint8_t *hout = h8 + (size_t)((s + 1) & 1) * h8_half;
            dim3 g1((unsigned)((B + 63) / 64), (unsigned)((C + 63) / 64));
            if (h->h_uns)
                k_gemm_wx_simt<true, int32_t, true><<<g1, 256, 0, st>>>(hin, h->d_w8[1], (int32_t *)h->hh32.p, B, C,
                                                                      h->Hpad, LinearConsts{});
            else
                k_gemm_wx_simt<false, int32_t, true><<<g1, 256, 0, st>>>(hin, h->d_w8[1], (int32_t *)h->hh32.p, B, C,
                                                                       h->Hpad, LinearConsts{});
            dim3 g2((H + 127) / 128, B);
            if (ih_bytes == 1)
                k_fs_cell<int8_t><<<g2, 128, 0, st>>>((const int8_t *)h->ih.p + (size_t)t * B * C, (const int32_t *)h->hh32.p,
                                                      chan, hin, hout, h_out + out_slot * BH, B, H, h->Hpad, fc);
            else
                k_fs_cell<int16_t><<<g2, 128, 0, st>>>((const int16_t *)h->ih.p + (size_t)t * B * C, (const int32_t *)h->hh32.p,
                                                       chan, hin, hout, h_out + out_slot * BH, B, H, h->Hpad, fc);
            h->launches += 2;
        }
        snprintf(buf, sizeof(buf), "path=float_storage gemm=%s rec=per_step_float_cell ih_bytes=%d",
                 used_tc ? "tcgen05_i8" : "simt_dp4a", ih_bytes);
    }
    CK(cudaGetLastError());
    CK(cudaEventRecord(h->ev[3], st));
    h->timing_valid = true;
    h->plan_text = buf;
    return QGRU_OK;
}

}  // namespace qgru

extern "C" {

int qgru_forward_fstorage(qgru_handle *h, int T, int B, const float *x, const float *h0, float *h_out,
                          float *x_q_out, unsigned flags, void *stream) {
    if (!h || !x || !h_out) return QGRU_ERR_BAD_ARG;
    if (T <= 0 || B <= 0) return fail(h, QGRU_ERR_BAD_ARG, "T and B must be positive");
    if (!h->params_set || !h->weights_set)
        return fail(h, QGRU_ERR_NOT_READY, "set_params and set_weights first");
    CK(cudaSetDevice(h->device));
    return qgru::fstorage_forward(h, T, B, x, h0, h_out, x_q_out, flags, (cudaStream_t)stream);
}

// out[i] = q[i] * scale[i % C]  (dequantizeGRUWeights: weights have zero point 0)
__global__ void k_dequantize_weights(const int32_t *__restrict__ q, float *__restrict__ out, long long n, int C,
                                     const float *__restrict__ scales) {
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n;
         i += (long long)gridDim.x * blockDim.x)
        out[i] = (float)q[i] * scales[i % C];
}
// out[i] = (q[i] - zp) * scale on float-stored quantized values (dequantize_f)
__global__ void k_dequantize_fq(const float *__restrict__ q, float *__restrict__ out, long long n, float scale,
                                float zp) {
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n;
         i += (long long)gridDim.x * blockDim.x)
        out[i] = (q[i] - zp) * scale;
}

int qgru_get_weights_dequantized(qgru_handle *h, float *W, float *R, float *bw, float *br, void *stream) {
    if (!h) return QGRU_ERR_BAD_ARG;
    if (!h->weights_set) return fail(h, QGRU_ERR_NOT_READY, "set_weights first");
    CK(cudaSetDevice(h->device));
    cudaStream_t st = (cudaStream_t)stream;
    const int C = h->C;
    const long long n[4] = {(long long)h->I * C, (long long)h->H * C, C, C};
    float *dst[4] = {W, R, bw, br};
    for (int k = 0; k < 4; ++k)
        if (dst[k])
            k_dequantize_weights<<<grid_for(n[k], 256, h->sm_count), 256, 0, st>>>(h->d_wq[k], dst[k], n[k], C,
                                                                                h->d_wscale[k]);
    CK(cudaGetLastError());
    return QGRU_OK;
}

int qgru_dequantize_f32(qgru_handle *h, int op, const float *q, float *out, long long n, void *stream) {
    if (!h || !q || !out || op < 0 || op >= QGRU_NUM_OPS || n < 0) return QGRU_ERR_BAD_ARG;
    if (!h->params_set) return fail(h, QGRU_ERR_NOT_READY, "set_params first");
    CK(cudaSetDevice(h->device));
    Rescale f;
    if (!to_fixed_scale(h->p.op[op].scale, h->p.use_pot2 != 0, &f)) return fail(h, QGRU_ERR_RANGE, "scale cannot be encoded");
    if (n)
        k_dequantize_fq<<<grid_for(n, 256, h->sm_count), 256, 0, (cudaStream_t)stream>>>(
            q, out, n, decode_scale(f), (float)h->p.op[op].zero_point);
    CK(cudaGetLastError());
    return QGRU_OK;
}

int qgru_forward_fstorage_train(qgru_handle *h, int T, int B, const float *W, const float *R, const float *bw,
                                const float *br, const float *x, const float *h0, float *h_out, float *v_out,
                                float *x_q_out, const qgru_train_masks *masks, unsigned flags, void *stream) {
    if (!h || !x || !h_out || !v_out) return QGRU_ERR_BAD_ARG;
    if (T <= 0 || B <= 0) return fail(h, QGRU_ERR_BAD_ARG, "T and B must be positive");
    if (!h->params_set || !h->weights_set)
        return fail(h, QGRU_ERR_NOT_READY, "set_params and set_weights first");
    CK(cudaSetDevice(h->device));
    qgru::FsTrainArgs tr{W, R, bw, br, v_out, masks ? *masks : qgru_train_masks{}};
    return qgru::fstorage_forward(h, T, B, x, h0, h_out, x_q_out, flags, (cudaStream_t)stream, &tr);
}

}  // extern "C"
