// qgru_float.cu - the unquantized fp32 GRU ("float mode") and the MinMax calibration pass.
//
// Float mode follows hasteGRUForward / ForwardPass<float> of the reference
// (src/gru_interface.cc:173-207, src/gru_forward_gpu.cu:23-125, 342-414): one GEMM for W*x
// over all timesteps, then per step R*h and the pointwise gate kernel; here the per-step
// GEMV and the gates are one kernel.  Calibration runs the same forward and folds the
// min/max of every operator while the values are still in registers - the reference
// materialises five capture tensors and seven temporaries of T*B*H floats and reduces each in
// its own pass (src/calibration_gpu.cu:1776-1953).
#include <cfloat>

#include "qgru_handle.h"

using namespace qgru;

namespace {

// ---- order-preserving float <-> uint mapping so min/max can use integer atomics
__device__ __forceinline__ unsigned f2key(float f) {
    const unsigned u = __float_as_uint(f);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
inline float key2f(unsigned k) {
    const unsigned u = (k & 0x80000000u) ? (k & 0x7fffffffu) : ~k;
    float f;
    memcpy(&f, &u, 4);
    return f;
}
constexpr unsigned KEY_EMPTY_MIN = 0xffffffffu;  // larger than every finite key
constexpr unsigned KEY_EMPTY_MAX = 0u;

struct MinMax {
    float mn, mx;
    __device__ __forceinline__ void init() { mn = FLT_MAX; mx = -FLT_MAX; }
    // NaN and Inf are skipped, as the reference's reductions do (src/calibration_gpu.cu:254-259)
    __device__ __forceinline__ void add(float v) {
        if (isfinite(v)) { mn = fminf(mn, v); mx = fmaxf(mx, v); }
    }
};

__device__ __forceinline__ void warp_fold(MinMax m, unsigned *acc_min, unsigned *acc_max, int slot,
                                          bool any) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        m.mn = fminf(m.mn, __shfl_xor_sync(0xffffffffu, m.mn, o));
        m.mx = fmaxf(m.mx, __shfl_xor_sync(0xffffffffu, m.mx, o));
    }
    if (any && (threadIdx.x & 31) == 0 && m.mn <= m.mx) {
        atomicMin(acc_min + slot, f2key(m.mn));
        atomicMax(acc_max + slot, f2key(m.mx));
    }
}

// ---- C[n][c] = sum_k x[n][k] * W[k][c]   (fp32, 64x64 tile, 4x4 per thread)
__global__ void __launch_bounds__(256)
k_sgemm_xw(const float *__restrict__ x, const float *__restrict__ W, float *__restrict__ out,
           long long N, int K, int Cn) {
    __shared__ float xs[16][64 + 1];
    __shared__ float ws[16][64];
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const long long n0 = (long long)blockIdx.x * 64;
    const int c0 = blockIdx.y * 64;
    float acc[4][4] = {};
    for (int k0 = 0; k0 < K; k0 += 16) {
        for (int i = threadIdx.x; i < 64 * 16; i += 256) {
            const int r = i >> 4, kk = i & 15;
            xs[kk][r] = (n0 + r < N && k0 + kk < K) ? x[(n0 + r) * K + k0 + kk] : 0.f;
            const int kr = i >> 6, cc = i & 63;
            ws[kr][cc] = (k0 + kr < K && c0 + cc < Cn) ? W[(size_t)(k0 + kr) * Cn + c0 + cc] : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < 16; ++kk) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = xs[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = ws[kk][tx + 16 * j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const long long n = n0 + ty * 4 + i;
        if (n >= N) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int c = c0 + tx + 16 * j;
            if (c < Cn) out[n * Cn + c] = acc[i][j];
        }
    }
}

// ---- one timestep after R*h has been multiplied (k_sgemm_xw on h_{t-1}): the float gates of
// src/gru_forward_gpu.cu:23-125 for (b, j).  rh [B][3H] holds R*h without its bias.
template <bool Calib>
__global__ void __launch_bounds__(256)
k_float_step(const float *__restrict__ wx, const float *__restrict__ rh, const float *__restrict__ bw,
             const float *__restrict__ br, const float *__restrict__ h_in, float *__restrict__ h_out,
             float *__restrict__ v, int v_stride, int B, int H, unsigned *acc_min, unsigned *acc_max) {
    const int j = blockIdx.x * 128 + (threadIdx.x & 127);
    const int b = blockIdx.y * 2 + (threadIdx.x >> 7);
    const bool ok = j < H && b < B;
    const int Cn = 3 * H;
    MinMax m_h, m_ih, m_hh, m_zin, m_rin, m_nin, m_z, m_r, m_n, m_rh, m_new, m_old;
    if (Calib) {
        m_h.init(); m_ih.init(); m_hh.init(); m_zin.init(); m_rin.init(); m_nin.init();
        m_z.init(); m_r.init(); m_n.init(); m_rh.init(); m_new.init(); m_old.init();
    }
    if (ok) {
        const float *rhr = rh + (size_t)b * Cn + j;
        const float az = rhr[0], ar = rhr[H], an = rhr[2 * H];
        const float *wxr = wx + (size_t)b * Cn + j;
        const float wz = wxr[0] + bw[j], rz = az + br[j];
        const float z_pre = wz + rz;
        const float z = 1.0f / (1.0f + expf(-z_pre));
        const float wr = wxr[H] + bw[H + j], rr_ = ar + br[H + j];
        const float r_pre = wr + rr_;
        const float r = 1.0f / (1.0f + expf(-r_pre));
        const float wg = wxr[2 * H] + bw[2 * H + j], rg = an + br[2 * H + j];
        const float g_pre = wg + r * rg;
        const float g = tanhf(g_pre);
        const float h_old = h_in[(size_t)b * H + j];
        const float old_c = z * h_old;
        const float new_c = (1.0f - z) * g;
        const float hn = old_c + new_c;
        h_out[(size_t)b * H + j] = hn;
        if (v) {
            // 4 slots per row: the reference's training buffer (z, r, n, Rh_n + br_n); 6 slots:
            // all three R*h + br rows as well (z, r, n, Rh_z+br_z, Rh_r+br_r, Rh_n+br_n)
            float *vb = v + (size_t)b * v_stride * H + j;
            vb[0] = z; vb[H] = r; vb[2 * H] = g;
            if (v_stride == 6) { vb[3 * H] = rz; vb[4 * H] = rr_; vb[5 * H] = rg; }
            else vb[3 * H] = rg;
        }
        if (Calib) {
            m_h.add(hn);
            m_ih.add(wz); m_ih.add(wr); m_ih.add(wg);
            m_hh.add(rz); m_hh.add(rr_); m_hh.add(rg);
            m_zin.add(z_pre); m_rin.add(r_pre); m_nin.add(g_pre);
            m_z.add(z); m_r.add(r); m_n.add(g);
            m_rh.add(r * rg); m_new.add(new_c); m_old.add(old_c);
        }
    }
    if (Calib) {
        warp_fold(m_h, acc_min, acc_max, QGRU_OP_H, true);
        warp_fold(m_ih, acc_min, acc_max, QGRU_OP_IH_LINEAR, true);
        warp_fold(m_hh, acc_min, acc_max, QGRU_OP_HH_LINEAR, true);
        warp_fold(m_zin, acc_min, acc_max, QGRU_OP_UPDATE_IN, true);
        warp_fold(m_rin, acc_min, acc_max, QGRU_OP_RESET_IN, true);
        warp_fold(m_nin, acc_min, acc_max, QGRU_OP_NEW_IN, true);
        warp_fold(m_z, acc_min, acc_max, QGRU_OP_UPDATE_OUT, true);
        warp_fold(m_r, acc_min, acc_max, QGRU_OP_RESET_OUT, true);
        warp_fold(m_n, acc_min, acc_max, QGRU_OP_NEW_OUT, true);
        warp_fold(m_rh, acc_min, acc_max, QGRU_OP_MUL_RESET_HIDDEN, true);
        warp_fold(m_new, acc_min, acc_max, QGRU_OP_MUL_NEW_CONTRIB, true);
        warp_fold(m_old, acc_min, acc_max, QGRU_OP_MUL_OLD_CONTRIB, true);
    }
}

// min/max of a whole tensor into slot `slot` (warp shuffles, one atomic pair per warp)
__global__ void k_minmax_tensor(const float *__restrict__ x, long long n, unsigned *acc_min,
                                unsigned *acc_max, int slot) {
    MinMax m;
    m.init();
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n;
         i += (long long)gridDim.x * blockDim.x)
        m.add(x[i]);
    warp_fold(m, acc_min, acc_max, slot, true);
}

// per-channel min/max of a [K][Cn] matrix: one warp per 32 channels, coalesced over channels
__global__ void k_minmax_channels(const float *__restrict__ w, int K, int Cn, unsigned *cmin,
                                  unsigned *cmax) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= Cn) return;
    MinMax m;
    m.init();
    for (int k = 0; k < K; ++k) m.add(w[(size_t)k * Cn + c]);
    if (m.mn <= m.mx) {
        cmin[c] = f2key(m.mn);
        cmax[c] = f2key(m.mx);
    } else {
        cmin[c] = KEY_EMPTY_MIN;
        cmax[c] = KEY_EMPTY_MAX;
    }
}

__global__ void k_fill_u32(unsigned *p, int n, unsigned v) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) p[i] = v;
}

__global__ void k_init_h_float(const float *__restrict__ h0, float *__restrict__ h, long long n) {
    const long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
    if (i < n) h[i] = h0 ? h0[i] : 0.f;
}

}  // namespace

namespace qgru {

int float_forward(qgru_handle *h, int T, int B, const float *W, const float *R, const float *bw,
                  const float *br, const float *x, const float *h0, float *h_out, float *v_out,
                  int v_stride, unsigned *acc_min, unsigned *acc_max, cudaStream_t st) {
    const int H = h->H, Cn = h->C, I = h->I;
    const long long N = (long long)T * B;
    int rc;
    if ((rc = ensure(h, h->f_wx, (size_t)N * Cn * 4))) return rc;
    float *wx = (float *)h->f_wx.p;
    const long long NH = (long long)B * H;
    k_init_h_float<<<(unsigned)((NH + 255) / 256), 256, 0, st>>>(h0, h_out, NH);
    dim3 gg((unsigned)((N + 63) / 64), (unsigned)((Cn + 63) / 64));
    k_sgemm_xw<<<gg, 256, 0, st>>>(x, W, wx, N, I, Cn);
    h->launches += 2;
    // per step: R*h as a tiled fp32 GEMM ([B][H] x [H][3H], the kernel of the input projection),
    // then the pointwise gates
    if ((rc = ensure(h, h->f_acc2, (size_t)B * Cn * 4))) return rc;
    float *rh = (float *)h->f_acc2.p;
    dim3 grid((H + 127) / 128, (B + 1) / 2), gr((unsigned)((B + 63) / 64), (unsigned)((Cn + 63) / 64));
    for (int t = 0; t < T; ++t) {
        const float *hin = h_out + (size_t)t * NH;
        float *hout = h_out + (size_t)(t + 1) * NH;
        float *vt = v_out ? v_out + (size_t)t * B * v_stride * H : nullptr;
        k_sgemm_xw<<<gr, 256, 0, st>>>(hin, R, rh, B, H, Cn);
        if (acc_min)
            k_float_step<true><<<grid, 256, 0, st>>>(wx + (size_t)t * B * Cn, rh, bw, br, hin, hout, vt, v_stride, B, H, acc_min, acc_max);
        else
            k_float_step<false><<<grid, 256, 0, st>>>(wx + (size_t)t * B * Cn, rh, bw, br, hin, hout, vt, v_stride, B, H, nullptr, nullptr);
        h->launches += 2;
    }
    CK(cudaGetLastError());
    return QGRU_OK;
}

}  // namespace qgru

extern "C" {

int qgru_forward_float(qgru_handle *h, int T, int B, const float *W, const float *R, const float *bw,
                       const float *br, const float *x, const float *h0, float *h_out, float *v_out,
                       void *stream) {
    if (!h || !W || !R || !bw || !br || !x || !h_out) return QGRU_ERR_BAD_ARG;
    if (T <= 0 || B <= 0) return fail(h, QGRU_ERR_BAD_ARG, "T and B must be positive");
    CK(cudaSetDevice(h->device));
    return float_forward(h, T, B, W, R, bw, br, x, h0, h_out, v_out, 4, nullptr, nullptr, (cudaStream_t)stream);
}

int qgru_calibrate_minmax(qgru_handle *h, int T, int B, const float *W, const float *R,
                          const float *bw, const float *br, const float *x, const float *h0,
                          qgru_ranges *ranges, float *h_out, void *stream) {
    if (!h || !W || !R || !bw || !br || !x || !ranges) return QGRU_ERR_BAD_ARG;
    if (T <= 0 || B <= 0) return fail(h, QGRU_ERR_BAD_ARG, "T and B must be positive");
    if (ranges->hidden != h->H) return fail(h, QGRU_ERR_BAD_ARG, "ranges.hidden != handle hidden_size");
    if (!ranges->min_W || !ranges->max_W || !ranges->min_R || !ranges->max_R || !ranges->min_bw ||
        !ranges->max_bw || !ranges->min_br || !ranges->max_br)
        return fail(h, QGRU_ERR_BAD_ARG, "ranges: per-channel arrays missing");
    CK(cudaSetDevice(h->device));
    cudaStream_t st = (cudaStream_t)stream;
    const int H = h->H, Cn = h->C;
    const size_t nh = (size_t)(T + 1) * B * H;
    int rc;
    float *hbuf = h_out;
    if (!hbuf) {
        if ((rc = ensure(h, h->f_h, nh * 4))) return rc;
        hbuf = (float *)h->f_h.p;
    }
    // accumulators: [0,17) scalar min keys, [17,34) scalar max keys, then 4 x (min[3H], max[3H])
    const int n_acc = 2 * QGRU_NUM_OPS + 8 * Cn;
    if ((rc = ensure(h, h->f_acc, (size_t)n_acc * 4))) return rc;
    unsigned *acc = (unsigned *)h->f_acc.p;
    unsigned *acc_min = acc, *acc_max = acc + QGRU_NUM_OPS, *ch = acc + 2 * QGRU_NUM_OPS;
    k_fill_u32<<<1, 32, 0, st>>>(acc_min, QGRU_NUM_OPS, KEY_EMPTY_MIN);
    k_fill_u32<<<1, 32, 0, st>>>(acc_max, QGRU_NUM_OPS, KEY_EMPTY_MAX);
    const long long nx = (long long)T * B * h->I;
    k_minmax_tensor<<<grid_for(nx, 256, h->sm_count), 256, 0, st>>>(x, nx, acc_min, acc_max, QGRU_OP_X);
    const float *mats[4] = {W, R, bw, br};
    const int rows[4] = {h->I, H, 1, 1};
    for (int k = 0; k < 4; ++k)
        k_minmax_channels<<<(Cn + 127) / 128, 128, 0, st>>>(mats[k], rows[k], Cn, ch + (2 * k) * Cn, ch + (2 * k + 1) * Cn);
    h->launches += 7;
    if ((rc = float_forward(h, T, B, W, R, bw, br, x, h0, hbuf, nullptr, 4, acc_min, acc_max, st))) return rc;
    std::vector<unsigned> host(n_acc);
    CK(cudaMemcpyAsync(host.data(), acc, (size_t)n_acc * 4, cudaMemcpyDeviceToHost, st));
    CK(cudaStreamSynchronize(st));
    for (int i = 0; i < QGRU_NUM_OPS; ++i) {
        if (host[i] == KEY_EMPTY_MIN && host[QGRU_NUM_OPS + i] == KEY_EMPTY_MAX) continue;
        ranges->min_v[i] = std::min(ranges->min_v[i], key2f(host[i]));
        ranges->max_v[i] = std::max(ranges->max_v[i], key2f(host[QGRU_NUM_OPS + i]));
    }
    float *mins[4] = {ranges->min_W, ranges->min_R, ranges->min_bw, ranges->min_br};
    float *maxs[4] = {ranges->max_W, ranges->max_R, ranges->max_bw, ranges->max_br};
    for (int k = 0; k < 4; ++k) {
        const unsigned *kmin = host.data() + 2 * QGRU_NUM_OPS + (2 * k) * Cn, *kmax = kmin + Cn;
        for (int c = 0; c < Cn; ++c) {
            if (kmin[c] == KEY_EMPTY_MIN && kmax[c] == KEY_EMPTY_MAX) continue;
            mins[k][c] = std::min(mins[k][c], key2f(kmin[c]));
            maxs[k][c] = std::max(maxs[k][c], key2f(kmax[c]));
        }
    }
    return QGRU_OK;
}

}  // extern "C"
