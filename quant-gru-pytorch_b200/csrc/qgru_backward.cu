// qgru_backward.cu - backward pass of the GRU: hasteGRUBackward (src/gru_interface.cc:215-240,
// src/gru_backward_gpu.cu) and quantGRUBackward with the straight-through masks of QAT
// (src/gru_interface.cc:246-290, src/gru_backward_gpu_quant.cu).  One implementation: the float
// backward is the masked one with every mask absent.
//
// Per timestep, last to first: the pointwise kernel turns dh into the gradients of the two
// linear layers' outputs (dp for W*x + bw, dq for R*h + br) and the part of dh that flows
// through the update gate; dh += dq * R^T.  After the loop: dbw / dbr as column sums of dp / dq
// (the reference adds them with atomics, in arbitrary order; here the sum is a fixed-order tree,
// so results repeat), then dx = dp * W^T, dR += h^T * dq, dW += x^T * dp.
// Not a hot path: plain fp32 SIMT GEMMs (the reference calls cuBLAS SGEMM, fp32 without
// tensor-op math in this pass).
#include "qgru_handle.h"

using namespace qgru;

namespace {

// C[n][j] (+)= sum_k A(n, k) * B[k][j].  A is [N][K] row-major, or with ATrans stored as [K][N].
// B is [K][M] row-major, C [N][M].  64x64 tile, 4x4 outputs per thread.
template <bool ATrans, bool Accum>
__global__ void __launch_bounds__(256)
k_bwd_sgemm(const float *__restrict__ A, const float *__restrict__ Bm, float *__restrict__ C,
            long long N, long long K, int M) {
    __shared__ float as[16][64 + 1];
    __shared__ float bs[16][64];
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const long long n0 = (long long)blockIdx.x * 64;
    const int c0 = blockIdx.y * 64;
    float acc[4][4] = {};
    for (long long k0 = 0; k0 < K; k0 += 16) {
        for (int i = threadIdx.x; i < 64 * 16; i += 256) {
            if (ATrans) {
                const int kk = i >> 6, r = i & 63;      // consecutive threads walk n: coalesced
                as[kk][r] = (n0 + r < N && k0 + kk < K) ? A[(k0 + kk) * N + n0 + r] : 0.f;
            } else {
                const int r = i >> 4, kk = i & 15;
                as[kk][r] = (n0 + r < N && k0 + kk < K) ? A[(n0 + r) * K + k0 + kk] : 0.f;
            }
            const int kr = i >> 6, cc = i & 63;
            bs[kr][cc] = (k0 + kr < K && c0 + cc < M) ? Bm[(k0 + kr) * M + c0 + cc] : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < 16; ++kk) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = as[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = bs[kk][tx + 16 * j];
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
            if (c >= M) continue;
            if (Accum) C[n * M + c] += acc[i][j];
            else C[n * M + c] = acc[i][j];
        }
    }
}

// The pointwise part of one timestep (kernel::PointwiseOperations, src/gru_backward_gpu.cu:26-88;
// with masks kernel::PointwiseOperationsQuant, src/gru_backward_gpu_quant.cu:72-250, zoneout
// off).  h: h_{t-1} [B][H]; v: (z, r, g, R*h_g + br_g) [B][4H]; dh_new: gradient arriving at
// h_t from outside; dh: in: gradient arriving from step t+1, out: its part through the update
// gate (the R^T part is added by the GEMM that follows).  Masks: 1 keeps the gradient, 0 (the
// forward clamped there) drops it; any may be null.
__global__ void __launch_bounds__(256)
k_bwd_pointwise(int B, int H, const float *__restrict__ h, const float *__restrict__ v,
                const float *__restrict__ dh_new, float *__restrict__ dh, float *__restrict__ dp,
                float *__restrict__ dq, const uint8_t *__restrict__ m_hh, const uint8_t *__restrict__ m_gin,
                const uint8_t *__restrict__ m_gout, const uint8_t *__restrict__ m_h) {
    const int j = blockIdx.x * blockDim.x + threadIdx.x;
    const int b = blockIdx.y;
    if (j >= H || b >= B) return;
    const size_t base = (size_t)b * H + j;
    float dh_total = dh_new[base] + dh[base];
    if (m_h) dh_total *= (float)m_h[base];
    const float *vb = v + (size_t)b * 4 * H + j;
    const float z = vb[0], r = vb[H], g = vb[2 * H], q_g = vb[3 * H];
    dh[base] = z * dh_total;
    const float dg = (1.0f - z) * dh_total;
    const float dz = (h[base] - g) * dh_total;
    const float dp_g = (1.0f - g * g) * dg;            // d_tanh(g) * dg
    const float dq_g = dp_g * r;
    const float dr = dp_g * q_g;
    const float dp_r = (r * (1.0f - r)) * dr;          // d_sigmoid(r) * dr
    const float dp_z = (z * (1.0f - z)) * dz;
    float p[3] = {dp_z, dp_r, dp_g};
    float q[3] = {dp_z, dp_r, dq_g};
    const size_t idx = (size_t)b * 3 * H + j;
#pragma unroll
    for (int k = 0; k < 3; ++k) {
        const size_t at = idx + (size_t)k * H;
        if (m_gout) { const float m = (float)m_gout[at]; p[k] *= m; q[k] *= m; }
        if (m_gin) { const float m = (float)m_gin[at]; p[k] *= m; q[k] *= m; }
        if (m_hh) q[k] *= (float)m_hh[at];
        dp[at] = p[k];
        dq[at] = q[k];
    }
}

// out[c] += mask[c] * sum_n a[n][c]: the bias gradients.  One block of 256 threads per 32
// columns; rows are added in a fixed order (8 row lanes, then a tree over them).
__global__ void __launch_bounds__(256)
k_bwd_colsum(const float *__restrict__ a, long long N, int M, const uint8_t *__restrict__ mask,
             float *__restrict__ out) {
    __shared__ float part[8][32];
    const int cx = threadIdx.x & 31, ry = threadIdx.x >> 5;
    const int c = blockIdx.x * 32 + cx;
    float s = 0.f;
    if (c < M)
        for (long long n = ry; n < N; n += 8) s += a[n * M + c];
    part[ry][cx] = s;
    __syncthreads();
    if (ry == 0 && c < M) {
        float t = 0.f;
#pragma unroll
        for (int k = 0; k < 8; ++k) t += part[k][cx];
        if (mask) t *= (float)mask[c];
        out[c] += t;
    }
}

// ApplyMaskKernel (src/gru_backward_gpu_quant.cu:37-42)
__global__ void k_bwd_apply_mask(float *__restrict__ data, const uint8_t *__restrict__ mask, long long n) {
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n;
         i += (long long)gridDim.x * blockDim.x)
        data[i] *= (float)mask[i];
}

template <bool ATrans, bool Accum>
void sgemm(const float *A, const float *Bm, float *C, long long N, long long K, int M, cudaStream_t st) {
    dim3 grid((unsigned)((N + 63) / 64), (unsigned)((M + 63) / 64));
    k_bwd_sgemm<ATrans, Accum><<<grid, 256, 0, st>>>(A, Bm, C, N, K, M);
}

}  // namespace

extern "C" {

int qgru_backward(qgru_handle *h, int T, int B, const float *W_t, const float *R_t, const float *x_t,
                  const float *dh_new, const float *h_all, const float *v, float *dx, float *dW,
                  float *dR, float *dbw, float *dbr, float *dh, const qgru_bwd_masks *mk, void *stream) {
    if (!h || !W_t || !R_t || !x_t || !dh_new || !h_all || !v || !dx || !dW || !dR || !dbw || !dbr || !dh)
        return QGRU_ERR_BAD_ARG;
    if (T <= 0 || B <= 0) return fail(h, QGRU_ERR_BAD_ARG, "T and B must be positive");
    CK(cudaSetDevice(h->device));
    cudaStream_t st = (cudaStream_t)stream;
    const int H = h->H, I = h->I, C = h->C;
    const long long N = (long long)T * B;
    const size_t NH = (size_t)B * H, NH3 = (size_t)B * C;
    int rc;
    if ((rc = ensure(h, h->bwd_dp, (size_t)N * C * sizeof(float)))) return rc;
    if ((rc = ensure(h, h->bwd_dq, (size_t)N * C * sizeof(float)))) return rc;
    float *dp = (float *)h->bwd_dp.p, *dq = (float *)h->bwd_dq.p;
    const qgru_bwd_masks none{};
    const qgru_bwd_masks &m = mk ? *mk : none;

    const dim3 pw_grid((H + 255) / 256, B);
    for (int i = T - 1; i >= 0; --i) {
        k_bwd_pointwise<<<pw_grid, 256, 0, st>>>(
            B, H, h_all + (size_t)i * NH, v + (size_t)i * NH * 4, dh_new + (size_t)(i + 1) * NH, dh,
            dp + (size_t)i * NH3, dq + (size_t)i * NH3, m.hh_linear ? m.hh_linear + (size_t)i * NH3 : nullptr,
            m.gate_input ? m.gate_input + (size_t)i * NH3 : nullptr,
            m.gate_output ? m.gate_output + (size_t)i * NH3 : nullptr, m.h ? m.h + (size_t)i * NH : nullptr);
        // dh[b][k] += sum_m dq[b][m] * R_t[m][k]
        sgemm<false, true>(dq + (size_t)i * NH3, R_t, dh, B, C, H, st);
    }
    h->launches += 2ull * T;
    // bias gradients: column sums of dp / dq before the W*x + bw mask is applied to dp
    k_bwd_colsum<<<(C + 31) / 32, 256, 0, st>>>(dp, N, C, m.bw, dbw);
    k_bwd_colsum<<<(C + 31) / 32, 256, 0, st>>>(dq, N, C, m.br, dbr);
    if (m.ih_linear)
        k_bwd_apply_mask<<<grid_for(N * C, 256, h->sm_count), 256, 0, st>>>(dp, m.ih_linear, N * C);
    // dx[n][i] = sum_m dp[n][m] * W_t[m][i]
    sgemm<false, false>(dp, W_t, dx, N, C, I, st);
    if (m.x) k_bwd_apply_mask<<<grid_for(N * I, 256, h->sm_count), 256, 0, st>>>(dx, m.x, N * I);
    // dR[k][m] += sum_n h[n][k] * dq[n][m]   (h_all's first T slots: h_{t-1} of every step)
    sgemm<true, true>(h_all, dq, dR, H, N, C, st);
    if (m.R) k_bwd_apply_mask<<<grid_for((long long)H * C, 256, h->sm_count), 256, 0, st>>>(dR, m.R, (long long)H * C);
    // dW[i][m] += sum_n x_t[i][n] * dp[n][m]
    sgemm<false, true>(x_t, dp, dW, I, N, C, st);
    if (m.W) k_bwd_apply_mask<<<grid_for((long long)I * C, 256, h->sm_count), 256, 0, st>>>(dW, m.W, (long long)I * C);
    if (m.h0) k_bwd_apply_mask<<<grid_for((long long)NH, 256, h->sm_count), 256, 0, st>>>(dh, m.h0, (long long)NH);
    h->launches += 9;
    CK(cudaGetLastError());
    return QGRU_OK;
}

}  // extern "C"
