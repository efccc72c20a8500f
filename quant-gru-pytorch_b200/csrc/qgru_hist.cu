// qgru_hist.cu - histogram calibration: 2048-bin histograms with range growth of every operator
// of the float GRU, collected on the GPU, and the Percentile / SQNR parameter derivation.
//
// Follows the reference's GPU collector (GPUHistogramCollector::collect,
// src/calibration_gpu.cu:820-876; build_histogram :499-522; redistribute_histogram :524-540;
// kernels :66-158) and its driver collectAllHistogramsGPU
// (src/histogram_calibration_utils.cu:18-123): per tensor and per batch a min/max pass over the
// finite values, the host range rules (first batch fixes the range limit, later batches grow
// the range inside it), a proportional redistribution of the old counts when the range
// changes, and the binning pass.  Differences in how the work is done, not in what is counted:
// the gate tensors are not materialised (a generator computes each value from the float
// forward's buffers inside both passes), one privatised binning kernel serves every tensor, and
// the per-channel weight histograms are built by one block per channel.
//
// Float expressions that decide a bin keep the reference kernels' operand order, with explicit
// round-to-nearest multiplies and adds so that no fused multiply-add changes a boundary case.
#include <cuda_runtime.h>

#include <algorithm>
#include <cfloat>
#include <cmath>
#include <cstring>
#include <string>
#include <thread>
#include <vector>

#include "qgru_handle.h"

using namespace qgru;

namespace qgru {
int float_forward(qgru_handle *h, int T, int B, const float *W, const float *R, const float *bw,
                  const float *br, const float *x, const float *h0, float *h_out, float *v_out,
                  int v_stride, unsigned *acc_min, unsigned *acc_max, cudaStream_t st);
int calibrate_histogram_op(const float *counts, int bins, float min_val, float max_val, long long total,
                           bool pot2, bool use_percentile, float percentile, qgru_op *op);
}  // namespace qgru

// One collector: counts live on the device, range and bookkeeping on the host.
struct HistMeta {
    float min_val = FLT_MAX, max_val = -FLT_MAX;
    long long total = 0;
    bool valid = false;
    bool limit_set = false;
    float limit_min = 0.f, limit_max = 0.f;
};

struct qgru_hist {
    int device = 0, H = 0, bins = 0, n = 0;
    float *d_counts = nullptr;     // [n][bins]
    float *d_tmp = nullptr;        // [bins] redistribution target
    float *d_mm = nullptr;         // [2] min / max of one pass, then per-channel [2 * 3H]
    std::vector<HistMeta> meta;
    bool channels_done[4] = {false, false, false, false};
    std::string err;
};

namespace {

// ---- value generators: element i of a logical tensor, computed from the float forward's buffers
enum GenKind : int {
    GEN_PLAIN = 0,     // p0[i]
    GEN_WX_BIAS,       // p0[i] + p1[i % C]                         (W*x + bw, C = 3H)
    GEN_V3,            // v slots 3..5 as one [N][3H] tensor        (R*h + br)
    GEN_V_SLOT,        // v slot `slot` as an [N][H] tensor          (z, r, n)
    GEN_PRE_ZR,        // (wx[g] + bw[g]) + v[3 + g]                (update / reset gate input, g = slot)
    GEN_PRE_N,         // (wx[2] + bw[2]) + v[1] * v[5]             (new gate input)
    GEN_RH,            // v[1] * v[5]                               (r * (R*h + br)_n)
    GEN_NEW,           // (1 - v[0]) * v[2]
    GEN_OLD,           // v[0] * h[t]                               (h = p1: [(T+1)][B][H], row n of slot t)
    GEN_COLS,          // p0[k * ld + c0 + j], j < width             (a column block of a [K][ld] matrix)
};

struct Gen {
    int kind, slot;
    const float *p0, *p1, *v, *wx;
    int H, ld, c0, width;
    long long n;   // number of elements
};

__device__ __forceinline__ float gen_value(const Gen &g, long long i) {
    const int H = g.H;
    switch (g.kind) {
        case GEN_PLAIN: return g.p0[i];
        case GEN_WX_BIAS: return g.p0[i] + g.p1[i % (3 * H)];
        case GEN_V3: {
            const long long row = i / (3 * H);
            const int c = (int)(i % (3 * H));
            return g.v[row * 6 * H + 3 * H + c];
        }
        case GEN_V_SLOT: {
            const long long row = i / H;
            const int j = (int)(i % H);
            return g.v[row * 6 * H + (long long)g.slot * H + j];
        }
        case GEN_PRE_ZR: {
            const long long row = i / H;
            const int j = (int)(i % H);
            const float w = g.wx[row * 3 * H + (long long)g.slot * H + j] + g.p1[g.slot * H + j];
            return w + g.v[row * 6 * H + (long long)(3 + g.slot) * H + j];
        }
        case GEN_PRE_N: {
            const long long row = i / H;
            const int j = (int)(i % H);
            const float w = g.wx[row * 3 * H + 2LL * H + j] + g.p1[2 * H + j];
            return w + __fmul_rn(g.v[row * 6 * H + H + j], g.v[row * 6 * H + 5LL * H + j]);
        }
        case GEN_RH: {
            const long long row = i / H;
            const int j = (int)(i % H);
            return __fmul_rn(g.v[row * 6 * H + H + j], g.v[row * 6 * H + 5LL * H + j]);
        }
        case GEN_NEW: {
            const long long row = i / H;
            const int j = (int)(i % H);
            return __fmul_rn(1.0f - g.v[row * 6 * H + j], g.v[row * 6 * H + 2LL * H + j]);
        }
        case GEN_OLD: {
            const long long row = i / H;
            const int j = (int)(i % H);
            return __fmul_rn(g.v[row * 6 * H + j], g.p1[row * H + j]);
        }
        default: {   // GEN_COLS
            const long long k = i / g.width;
            const int j = (int)(i % g.width);
            return g.p0[k * g.ld + g.c0 + j];
        }
    }
}

// ordered-integer keys so that float min/max can use integer atomics
__device__ __forceinline__ unsigned fkey(float f) {
    const unsigned u = __float_as_uint(f);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
inline float key_to_float(unsigned k) {
    const unsigned u = (k & 0x80000000u) ? (k & 0x7fffffffu) : ~k;
    float f;
    std::memcpy(&f, &u, 4);
    return f;
}
constexpr unsigned KEY_MIN_EMPTY = 0xffffffffu, KEY_MAX_EMPTY = 0u;

// min / max of the finite values (compute_minmax of the reference filters inf and NaN)
__global__ void __launch_bounds__(256) k_hist_minmax(Gen g, unsigned *mm) {
    float mn = FLT_MAX, mx = -FLT_MAX;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < g.n;
         i += (long long)gridDim.x * blockDim.x) {
        const float v = gen_value(g, i);
        if (isfinite(v)) {
            mn = fminf(mn, v);
            mx = fmaxf(mx, v);
        }
    }
    for (int o = 16; o > 0; o >>= 1) {
        mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    }
    if ((threadIdx.x & 31) == 0 && mn <= mx) {
        atomicMin(mm, fkey(mn));
        atomicMax(mm + 1, fkey(mx));
    }
}

// histogram_kernel_shared (src/calibration_gpu.cu:66-104): values below / above the range go to
// the first / last bin, non-finite values are skipped; counts are whole numbers held as float.
__global__ void __launch_bounds__(256) k_hist_add(Gen g, float *counts, float min_val, float max_val,
                                                  float inv_bw, int bins) {
    extern __shared__ float sh[];
    for (int i = threadIdx.x; i < bins; i += blockDim.x) sh[i] = 0.0f;
    __syncthreads();
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < g.n;
         i += (long long)gridDim.x * blockDim.x) {
        const float v = gen_value(g, i);
        if (!isfinite(v)) continue;
        int b;
        if (v < min_val) b = 0;
        else if (v > max_val) b = bins - 1;
        else b = min((int)__fmul_rn(v - min_val, inv_bw), bins - 1);
        atomicAdd(&sh[b], 1.0f);
    }
    __syncthreads();
    for (int i = threadIdx.x; i < bins; i += blockDim.x)
        if (sh[i] > 0) atomicAdd(&counts[i], sh[i]);
}

// redistribute_histogram_kernel (src/calibration_gpu.cu:116-158): each source bin goes to the
// destination bin holding its left edge; the share beyond that bin's right edge goes to the
// bin one destination width further.
__global__ void k_hist_redistribute(const float *__restrict__ src, float src_min, float src_bw,
                                    float *__restrict__ dst, float dst_min, float dst_bw, int bins) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= bins) return;
    const float count = src[i];
    if (count <= 0) return;
    const float inv = 1.0f / dst_bw;
    const float start = __fmaf_rn((float)i, src_bw, src_min);   // fused, as the reference's kernel compiles
    int d = (int)__fmul_rn(start - dst_min, inv);
    d = min(d, bins - 1);
    const float end = __fmaf_rn(dst_bw, (float)(d + 1), dst_min);
    const float split = rintf(__fmul_rn((end - start) / src_bw, count));
    const float first = fminf(split, count);
    atomicAdd(&dst[d], first);
    const float rest = count - first;
    if (rest > 0) {
        int o = (int)__fmul_rn(__fadd_rn(start, dst_bw) - dst_min, inv);
        o = min(o, bins - 1);
        atomicAdd(&dst[o], rest);
    }
}

// per-channel min / max of a [K][C] matrix (compute_per_channel_minmax_kernel, :232-275)
__global__ void k_channel_minmax(const float *__restrict__ w, int K, int C, float *mins, float *maxs) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= C) return;
    float mn = FLT_MAX, mx = -FLT_MAX;
    for (int k = 0; k < K; ++k) {
        const float v = w[(size_t)k * C + c];
        if (isfinite(v)) {
            mn = fminf(mn, v);
            mx = fmaxf(mx, v);
        }
    }
    mins[c] = mn;
    maxs[c] = mx;
}

// build_per_channel_histogram_kernel (:389-440): one block per channel, ranges prepared on the host
__global__ void __launch_bounds__(128) k_channel_hist(const float *__restrict__ w, int K, int C,
                                                      const float *__restrict__ mins,
                                                      const float *__restrict__ maxs, float *counts, int bins) {
    extern __shared__ float sh[];
    const int c = blockIdx.x;
    for (int i = threadIdx.x; i < bins; i += blockDim.x) sh[i] = 0.0f;
    __syncthreads();
    const float mn = mins[c], mx = maxs[c];
    float bw = (mx - mn) / bins;
    if (bw < 1e-9f) bw = 1e-9f;
    const float inv = 1.0f / bw;
    for (int k = threadIdx.x; k < K; k += blockDim.x) {
        const float v = w[(size_t)k * C + c];
        if (!isfinite(v)) continue;
        int b;
        if (v < mn) b = 0;
        else if (v > mx) b = bins - 1;
        else b = min((int)__fmul_rn(v - mn, inv), bins - 1);
        atomicAdd(&sh[b], 1.0f);
    }
    __syncthreads();
    float *out = counts + (size_t)c * bins;
    for (int i = threadIdx.x; i < bins; i += blockDim.x) out[i] = sh[i];
}

int hfail(qgru_hist *hs, int code, const std::string &msg) {
    hs->err = msg;
    return code;
}
#define HCK(call)                                                                       \
    do {                                                                                \
        cudaError_t e_ = (call);                                                        \
        if (e_ != cudaSuccess) {                                                        \
            cudaGetLastError();                                                         \
            return hfail(hs, QGRU_ERR_CUDA, std::string(#call) + ": " + cudaGetErrorString(e_)); \
        }                                                                               \
    } while (0)

float min_scale_bins(int bins) { return std::min(1.19209290e-07f, 0.01f / static_cast<float>(bins)); }

int blocks_for(long long n) { return (int)std::max<long long>(1, std::min<long long>((n + 255) / 256, 1184)); }

void add_data(qgru_hist *hs, const Gen &g, float *counts, float min_val, float max_val, cudaStream_t st) {
    float bw = (max_val - min_val) / hs->bins;                  // build_histogram, :503-505
    if (bw < 1e-9f) bw = 1e-9f;
    const float inv = 1.0f / bw;
    k_hist_add<<<blocks_for(g.n), 256, (size_t)hs->bins * 4, st>>>(g, counts, min_val, max_val, inv, hs->bins);
}

// GPUHistogramCollector::collect for collector `idx` with the values `g` generates.
int collect(qgru_hist *hs, int idx, const Gen &g, cudaStream_t st) {
    if (g.n <= 0) return QGRU_OK;
    HistMeta &m = hs->meta[idx];
    float *counts = hs->d_counts + (size_t)idx * hs->bins;
    unsigned keys[2] = {KEY_MIN_EMPTY, KEY_MAX_EMPTY};
    HCK(cudaMemcpyAsync(hs->d_mm, keys, 8, cudaMemcpyHostToDevice, st));
    k_hist_minmax<<<blocks_for(g.n), 256, 0, st>>>(g, reinterpret_cast<unsigned *>(hs->d_mm));
    HCK(cudaMemcpyAsync(keys, hs->d_mm, 8, cudaMemcpyDeviceToHost, st));
    HCK(cudaStreamSynchronize(st));
    float dmin, dmax;
    if (keys[0] == KEY_MIN_EMPTY && keys[1] == KEY_MAX_EMPTY) {
        dmin = dmax = 0.0f;                                     // nothing finite
    } else {
        dmin = key_to_float(keys[0]);
        dmax = key_to_float(keys[1]);
    }
    if (dmin == dmax) {                                         // :829-832
        dmin -= 0.5f;
        dmax += 0.5f;
    }
    const float tiny_range = min_scale_bins(hs->bins) * hs->bins;
    float range = dmax - dmin;
    if (range < tiny_range || std::isnan(range) || std::isinf(range)) {   // :839-844
        dmin = std::min(dmin, 0.0f);
        dmax = std::max(dmax, 0.0f);
        range = tiny_range;
        dmax = dmin + tiny_range;
    }
    if (!m.valid) {
        HCK(cudaMemsetAsync(counts, 0, (size_t)hs->bins * 4, st));
        m.min_val = dmin;
        m.max_val = dmax;
        add_data(hs, g, counts, dmin, dmax, st);
        m.total = g.n;
        m.valid = true;
        // growth limit is infinite (HistogramCollector::Config), as in the reference's default
        m.limit_min = dmin - range * INFINITY / 2.0f;
        m.limit_max = dmax + range * INFINITY / 2.0f;
        m.limit_set = true;
    } else {
        float new_min, new_max;
        if (m.limit_set) {
            new_min = std::max(m.limit_min, std::min(dmin, m.min_val));
            new_max = std::min(m.limit_max, std::max(dmax, m.max_val));
        } else {
            new_min = std::min(dmin, m.min_val);
            new_max = std::max(dmax, m.max_val);
        }
        if (new_min == m.min_val && new_max == m.max_val) {
            add_data(hs, g, counts, m.min_val, m.max_val, st);
        } else {
            // _merge_with_extended_range_gpu, :924-955
            HCK(cudaMemsetAsync(hs->d_tmp, 0, (size_t)hs->bins * 4, st));
            const float src_bw = (hs->bins <= 0 || m.max_val <= m.min_val) ? 1.0f : (m.max_val - m.min_val) / hs->bins;
            if (std::fabs(src_bw) >= min_scale_bins(hs->bins) && !std::isnan(src_bw) && !std::isinf(src_bw)) {
                const float s_bw = (m.max_val - m.min_val) / hs->bins;      // redistribute_histogram, :528-530
                float d_bw = (new_max - new_min) / hs->bins;
                if (d_bw < 1e-9f) d_bw = 1e-9f;
                k_hist_redistribute<<<(hs->bins + 255) / 256, 256, 0, st>>>(counts, m.min_val, s_bw, hs->d_tmp,
                                                                            new_min, d_bw, hs->bins);
            }
            add_data(hs, g, hs->d_tmp, new_min, new_max, st);
            HCK(cudaMemcpyAsync(counts, hs->d_tmp, (size_t)hs->bins * 4, cudaMemcpyDeviceToDevice, st));
            m.min_val = new_min;
            m.max_val = new_max;
        }
        m.total += g.n;
    }
    HCK(cudaGetLastError());
    return QGRU_OK;
}

Gen plain(const float *p, long long n) {
    Gen g{};
    g.kind = GEN_PLAIN;
    g.p0 = p;
    g.n = n;
    return g;
}

// collect_per_channel_histograms_batch (src/calibration_gpu.cu:581-676): built once.
int collect_channels(qgru_hist *hs, int k, const float *w, int K, cudaStream_t st) {
    const int C = 3 * hs->H, bins = hs->bins;
    float *d_min = hs->d_mm + 2, *d_max = d_min + C;
    k_channel_minmax<<<(C + 127) / 128, 128, 0, st>>>(w, K, C, d_min, d_max);
    std::vector<float> mn(C), mx(C);
    HCK(cudaMemcpyAsync(mn.data(), d_min, (size_t)C * 4, cudaMemcpyDeviceToHost, st));
    HCK(cudaMemcpyAsync(mx.data(), d_max, (size_t)C * 4, cudaMemcpyDeviceToHost, st));
    HCK(cudaStreamSynchronize(st));
    const float tiny_range = min_scale_bins(bins) * bins;
    for (int c = 0; c < C; ++c) {
        if (mn[c] > mx[c]) mn[c] = mx[c] = 0.0f;
        if (mn[c] == mx[c]) {
            mn[c] -= 0.5f;
            mx[c] += 0.5f;
        }
        const float range = mx[c] - mn[c];
        if (range < tiny_range || std::isnan(range) || std::isinf(range)) {
            mn[c] = std::min(mn[c], 0.0f);
            mx[c] = std::max(mx[c], 0.0f);
            mx[c] = mn[c] + tiny_range;
        }
    }
    HCK(cudaMemcpyAsync(d_min, mn.data(), (size_t)C * 4, cudaMemcpyHostToDevice, st));
    HCK(cudaMemcpyAsync(d_max, mx.data(), (size_t)C * 4, cudaMemcpyHostToDevice, st));
    const int base = QGRU_HIST_CHANNEL0 + k * C;
    k_channel_hist<<<C, 128, (size_t)bins * 4, st>>>(w, K, C, d_min, d_max, hs->d_counts + (size_t)base * bins, bins);
    HCK(cudaStreamSynchronize(st));
    for (int c = 0; c < C; ++c) {
        HistMeta &m = hs->meta[base + c];
        m.min_val = mn[c];
        m.max_val = mx[c];
        m.total = K;
        m.valid = true;
    }
    hs->channels_done[k] = true;
    return QGRU_OK;
}

}  // namespace

extern "C" {

int qgru_hist_create(qgru_hist **out, int device, int hidden_size, int num_bins) {
    if (!out || hidden_size <= 0 || num_bins <= 0 || num_bins > 2048) return QGRU_ERR_BAD_ARG;
    *out = nullptr;
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || device < 0 || device >= count) {
        cudaGetLastError();
        return QGRU_ERR_CUDA;
    }
    qgru_hist *hs = new qgru_hist();
    hs->device = device;
    hs->H = hidden_size;
    hs->bins = num_bins;
    hs->n = QGRU_HIST_CHANNEL0 + 4 * 3 * hidden_size;
    hs->meta.resize(hs->n);
    bool ok = cudaSetDevice(device) == cudaSuccess;
    ok = ok && cudaMalloc(&hs->d_counts, (size_t)hs->n * num_bins * 4) == cudaSuccess;
    ok = ok && cudaMalloc(&hs->d_tmp, (size_t)num_bins * 4) == cudaSuccess;
    ok = ok && cudaMalloc(&hs->d_mm, (size_t)(2 + 2 * 3 * hidden_size) * 4) == cudaSuccess;
    ok = ok && cudaMemset(hs->d_counts, 0, (size_t)hs->n * num_bins * 4) == cudaSuccess;
    if (!ok) {
        cudaGetLastError();
        qgru_hist_destroy(hs);
        return QGRU_ERR_NOMEM;
    }
    *out = hs;
    return QGRU_OK;
}

void qgru_hist_destroy(qgru_hist *hs) {
    if (!hs) return;
    cudaSetDevice(hs->device);
    cudaFree(hs->d_counts);
    cudaFree(hs->d_tmp);
    cudaFree(hs->d_mm);
    cudaGetLastError();
    delete hs;
}

const char *qgru_hist_last_error(const qgru_hist *hs) { return hs ? hs->err.c_str() : "null histogram set"; }

int qgru_hist_count(const qgru_hist *hs) { return hs ? hs->n : 0; }

int qgru_hist_reset(qgru_hist *hs) {
    if (!hs) return QGRU_ERR_BAD_ARG;
    HCK(cudaSetDevice(hs->device));
    HCK(cudaMemset(hs->d_counts, 0, (size_t)hs->n * hs->bins * 4));
    for (HistMeta &m : hs->meta) m = HistMeta();
    for (bool &b : hs->channels_done) b = false;
    return QGRU_OK;
}

int qgru_hist_collect(qgru_hist *hs, int index, const float *data, long long n, void *stream) {
    if (!hs || !data || index < 0 || index >= hs->n || n < 0) return QGRU_ERR_BAD_ARG;
    HCK(cudaSetDevice(hs->device));
    return collect(hs, index, plain(data, n), (cudaStream_t)stream);
}

int qgru_hist_export(const qgru_hist *hs_c, int index, float *counts, float *min_val, float *max_val,
                     int64_t *total_count) {
    qgru_hist *hs = const_cast<qgru_hist *>(hs_c);
    if (!hs || index < 0 || index >= hs->n) return QGRU_ERR_BAD_ARG;
    const HistMeta &m = hs->meta[index];
    if (min_val) *min_val = m.min_val;
    if (max_val) *max_val = m.max_val;
    if (total_count) *total_count = m.valid ? m.total : 0;
    if (counts) {
        HCK(cudaSetDevice(hs->device));
        HCK(cudaMemcpy(counts, hs->d_counts + (size_t)index * hs->bins, (size_t)hs->bins * 4, cudaMemcpyDeviceToHost));
    }
    return QGRU_OK;
}

int qgru_hist_import(qgru_hist *hs, int index, const float *counts, float min_val, float max_val,
                     int64_t total_count) {
    if (!hs || !counts || index < 0 || index >= hs->n || total_count < 0) return QGRU_ERR_BAD_ARG;
    HCK(cudaSetDevice(hs->device));
    HCK(cudaMemcpy(hs->d_counts + (size_t)index * hs->bins, counts, (size_t)hs->bins * 4, cudaMemcpyHostToDevice));
    HistMeta &m = hs->meta[index];
    m = HistMeta();
    m.min_val = min_val;
    m.max_val = max_val;
    m.total = total_count;
    m.valid = total_count > 0;
    // GPUHistogramCollector::merge into an empty collector, src/calibration_gpu.cu:961-979
    const float tiny_range = min_scale_bins(hs->bins) * hs->bins;
    float range = max_val - min_val;
    if (range < tiny_range) range = tiny_range;
    m.limit_min = min_val - range * INFINITY / 2.0f;
    m.limit_max = max_val + range * INFINITY / 2.0f;
    m.limit_set = true;
    if (index >= QGRU_HIST_CHANNEL0) hs->channels_done[(index - QGRU_HIST_CHANNEL0) / (3 * hs->H)] = true;
    return QGRU_OK;
}

int qgru_calibrate_hist(qgru_handle *h, qgru_hist *hs, int T, int B, const float *W, const float *R,
                        const float *bw, const float *br, const float *x, const float *h0,
                        const int32_t *granularity, void *stream) {
    if (!h || !hs || !W || !R || !bw || !br || !x || !granularity) return QGRU_ERR_BAD_ARG;
    if (T <= 0 || B <= 0) return fail(h, QGRU_ERR_BAD_ARG, "T and B must be positive");
    if (hs->H != h->H || hs->device != h->device)
        return fail(h, QGRU_ERR_BAD_ARG, "histogram set belongs to another hidden size or device");
    CK(cudaSetDevice(h->device));
    cudaStream_t st = (cudaStream_t)stream;
    const int H = h->H, C = h->C, I = h->I;
    const long long N = (long long)T * B, NH = N * H;
    int rc;
    if ((rc = ensure(h, h->f_h, (size_t)(T + 1) * B * H * 4))) return rc;
    if ((rc = ensure(h, h->f_v, (size_t)N * 6 * H * 4))) return rc;
    float *hbuf = (float *)h->f_h.p, *v = (float *)h->f_v.p;
    if ((rc = float_forward(h, T, B, W, R, bw, br, x, h0, hbuf, v, 6, nullptr, nullptr, st))) return rc;
    const float *wx = (const float *)h->f_wx.p;

    auto run = [&](int idx, Gen g) -> int {
        g.H = H;
        g.v = v;
        g.wx = wx;
        const int r = collect(hs, idx, g, st);
        if (r) h->err = "histogram collection: " + hs->err;
        return r;
    };
    auto make = [&](int kind, int slot, const float *p0, const float *p1, long long n) {
        Gen g{};
        g.kind = kind;
        g.slot = slot;
        g.p0 = p0;
        g.p1 = p1;
        g.n = n;
        return g;
    };
    // x, h (without the initial state), W*x + bw, R*h + br  (collectAllHistogramsGPU, :27-48)
    if ((rc = run(QGRU_OP_X, make(GEN_PLAIN, 0, x, nullptr, N * I)))) return rc;
    if ((rc = run(QGRU_OP_H, make(GEN_PLAIN, 0, hbuf + (size_t)B * H, nullptr, NH)))) return rc;
    if ((rc = run(QGRU_OP_IH_LINEAR, make(GEN_WX_BIAS, 0, wx, bw, N * C)))) return rc;
    if ((rc = run(QGRU_OP_HH_LINEAR, make(GEN_V3, 0, nullptr, nullptr, N * C)))) return rc;
    // weights and biases by granularity (:50-97): per tensor and per gate every batch, per channel once
    const float *mats[4] = {W, R, bw, br};
    const int rows[4] = {I, H, 1, 1};
    static const int tensor_idx[4] = {QGRU_OP_W, QGRU_OP_R, QGRU_OP_BW, QGRU_OP_BR};
    for (int k = 0; k < 4; ++k) {
        if (granularity[k] == QGRU_PER_TENSOR) {
            if ((rc = run(tensor_idx[k], make(GEN_PLAIN, 0, mats[k], nullptr, (long long)rows[k] * C)))) return rc;
        } else if (granularity[k] == QGRU_PER_GATE) {
            for (int g3 = 0; g3 < 3; ++g3) {
                Gen g = make(GEN_COLS, 0, mats[k], nullptr, (long long)rows[k] * H);
                g.ld = C;
                g.c0 = g3 * H;
                g.width = H;
                if ((rc = run(QGRU_HIST_GATE0 + 3 * k + g3, g))) return rc;
            }
        } else if (!hs->channels_done[k]) {
            if ((rc = collect_channels(hs, k, mats[k], rows[k], st))) {
                h->err = "histogram collection: " + hs->err;
                return rc;
            }
        }
    }
    // gate outputs and products (collect_gate_histograms, src/calibration_gpu.cu:542-574)
    if ((rc = run(QGRU_OP_UPDATE_OUT, make(GEN_V_SLOT, 0, nullptr, nullptr, NH)))) return rc;
    if ((rc = run(QGRU_OP_RESET_OUT, make(GEN_V_SLOT, 1, nullptr, nullptr, NH)))) return rc;
    if ((rc = run(QGRU_OP_NEW_OUT, make(GEN_V_SLOT, 2, nullptr, nullptr, NH)))) return rc;
    if ((rc = run(QGRU_OP_MUL_RESET_HIDDEN, make(GEN_RH, 0, nullptr, nullptr, NH)))) return rc;
    if ((rc = run(QGRU_OP_MUL_NEW_CONTRIB, make(GEN_NEW, 0, nullptr, nullptr, NH)))) return rc;
    if ((rc = run(QGRU_OP_MUL_OLD_CONTRIB, make(GEN_OLD, 0, nullptr, hbuf, NH)))) return rc;
    // gate inputs (:109-117)
    if ((rc = run(QGRU_OP_UPDATE_IN, make(GEN_PRE_ZR, 0, nullptr, bw, NH)))) return rc;
    if ((rc = run(QGRU_OP_RESET_IN, make(GEN_PRE_ZR, 1, nullptr, bw, NH)))) return rc;
    if ((rc = run(QGRU_OP_NEW_IN, make(GEN_PRE_N, 0, nullptr, bw, NH)))) return rc;
    h->launches += 2 * 13 + 8;
    return QGRU_OK;
}

int qgru_calc_params_from_hist(const qgru_hist *hs_c, int use_percentile, float percentile, qgru_params *p,
                               float *scale_W, float *scale_R, float *scale_bw, float *scale_br) {
    qgru_hist *hs = const_cast<qgru_hist *>(hs_c);
    if (!hs || !p || !scale_W || !scale_R || !scale_bw || !scale_br) return QGRU_ERR_BAD_ARG;
    // ensureSymmetricWeightBiasConfig, src/gru_interface.cc:26-32
    if (!p->op[QGRU_OP_W].symmetric || !p->op[QGRU_OP_R].symmetric || !p->op[QGRU_OP_BW].symmetric ||
        !p->op[QGRU_OP_BR].symmetric)
        return QGRU_ERR_UNSUPPORTED;
    HCK(cudaSetDevice(hs->device));
    const int H = hs->H, C = 3 * H, bins = hs->bins;
    const bool pot2 = p->use_pot2 != 0;
    p->hidden = H;
    std::vector<float> counts((size_t)hs->n * bins);
    HCK(cudaMemcpy(counts.data(), hs->d_counts, counts.size() * 4, cudaMemcpyDeviceToHost));
    auto one = [&](int idx, qgru_op *op) -> int {
        const HistMeta &m = hs->meta[idx];
        if (!m.valid) return hfail(hs, QGRU_ERR_NOT_READY, "histogram " + std::to_string(idx) + " is empty");
        return calibrate_histogram_op(counts.data() + (size_t)idx * bins, bins, m.min_val, m.max_val, m.total, pot2,
                                      use_percentile != 0, percentile, op);
    };
    // calculateGRUQuantitativeParametersFromHistograms, src/gru_interface.cc:1079-1153
    static const int scalar_ops[] = {QGRU_OP_X, QGRU_OP_H, QGRU_OP_IH_LINEAR, QGRU_OP_HH_LINEAR,
                                     QGRU_OP_UPDATE_IN, QGRU_OP_RESET_IN, QGRU_OP_NEW_IN,
                                     QGRU_OP_UPDATE_OUT, QGRU_OP_RESET_OUT, QGRU_OP_NEW_OUT,
                                     QGRU_OP_MUL_RESET_HIDDEN, QGRU_OP_MUL_NEW_CONTRIB, QGRU_OP_MUL_OLD_CONTRIB};
    int rc;
    for (int k : scalar_ops)
        if ((rc = one(k, &p->op[k]))) return rc;
    static const int tensor_idx[4] = {QGRU_OP_W, QGRU_OP_R, QGRU_OP_BW, QGRU_OP_BR};
    float *scales[4] = {scale_W, scale_R, scale_bw, scale_br};
    for (int k = 0; k < 4; ++k) {
        qgru_op *op = &p->op[tensor_idx[k]];
        if (p->granularity[k] == QGRU_PER_TENSOR) {
            qgru_op t = *op;
            if ((rc = one(tensor_idx[k], &t))) return rc;
            std::fill(scales[k], scales[k] + C, t.scale);
        } else if (p->granularity[k] == QGRU_PER_GATE) {
            for (int g = 0; g < 3; ++g) {
                qgru_op t = *op;
                if ((rc = one(QGRU_HIST_GATE0 + 3 * k + g, &t))) return rc;
                std::fill(scales[k] + g * H, scales[k] + (g + 1) * H, t.scale);
            }
        } else {
            // 3H independent searches: spread over the host threads
            const int base = QGRU_HIST_CHANNEL0 + k * C;
            const unsigned nt = std::max(1u, std::min(16u, std::thread::hardware_concurrency()));
            std::vector<int> status(nt, QGRU_OK);
            std::vector<std::thread> pool;
            for (unsigned w = 0; w < nt; ++w)
                pool.emplace_back([&, w]() {
                    for (int c = (int)w; c < C; c += (int)nt) {
                        const HistMeta &m = hs->meta[base + c];
                        qgru_op t = *op;
                        const int r = m.valid ? calibrate_histogram_op(counts.data() + (size_t)(base + c) * bins, bins,
                                                                       m.min_val, m.max_val, m.total, pot2,
                                                                       use_percentile != 0, percentile, &t)
                                              : QGRU_ERR_NOT_READY;
                        if (r) status[w] = r;
                        scales[k][c] = t.scale;
                    }
                });
            for (std::thread &t : pool) t.join();
            for (int r : status)
                if (r) return hfail(hs, r, "per-channel histogram calibration failed");
        }
        op->scale = scales[k][0];
        op->zero_point = 0;
    }
    return qgru_generate_luts(p);
}

}  // extern "C"
