// qgru_handle.h - the handle behind the opaque qgru_handle of include/qgru.h and the small
// host utilities every translation unit of the library shares.
#pragma once
#include <cuda_runtime.h>

#include <algorithm>
#include <string>
#include <vector>

#include "qgru_gemm_tc.cuh"
#include "qgru_rec_mma.cuh"
#include "qgru_internal.h"

using qgru::GateConsts;
using qgru::Rescale;
using qgru::TcGemmState;

struct DevBuf {
    void *p = nullptr;
    size_t cap = 0;
};

struct qgru_handle {
    int device = 0, I = 0, H = 0, C = 0, Ipad = 0, Hpad = 0;
    int sm_count = 0, smem_optin = 0, coop = 0;
    std::string err;
    std::string plan_text;
    bool params_set = false, weights_set = false;
    qgru_params p{};
    std::vector<float> sc[4];  // W, R, bw, br scales
    // storage plan
    bool fast = false;         // 8-bit operands, int32 accumulation
    bool x_uns = false, h_uns = false;
    int ih_bytes = 1;
    float x_scale = 1.f, h_scale = 1.f;
    GateConsts gc_host{};
    // options
    int opt_gemm = 0;      // 0 auto, 1 simt, 2 tcgen05
    int opt_rec = 0;       // 0 auto, 1 dp4a, 3 generic
    int opt_sm_limit = 0;  // 0: all SMs
    int opt_exchange = 0;  // 0 auto (cluster where it fits), 1 global counter, 2 cluster only
    int opt_cell = 0;      // 0 auto (fused cell where valid), 1 generic cell
    int opt_mt = 0;                          // cluster recurrence: 2 = two 128-unit tiles per CTA where 128 < H <= 256
    int opt_r_where = 0;                     // cluster recurrence: 0 auto, 1 R in shared memory, 2 in tensor memory
    unsigned spin_limit = 1u << 24;
    int opt_ng = 0;                          // cluster recurrence: sub-groups per CTA (0 auto, 1, 2)
    int opt_kp = 1;                          // cluster recurrence: K halves with issuers of their own (1, 2)
    int opt_issue_delay = 0;                 // cluster recurrence: head start of a gate's MMAs over the next gate's, cycles
    int opt_tie = 0;                         // 0: drop the tie rule where it provably cannot matter, 1: always apply it
    int opt_ut = 0;                          // cluster recurrence: hidden units per CTA (0 auto, 64, 128)
#ifdef QGRU_STAMPS
    long long *dbg_stamps = nullptr;
#endif
    bool opt_withhold = false;               // failure-path test of the dp4a recurrence's bounded group barrier
    int opt_gemv_r = 0;                      // one-CTA-per-row recurrence: 0 auto (R in registers where the form exists), 1 R in shared memory
    int opt_tchunk = -1;                     // cluster recurrence: timesteps per GEMM / recurrence chunk (0 whole sequence, -1 auto)
    cudaStream_t aux = nullptr;              // chunked forward: the stream the next chunk's W*x GEMM runs on
    cudaEvent_t ev_g[2] = {}, ev_r[2] = {}, ev_fork = nullptr;   // chunked forward: GEMM / recurrence of a buffer done
    bool opt_floor = false;                  // cluster recurrence: run the synchronisation-floor probe instead
    // device state that lives with the handle
    GateConsts *d_gc = nullptr;
    int32_t *d_tables = nullptr;
    int n_table = 0;
    int32_t *d_ftables = nullptr;  // tables of the fused cell
    int n_ftable = 0;
    Rescale *d_rs[2] = {nullptr, nullptr};    // gemm rescale: x side, h side
    Rescale *d_brs[2] = {nullptr, nullptr};   // bias rescale
    qgru::FastLin *d_fl[2] = {nullptr, nullptr};  // rs + corr folded (filled with the weights)
    float *d_wscale[4] = {nullptr, nullptr, nullptr, nullptr};
    int64_t *d_corr[2] = {nullptr, nullptr};
    int32_t *d_wq[4] = {nullptr, nullptr, nullptr, nullptr};  // W_q, R_q, bw_q, br_q
    int32_t *d_wsum[2] = {nullptr, nullptr};
    int8_t *d_w8[2] = {nullptr, nullptr};     // W8 [3H][Ipad], R8 [3H][Hpad] (rows over-allocated)
    long long w8_rows[2] = {0, 0};
    bool lin_fits32[2] = {false, false};      // acc + corr fits int32 (x side, h side)
    bool lin_notie[2] = {false, false};       // no channel of that layer's requantization can meet an exact tie
    bool rs_fast[2] = {false, false};   // every per-channel GEMM rescale has the shift-free form
    int *d_flags = nullptr;                   // [0] data errors, [1] barrier abort
    int *h_flags = nullptr;                   // pinned mirror
    unsigned *d_bar = nullptr;
    int bar_groups = 0;
    // workspace
    DevBuf x8, ih, h8, x32, ih32, hh32, hq32, stage_in, stage_h0, stage_out;
    DevBuf f_wx, f_h, f_v, f_acc, f_acc2;  // float mode / calibration (f_acc2: R*h of one step)
    DevBuf vq32;                           // integer training forward: gate buffer before dequantization
    DevBuf bwd_dp, bwd_dq;                 // backward pass: gradients of W*x + bw and R*h + br, [T*B][3H] each
    DevBuf fs_ch;                          // float-storage forward: 4 x 3H per-channel scale ratios
    bool fs_ready = false;                 // fs_ch matches the current parameters
    static constexpr int kRing = 64;
    cudaEvent_t ring[kRing][4] = {};   // per forward: start, gemm start, gemm end, recurrence end
    cudaEvent_t *ev = ring[0];          // the slot the current forward records into
    uint64_t calls = 0;                 // forwards issued
    bool timing_valid = false;
    uint64_t launches = 0;
    TcGemmState tc;
    qgru::RecMmaState rec;       // tensor maps of the global-exchange recurrence
    qgru::RecMmaState rec_cl;    // tensor maps of the cluster-exchange recurrence
    qgru::RecMmaState rec_c64;   // tensor maps of its 64-units-per-CTA form
};

#define CK(call)                                                                          \
    do {                                                                                  \
        cudaError_t e_ = (call);                                                          \
        if (e_ != cudaSuccess) {                                                          \
            h->err = std::string(#call) + ": " + cudaGetErrorString(e_);                  \
            return QGRU_ERR_CUDA;                                                         \
        }                                                                                 \
    } while (0)

inline int fail(qgru_handle *h, int code, const std::string &msg) {
    h->err = msg;
    return code;
}

inline int ensure(qgru_handle *h, DevBuf &b, size_t bytes) {
    if (bytes <= b.cap) return QGRU_OK;
    if (b.p) cudaFree(b.p);
    b.p = nullptr;
    b.cap = 0;
    const size_t want = bytes + bytes / 8 + 256;
    cudaError_t e = cudaMalloc(&b.p, want);
    if (e != cudaSuccess) {
        h->err = std::string("cudaMalloc(workspace): ") + cudaGetErrorString(e);
        cudaGetLastError();
        return QGRU_ERR_NOMEM;
    }
    b.cap = want;
    return QGRU_OK;
}

template <class T>
inline int alloc_dev(qgru_handle *h, T **p, size_t n) {
    if (*p) {
        cudaFree(*p);
        *p = nullptr;
    }
    cudaError_t e = cudaMalloc(reinterpret_cast<void **>(p), std::max<size_t>(n, 1) * sizeof(T));
    if (e != cudaSuccess) {
        h->err = std::string("cudaMalloc: ") + cudaGetErrorString(e);
        cudaGetLastError();
        return QGRU_ERR_NOMEM;
    }
    return QGRU_OK;
}

inline int grid_for(long long n, int block, int sm_count) {
    long long g = (n + block - 1) / block;
    const long long cap = (long long)sm_count * 16;
    return (int)std::max<long long>(1, std::min(g, cap));
}

