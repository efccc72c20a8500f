// shim_driver.cc - TEST INFRASTRUCTURE: calls the reference-signature entry points of
// quant-gru-pytorch_b200/shim/gru_interface_b200.cc (compiled here into namespace b200shim)
// with host buffers, so that a test can hold them against the reference's CPU integer path.
// The quant params travel as the PODs of include/qgru.h, are turned into a real GRUQuantParams
// (oracle/ref_pod.h), and the shim marshals them back: both directions of the field mapping
// are exercised.  Links libqgru_b200.so only; nothing of the reference but its headers.
#include <cublas_v2.h>
#include <cuda_runtime.h>

#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

#include "gru_interface.h"
#include "ref_pod.h"

namespace b200shim {
void quantGRUForwardInt32(bool, int, int, int, int, const int32_t *, const int32_t *, const int32_t *, const int32_t *,
                          const int32_t *, const int32_t *, const GRUQuantParams &, const cublasHandle_t &, int32_t *,
                          int32_t *, uint8_t *, uint8_t *, uint8_t *, uint8_t *, uint8_t *);
void quantGRUForwardInt(bool, const int, const int, const int, const int, const float *, const float *, const float *,
                        const float *, const float *, const float *, const GRUQuantParams &, const cublasHandle_t &,
                        float *, float *, uint8_t *, uint8_t *, uint8_t *, uint8_t *, uint8_t *, uint8_t *, uint8_t *,
                        uint8_t *, uint8_t *, uint8_t *, uint8_t *, int32_t *, int32_t *, int32_t *, int32_t *, int32_t *);
void quantGRUForwardIntIO(bool, const int, const int, const int, const int, const float *, const float *,
                          const float *, const float *, const int32_t *, const int32_t *, const GRUQuantParams &,
                          const cublasHandle_t &, int32_t *, int32_t *, uint8_t *, uint8_t *, uint8_t *, uint8_t *,
                          uint8_t *, uint8_t *, uint8_t *, uint8_t *, uint8_t *);
}  // namespace b200shim

namespace {

thread_local std::string g_err;

template <class T>
struct Dev {
    T *p = nullptr;
    size_t n = 0;
    Dev(const T *host, size_t count) : n(host ? count : 0) {
        if (n && (cudaMalloc(&p, n * sizeof(T)) != cudaSuccess ||
                  cudaMemcpy(p, host, n * sizeof(T), cudaMemcpyHostToDevice) != cudaSuccess))
            throw std::runtime_error("device copy-in failed");
    }
    explicit Dev(size_t count) : n(count) {
        if (n && (cudaMalloc(&p, n * sizeof(T)) != cudaSuccess || cudaMemset(p, 0, n * sizeof(T)) != cudaSuccess))
            throw std::runtime_error("device allocation failed");
    }
    Dev(const Dev &) = delete;
    ~Dev() { cudaFree(p); }
    void out(T *host) const {
        if (host && n && cudaMemcpy(host, p, n * sizeof(T), cudaMemcpyDeviceToHost) != cudaSuccess)
            throw std::runtime_error("device copy-out failed");
    }
};

template <class F>
int guarded(F &&f) {
    try {
        f();
        return 0;
    } catch (const std::invalid_argument &e) {
        g_err = std::string("invalid_argument: ") + e.what();
        return 2;
    } catch (const std::exception &e) {
        g_err = e.what();
        return 1;
    }
}

const cublasHandle_t g_no_blas = nullptr;   // the integer path never uses the handle

}  // namespace

extern "C" {

const char *shimtest_last_error() { return g_err.c_str(); }

// quantGRUForwardInt32 through the shim; training != 0 also returns v_q and the five masks
int shimtest_forward_i32(int training, int T, int B, int I, int H, const int32_t *W, const int32_t *R,
                         const int32_t *bw, const int32_t *br, const int32_t *x_q, const int32_t *h0_q,
                         const qgru_params *p, const float *sW, const float *sR, const float *sbw, const float *sbr,
                         int32_t *h_q, int32_t *v_q, uint8_t *const *masks) {
    return guarded([&] {
        const GRUQuantParams q = refpod::fromPod(*p, sW, sR, sbw, sbr);
        const size_t C3 = size_t(H) * 3, TB = size_t(T) * B;
        Dev<int32_t> dW(W, size_t(I) * C3), dR(R, size_t(H) * C3), dbw(bw, C3), dbr(br, C3), dx(x_q, TB * I),
            dh0(h0_q, size_t(B) * H), dh((TB + B) * H), dv(training ? TB * H * 4 : 0);
        const size_t msz[5] = {TB * C3, TB * C3, TB * C3, TB * C3, TB * H};
        std::vector<std::unique_ptr<Dev<uint8_t>>> dm;
        uint8_t *mp[5] = {nullptr, nullptr, nullptr, nullptr, nullptr};
        for (int k = 0; k < 5 && training; ++k) {
            dm.emplace_back(new Dev<uint8_t>(msz[k]));
            mp[k] = dm.back()->p;
        }
        b200shim::quantGRUForwardInt32(training != 0, T, B, I, H, dW.p, dR.p, dbw.p, dbr.p, dx.p, dh0.p, q, g_no_blas,
                                       dh.p, dv.p, mp[0], mp[1], mp[2], mp[3], mp[4]);
        dh.out(h_q);
        dv.out(v_q);
        for (int k = 0; k < 5 && training; ++k)
            if (masks && masks[k]) dm[k]->out(masks[k]);
    });
}

// quantGRUForwardInt (float in, float out; inference) through the shim; also the quantized
// weights and input it hands back
int shimtest_forward_f32(int T, int B, int I, int H, const float *W, const float *R, const float *bw,
                         const float *br, const float *x, const float *h0, const qgru_params *p, const float *sW,
                         const float *sR, const float *sbw, const float *sbr, float *h_out, int32_t *W_q,
                         int32_t *R_q, int32_t *bw_q, int32_t *br_q, int32_t *x_q) {
    return guarded([&] {
        const GRUQuantParams q = refpod::fromPod(*p, sW, sR, sbw, sbr);
        const size_t C3 = size_t(H) * 3, TB = size_t(T) * B;
        Dev<float> dW(W, size_t(I) * C3), dR(R, size_t(H) * C3), dbw(bw, C3), dbr(br, C3), dx(x, TB * I),
            dh0(h0, size_t(B) * H), dh((TB + B) * H);
        Dev<int32_t> qW(size_t(I) * C3), qR(size_t(H) * C3), qbw(C3), qbr(C3), qx(TB * I);
        b200shim::quantGRUForwardInt(false, T, B, I, H, dW.p, dR.p, dbw.p, dbr.p, dx.p, dh0.p, q, g_no_blas, dh.p, nullptr,
                                     nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr,
                                     nullptr, nullptr, qW.p, qR.p, qbw.p, qbr.p, qx.p);
        dh.out(h_out);
        qW.out(W_q);
        qR.out(R_q);
        qbw.out(bw_q);
        qbr.out(br_q);
        qx.out(x_q);
    });
}

// quantGRUForwardIntIO (float weights, int32 x in, int32 h out; inference) through the shim
int shimtest_forward_intio(int T, int B, int I, int H, const float *W, const float *R, const float *bw,
                           const float *br, const int32_t *x_q, const int32_t *h0_q, const qgru_params *p,
                           const float *sW, const float *sR, const float *sbw, const float *sbr, int32_t *h_q) {
    return guarded([&] {
        const GRUQuantParams q = refpod::fromPod(*p, sW, sR, sbw, sbr);
        const size_t C3 = size_t(H) * 3, TB = size_t(T) * B;
        Dev<float> dW(W, size_t(I) * C3), dR(R, size_t(H) * C3), dbw(bw, C3), dbr(br, C3);
        Dev<int32_t> dx(x_q, TB * I), dh0(h0_q, size_t(B) * H), dh((TB + B) * H);
        b200shim::quantGRUForwardIntIO(false, T, B, I, H, dW.p, dR.p, dbw.p, dbr.p, dx.p, dh0.p, q, g_no_blas, dh.p,
                                       nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr,
                                       nullptr);
        dh.out(h_q);
    });
}

}  // extern "C"
