// Training mode of the integer forward with float interface: the reference's quantGRUForwardInt
// with is_training = true (src/gru_interface.cc:610-725).  Quantize x and h0 (masks kept), run the
// step-by-step integer kernels, which keep the gate buffer and the five computation masks, and
// dequantize h and v.  The weight masks come from the float master weights.
//
// Included at the end of qgru_api.cu, after qgru_fstorage.cuh.
#pragma once
#include "qgru_fstorage.cuh"

namespace qgru {

// quantize<true> (include/quantize_ops_helper.h:528-533): keep = 1 where rint(x / scale) + zp lies
// inside the operator's range.
__global__ void k_quantize_keep(const float *__restrict__ x, long long n, float scale, int32_t zp, int32_t lo,
                                int32_t hi, uint8_t *__restrict__ keep) {
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n;
         i += (long long)gridDim.x * blockDim.x) {
        const int32_t q = (int32_t)(rintf(__fdiv_rn(x[i], scale)) + (float)zp);
        keep[i] = (q < lo || q > hi) ? 0 : 1;
    }
}

// dequantificationV (src/quantize_ops.cu:439-470): the four slots of v with their own scales.
__global__ void k_dequantize_v(const int32_t *__restrict__ vq, float *__restrict__ v, long long rows, int H,
                               FsTrainConsts tc) {
    const long long total = rows * 4 * H;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const int slot = (int)((i / H) & 3);
        v[i] = (float)(vq[i] - (int32_t)tc.zp[slot]) * tc.scale[slot];
    }
}

}  // namespace qgru

extern "C" {

int qgru_forward_f32_train(qgru_handle *h, int T, int B, const float *W, const float *R, const float *bw,
                           const float *br, const float *x, const float *h0, float *h_out, float *v_out,
                           int32_t *x_q_out, const qgru_train_masks *masks, unsigned flags, void *stream) {
    if (!h || !x || !h_out || !v_out) return QGRU_ERR_BAD_ARG;
    int rc = check_forward_args(h, T, B);
    if (rc) return rc;
    CK(cudaSetDevice(h->device));
    cudaStream_t st = (cudaStream_t)stream;
    const qgru_params &p = h->p;
    const int H = h->H, I = h->I, C = h->C;
    const long long N = (long long)T * B;
    const qgru_op &xo = p.op[QGRU_OP_X], &ho = p.op[QGRU_OP_H];
    const qgru_train_masks m = masks ? *masks : qgru_train_masks{};
    qgru::FsTrainConsts tc{};
    const int v_ops[4] = {QGRU_OP_UPDATE_OUT, QGRU_OP_RESET_OUT, QGRU_OP_NEW_OUT, QGRU_OP_HH_LINEAR};
    for (int k = 0; k < 4; ++k) {
        Rescale f;
        if (!to_fixed_scale(p.op[v_ops[k]].scale, p.use_pot2 != 0, &f)) return fail(h, QGRU_ERR_RANGE, "scale cannot be encoded");
        tc.scale[k] = decode_scale(f);
        tc.zp[k] = (float)p.op[v_ops[k]].zero_point;
    }
    const size_t nh = (size_t)(T + 1) * B * H, nv = (size_t)N * 4 * H;
    int32_t *x32 = x_q_out;
    if (!x32) {
        if ((rc = ensure(h, h->x32, (size_t)N * I * 4))) return rc;
        x32 = (int32_t *)h->x32.p;
    }
    if ((rc = ensure(h, h->hq32, nh * 4))) return rc;
    if ((rc = ensure(h, h->vq32, nv * 4))) return rc;
    const long long init_slot = (flags & QGRU_FLAG_REVERSE) ? T : 0;
    h->ev = h->ring[h->calls % qgru_handle::kRing];
    h->calls++;
    CK(cudaEventRecord(h->ev[0], st));
    CK(cudaMemsetAsync(h->d_flags, 0, 2 * sizeof(int), st));
    k_quantize_f32_i32<<<grid_for(N * I, 256, h->sm_count), 256, 0, st>>>(x, x32, N * I, h->x_scale, xo.zero_point,
                                                                         op_qmin(xo), op_qmax(xo));
    if (m.x)
        qgru::k_quantize_keep<<<grid_for(N * I, 256, h->sm_count), 256, 0, st>>>(x, N * I, h->x_scale, xo.zero_point,
                                                                             op_qmin(xo), op_qmax(xo), m.x);
    k_init_state<<<grid_for((long long)B * h->Hpad, 256, h->sm_count), 256, 0, st>>>(
        nullptr, h0, nullptr, (int32_t *)h->hq32.p, nullptr, nullptr, B, H, h->Hpad, init_slot, h->h_scale, ho.zero_point,
        op_qmin(ho), op_qmax(ho), h->d_flags);
    if (m.h0 && h0)
        qgru::k_quantize_keep<<<grid_for((long long)B * H, 256, h->sm_count), 256, 0, st>>>(
            h0, (long long)B * H, h->h_scale, ho.zero_point, op_qmin(ho), op_qmax(ho), m.h0);
    const float *wsrc[4] = {W, R, bw, br};
    uint8_t *wmask[4] = {m.W, m.R, m.bw, m.br};
    const long long wn[4] = {(long long)I * C, (long long)H * C, C, C};
    const int wop[4] = {QGRU_OP_W, QGRU_OP_R, QGRU_OP_BW, QGRU_OP_BR};
    for (int k = 0; k < 4; ++k)
        if (wsrc[k] && wmask[k])
            qgru::k_fs_weight_mask<<<grid_for(wn[k], 256, h->sm_count), 256, 0, st>>>(
                wsrc[k], wn[k], C, h->d_wscale[k], (float)op_qmin(p.op[wop[k]]), (float)op_qmax(p.op[wop[k]]), wmask[k]);
    h->launches += 8;
    const qgru_masks cm{m.ih_linear, m.hh_linear, m.gate_input, m.gate_output, m.h};
    if ((rc = run_generic(h, T, B, x32, (int32_t *)h->hq32.p, (int32_t *)h->vq32.p, flags, st, &cm))) return rc;
    k_dequantize<<<grid_for((long long)nh, 256, h->sm_count), 256, 0, st>>>((const int32_t *)h->hq32.p, h_out,
                                                                          (long long)nh, h->h_scale, ho.zero_point);
    qgru::k_dequantize_v<<<grid_for((long long)nv, 256, h->sm_count), 256, 0, st>>>((const int32_t *)h->vq32.p, v_out,
                                                                                N, H, tc);
    h->launches += 2;
    CK(cudaGetLastError());
    return QGRU_OK;
}

}  // extern "C"
