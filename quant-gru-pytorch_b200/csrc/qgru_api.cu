// qgru_api.cu - the device half of the C ABI (include/qgru.h): handle, parameter derivation,
// weight packing and the forward orchestration.  Replaces, for the integer inference path,
// gru::ForwardPassQuant (src/gru_forward_gpu_quant.cu:412-831 of the reference) and the three
// quantGRUForwardInt* drivers (src/gru_interface.cc:551-790): the per-call stream creation,
// device allocations and device-wide synchronisations of the reference become a handle with a
// growing workspace; all work is queued on the caller's stream.
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <string>
#include <vector>

#include "qgru_handle.h"
#include "qgru_kernels.cuh"
#include "qgru_rec_mma.cuh"

using namespace qgru;

namespace {

bool shift_ok(Rescale r) { return r.shift >= -62 && r.shift <= 62; }

// Largest |q - zp| an operator's clamped value can reach.
int64_t max_abs_diff(const qgru_op &o) {
    const int64_t lo = op_qmin(o), hi = op_qmax(o), zp = o.zero_point;
    return std::max(std::llabs(hi - zp), std::llabs(lo - zp));
}

bool narrow_ok(Rescale r, int64_t max_abs) {
    return r.shift >= 1 && r.shift <= 31 && max_abs * (int64_t)r.mult < (int64_t)0x7fffffff - ((int64_t)1 << 30);
}

struct RecPlan {
    int Hs = 0, Bt = 0, P = 0, G = 0;
    size_t smem = 0;
};

size_t rec_smem(const qgru_handle *h, int Hs, int Bt) {
    size_t s = (sizeof(GateConsts) + 15) & ~size_t(15);
    s += ((size_t)h->n_table * 4 + 15) & ~size_t(15);
    s += (size_t)3 * Hs * (8 + sizeof(Rescale));
    s += (size_t)3 * Hs * h->Hpad;
    s += (size_t)Bt * h->Hpad;
    return s;
}

bool plan_recurrence(const qgru_handle *h, int B, RecPlan *out) {
    const int sms = h->opt_sm_limit > 0 ? std::min(h->opt_sm_limit, h->sm_count) : h->sm_count;
    static const int cand[4] = {256, 128, 64, 32};
    for (int Hs : cand) {
        if (Hs > 32 && Hs >= 2 * ((h->H + 31) / 32 * 32)) continue;  // no slice wider than needed
        const int P = (h->H + Hs - 1) / Hs;
        if (P > sms) continue;
        const int groups_max = std::max(1, sms / P);
        const int Bt = (B + groups_max - 1) / groups_max;
        const size_t s = rec_smem(h, Hs, Bt);
        if (s > (size_t)h->smem_optin) continue;
        out->Hs = Hs;
        out->Bt = Bt;
        out->P = P;
        out->G = (B + Bt - 1) / Bt;
        out->smem = s;
        return true;
    }
    return false;
}

}  // namespace

extern "C" {

int qgru_create(qgru_handle **out, int device, int input_size, int hidden_size) {
    if (!out || input_size <= 0 || hidden_size <= 0) return QGRU_ERR_BAD_ARG;
    *out = nullptr;
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || device < 0 || device >= count) {
        cudaGetLastError();
        return QGRU_ERR_CUDA;
    }
    qgru_handle *h = new qgru_handle();
    h->device = device;
    h->I = input_size;
    h->H = hidden_size;
    h->C = 3 * hidden_size;
    h->Ipad = (input_size + 127) / 128 * 128;   // K padded to whole 128-byte swizzle rows
    h->Hpad = (hidden_size + 127) / 128 * 128;
    bool ok = cudaSetDevice(device) == cudaSuccess;
    ok = ok && cudaDeviceGetAttribute(&h->sm_count, cudaDevAttrMultiProcessorCount, device) == cudaSuccess;
    ok = ok && cudaDeviceGetAttribute(&h->smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, device) == cudaSuccess;
    ok = ok && cudaDeviceGetAttribute(&h->coop, cudaDevAttrCooperativeLaunch, device) == cudaSuccess;
    ok = ok && cudaMalloc(&h->d_flags, 2 * sizeof(int)) == cudaSuccess;
    ok = ok && cudaMemset(h->d_flags, 0, 2 * sizeof(int)) == cudaSuccess;
    ok = ok && cudaMallocHost(&h->h_flags, 2 * sizeof(int)) == cudaSuccess;
    for (int r = 0; r < qgru_handle::kRing && ok; ++r)
        for (int i = 0; i < 4 && ok; ++i) ok = cudaEventCreate(&h->ring[r][i]) == cudaSuccess;
    if (!ok) {
        cudaGetLastError();
        qgru_destroy(h);
        return QGRU_ERR_CUDA;
    }
    h->h_flags[0] = h->h_flags[1] = 0;
    *out = h;
    return QGRU_OK;
}

void qgru_destroy(qgru_handle *h) {
    if (!h) return;
    cudaSetDevice(h->device);
    cudaDeviceSynchronize();
    cudaFree(h->d_gc);
    cudaFree(h->d_tables);
    cudaFree(h->d_ftables);
    for (int i = 0; i < 2; ++i) {
        cudaFree(h->d_rs[i]);
        cudaFree(h->d_brs[i]);
        cudaFree(h->d_fl[i]);
        cudaFree(h->d_corr[i]);
        cudaFree(h->d_wsum[i]);
        cudaFree(h->d_w8[i]);
    }
    for (int i = 0; i < 4; ++i) {
        cudaFree(h->d_wscale[i]);
        cudaFree(h->d_wq[i]);
    }
    for (int r = 0; r < qgru_handle::kRing; ++r)
        for (int i = 0; i < 4; ++i)
            if (h->ring[r][i]) cudaEventDestroy(h->ring[r][i]);
    for (int i = 0; i < 2; ++i) {
        if (h->ev_g[i]) cudaEventDestroy(h->ev_g[i]);
        if (h->ev_r[i]) cudaEventDestroy(h->ev_r[i]);
    }
    if (h->ev_fork) cudaEventDestroy(h->ev_fork);
    if (h->aux) cudaStreamDestroy(h->aux);
    cudaFree(h->d_flags);
    if (h->h_flags) cudaFreeHost(h->h_flags);
    cudaFree(h->d_bar);
    for (DevBuf *b : {&h->x8, &h->ih, &h->h8, &h->x32, &h->ih32, &h->hh32, &h->hq32, &h->stage_in,
                      &h->stage_h0, &h->stage_out, &h->f_wx, &h->f_h, &h->f_v, &h->f_acc, &h->f_acc2})
        cudaFree(b->p);
    cudaGetLastError();
    delete h;
}

const char *qgru_last_error(const qgru_handle *h) { return h ? h->err.c_str() : "null handle"; }

uint64_t qgru_launch_count(const qgru_handle *h) { return h ? h->launches : 0; }

int qgru_set_option(qgru_handle *h, const char *name, const char *value) {
    if (!h || !name || !value) return QGRU_ERR_BAD_ARG;
    const std::string n(name), v(value);
    if (n == "gemm") {
        if (v == "auto") h->opt_gemm = 0;
        else if (v == "simt") h->opt_gemm = 1;
        else if (v == "tcgen05") h->opt_gemm = 2;
        else return fail(h, QGRU_ERR_BAD_ARG, "gemm: auto|simt|tcgen05");
    } else if (n == "rec") {
        if (v == "auto") h->opt_rec = 0;
        else if (v == "dp4a") h->opt_rec = 1;
        else if (v == "mma") h->opt_rec = 2;
        else if (v == "generic") h->opt_rec = 3;
        else if (v == "gemv") h->opt_rec = 4;
        else return fail(h, QGRU_ERR_BAD_ARG, "rec: auto|dp4a|mma|gemv|generic");
    } else if (n == "exchange") {
        if (v == "auto") h->opt_exchange = 0;
        else if (v == "global") h->opt_exchange = 1;
        else if (v == "cluster") h->opt_exchange = 2;
        else return fail(h, QGRU_ERR_BAD_ARG, "exchange: auto|global|cluster");
    } else if (n == "r_resident") {
        if (v == "auto") h->opt_r_where = 0;
        else if (v == "smem") h->opt_r_where = 1;
        else if (v == "tmem") h->opt_r_where = 2;
        else return fail(h, QGRU_ERR_BAD_ARG, "r_resident: auto|smem|tmem");
    } else if (n == "tiles_per_cta") {
        h->opt_mt = std::max(0, atoi(value));
    } else if (n == "gemm_order") {
        if (v == "auto") h->tc.order = 0;
        else if (v == "stream") h->tc.order = 1;
        else if (v == "w_stationary") h->tc.order = 2;
        else return fail(h, QGRU_ERR_BAD_ARG, "gemm_order: auto|stream|w_stationary");
    } else if (n == "cell") {
        if (v == "auto") h->opt_cell = 0;
        else if (v == "generic") h->opt_cell = 1;
        else if (v == "fused") h->opt_cell = 2;   // tabulated cell, but never its shift-free form
        else return fail(h, QGRU_ERR_BAD_ARG, "cell: auto|generic|fused");
    } else if (n == "subgroups") {
        if (v == "auto") h->opt_ng = 0;
        else if (v == "1") h->opt_ng = 1;
        else if (v == "2") h->opt_ng = 2;
        else return fail(h, QGRU_ERR_BAD_ARG, "subgroups: auto|1|2");
    } else if (n == "tie_rule") {
        if (v == "auto") h->opt_tie = 0;
        else if (v == "always") h->opt_tie = 1;
        else return fail(h, QGRU_ERR_BAD_ARG, "tie_rule: auto|always");
    } else if (n == "k_parts") {
        h->opt_kp = atoi(value) == 2 ? 2 : 1;
    } else if (n == "issue_delay") {
        h->opt_issue_delay = std::max(0, atoi(value));
    } else if (n == "unit_tile") {
        if (v == "auto") h->opt_ut = 0;
        else if (v == "64") h->opt_ut = 64;
        else if (v == "128") h->opt_ut = 128;
        else return fail(h, QGRU_ERR_BAD_ARG, "unit_tile: auto|64|128");
#ifdef QGRU_STAMPS
    } else if (n == "debug_stamps") {
        h->dbg_stamps = reinterpret_cast<long long *>(strtoull(value, nullptr, 10));
#endif
    } else if (n == "test_withhold_arrive") {
        h->opt_withhold = atoi(value) != 0;
    } else if (n == "gemv_r") {
        if (v == "auto") h->opt_gemv_r = 0;
        else if (v == "smem") h->opt_gemv_r = 1;
        else return fail(h, QGRU_ERR_BAD_ARG, "gemv_r: auto|smem");
    } else if (n == "t_chunk") {
        if (v == "auto") h->opt_tchunk = -1;
        else if (atoi(value) >= 0) h->opt_tchunk = atoi(value);
        else return fail(h, QGRU_ERR_BAD_ARG, "t_chunk: auto | 0 (whole sequence) | timesteps per chunk");
    } else if (n == "probe_floor") {
        h->opt_floor = atoi(value) != 0;
    } else if (n == "sm_limit") {
        h->opt_sm_limit = std::max(0, atoi(value));
    } else if (n == "spin_limit") {
        h->spin_limit = (unsigned)std::max(1, atoi(value));
    } else {
        return fail(h, QGRU_ERR_BAD_ARG, "unknown option " + n);
    }
    return QGRU_OK;
}

int qgru_set_params(qgru_handle *h, const qgru_params *p, const float *scale_W,
                    const float *scale_R, const float *scale_bw, const float *scale_br) {
    if (!h || !p || !scale_W || !scale_R || !scale_bw || !scale_br) return QGRU_ERR_BAD_ARG;
    if (p->hidden != h->H) return fail(h, QGRU_ERR_BAD_ARG, "params.hidden != handle hidden_size");
    CK(cudaSetDevice(h->device));
    const int C = h->C;
    const bool pot2 = p->use_pot2 != 0;
    for (int i = 0; i < QGRU_NUM_OPS; ++i)
        if (p->op[i].bits < 1 || p->op[i].bits > 32) return fail(h, QGRU_ERR_BAD_ARG, "bits outside 1..32");
    // W/R/bw/br are symmetric with zp = 0 (ensureSymmetricWeightBiasConfig, src/gru_interface.cc:26-32)
    for (int k : {QGRU_OP_W, QGRU_OP_R, QGRU_OP_BW, QGRU_OP_BR})
        if (!p->op[k].symmetric) return fail(h, QGRU_ERR_UNSUPPORTED, "W/R/bw/br must be symmetric");

    h->params_set = false;
    h->weights_set = false;
    h->p = *p;
    const float *src[4] = {scale_W, scale_R, scale_bw, scale_br};
    for (int k = 0; k < 4; ++k) h->sc[k].assign(src[k], src[k] + C);

    const qgru_op *op = p->op;
    const float s_x = op[QGRU_OP_X].scale, s_h = op[QGRU_OP_H].scale;
    const float s_ih = op[QGRU_OP_IH_LINEAR].scale, s_hh = op[QGRU_OP_HH_LINEAR].scale;

    // fillLinearParams (src/gru_forward_gpu_quant.cu:672-700)
    std::vector<Rescale> rs_x(C), rs_h(C), brs_x(C), brs_h(C);
    std::vector<float> wscale[4];
    for (int k = 0; k < 4; ++k) wscale[k].resize(C);
    bool ok = true;
    for (int c = 0; c < C && ok; ++c) {
        ok = ok && make_rescale_product(scale_W[c], s_x, s_ih, pot2, &rs_x[c]);
        ok = ok && make_rescale_to_product(scale_bw[c], scale_W[c], s_x, pot2, &brs_x[c]);
        ok = ok && make_rescale_product(scale_R[c], s_h, s_hh, pot2, &rs_h[c]);
        ok = ok && make_rescale_to_product(scale_br[c], scale_R[c], s_h, pot2, &brs_h[c]);
        for (int k = 0; k < 4 && ok; ++k) {
            Rescale fs;
            ok = to_fixed_scale(src[k][c], pot2, &fs);
            wscale[k][c] = decode_scale(fs);
        }
        ok = ok && shift_ok(rs_x[c]) && shift_ok(rs_h[c]) && shift_ok(brs_x[c]) && shift_ok(brs_h[c]);
    }
    if (!ok) return fail(h, QGRU_ERR_RANGE, "a per-channel scale cannot be encoded as M*2^-shift");

    // fillGateParams (src/gru_forward_gpu_quant.cu:702-735)
    GateConsts &g = h->gc_host;
    std::memset(&g, 0, sizeof(g));
    g.zp_ih = op[QGRU_OP_IH_LINEAR].zero_point;
    g.zp_hh = op[QGRU_OP_HH_LINEAR].zero_point;
    g.zp_h = op[QGRU_OP_H].zero_point;
    static const int in_op[3] = {QGRU_OP_UPDATE_IN, QGRU_OP_RESET_IN, QGRU_OP_NEW_IN};
    static const int out_op[3] = {QGRU_OP_UPDATE_OUT, QGRU_OP_RESET_OUT, QGRU_OP_NEW_OUT};
    for (int a = 0; a < 3; ++a) {
        g.zp_in[a] = op[in_op[a]].zero_point;
        g.zp_out[a] = op[out_op[a]].zero_point;
        g.in_lo[a] = op_qmin(op[in_op[a]]);
        g.in_hi[a] = op_qmax(op[in_op[a]]);
        g.out_lo[a] = op_qmin(op[out_op[a]]);
        g.out_hi[a] = op_qmax(op[out_op[a]]);
        ok = ok && make_rescale(s_ih, op[in_op[a]].scale, pot2, &g.ih_to[a]);
        g.lut[a] = p->lut[a];
    }
    ok = ok && make_rescale(s_hh, op[QGRU_OP_UPDATE_IN].scale, pot2, &g.hh_to[ACT_Z]);
    ok = ok && make_rescale(s_hh, op[QGRU_OP_RESET_IN].scale, pot2, &g.hh_to[ACT_R]);
    ok = ok && make_rescale_product(op[QGRU_OP_RESET_OUT].scale, s_hh, op[QGRU_OP_NEW_IN].scale, pot2, &g.rh_to_n);
    ok = ok && make_rescale(op[QGRU_OP_NEW_OUT].scale, s_h, pot2, &g.n_to_h);
    ok = ok && make_rescale_product(op[QGRU_OP_UPDATE_OUT].scale, s_h, s_h, pot2, &g.uh_to_h);
    if (!ok) return fail(h, QGRU_ERR_RANGE, "a gate scale cannot be encoded as M*2^-shift");
    for (Rescale r : {g.ih_to[0], g.ih_to[1], g.ih_to[2], g.hh_to[0], g.hh_to[1], g.rh_to_n, g.n_to_h, g.uh_to_h})
        if (!shift_ok(r)) return fail(h, QGRU_ERR_UNSUPPORTED, "rescale shift outside [-62, 62]");
    for (int a = 0; a < 3; ++a)
        for (int s = 0; s < QGRU_LUT_SEGMENTS; ++s) {
            const int n = (int)(int8_t)p->lut[a].seg[s].n_bx;
            if (n > 62 || n < -62) return fail(h, QGRU_ERR_UNSUPPORTED, "LUT shift outside [-62, 62]");
        }
    for (Rescale *r : {&g.ih_to[0], &g.ih_to[1], &g.ih_to[2], &g.hh_to[0], &g.hh_to[1], &g.rh_to_n, &g.n_to_h, &g.uh_to_h})
        set_fast_form(r);
    h->rs_fast[0] = h->rs_fast[1] = true;
    for (int c = 0; c < C; ++c) {
        set_fast_form(&rs_x[c]);
        set_fast_form(&rs_h[c]);
        h->rs_fast[0] = h->rs_fast[0] && rs_x[c].mq != 0;
        h->rs_fast[1] = h->rs_fast[1] && rs_h[c].mq != 0;
    }
    // quant_one_in_update_gate_scale_ (src/gru_forward_gpu_quant.cu:719-720)
    g.one_q = (int32_t)rintf(1.0f / op[QGRU_OP_UPDATE_OUT].scale) + op[QGRU_OP_UPDATE_OUT].zero_point;
    g.h_lo = op_qmin(op[QGRU_OP_H]);
    g.h_hi = op_qmax(op[QGRU_OP_H]);
    g.ih_lo = op_qmin(op[QGRU_OP_IH_LINEAR]);
    g.ih_hi = op_qmax(op[QGRU_OP_IH_LINEAR]);
    g.hh_lo = op_qmin(op[QGRU_OP_HH_LINEAR]);
    g.hh_hi = op_qmax(op[QGRU_OP_HH_LINEAR]);
    {
        Rescale fx, fh;
        if (!to_fixed_scale(s_x, pot2, &fx) || !to_fixed_scale(s_h, pot2, &fh))
            return fail(h, QGRU_ERR_RANGE, "x or h scale cannot be encoded");
        h->x_scale = decode_scale(fx);
        h->h_scale = decode_scale(fh);
        g.h_scale = h->h_scale;
    }
    g.narrow = narrow_ok(g.ih_to[0], max_abs_diff(op[QGRU_OP_IH_LINEAR])) &&
               narrow_ok(g.ih_to[1], max_abs_diff(op[QGRU_OP_IH_LINEAR])) &&
               narrow_ok(g.ih_to[2], max_abs_diff(op[QGRU_OP_IH_LINEAR])) &&
               narrow_ok(g.hh_to[0], max_abs_diff(op[QGRU_OP_HH_LINEAR])) &&
               narrow_ok(g.hh_to[1], max_abs_diff(op[QGRU_OP_HH_LINEAR])) &&
               narrow_ok(g.n_to_h, max_abs_diff(op[QGRU_OP_NEW_OUT]));

    // Tabulate each activation over its whole clamped input range when that range is small.
    std::vector<int32_t> tables;
    for (int a = 0; a < 3; ++a) {
        g.table_size[a] = 0;
        g.table_off[a] = 0;
        if (op[in_op[a]].bits <= 10) {
            const int n = g.in_hi[a] - g.in_lo[a] + 1;
            g.table_off[a] = (int32_t)tables.size();
            g.table_size[a] = n;
            for (int q = g.in_lo[a]; q <= g.in_hi[a]; ++q)
                tables.push_back(lut_eval(p->lut[a], q, op[in_op[a]], op[out_op[a]]));
        }
    }
    h->n_table = (int)tables.size();

    // Tables of the fused cell (gru_cell_fused): every entry is computed with the same host
    // functions the kernels' generic path uses, so both forms give identical results.
    std::vector<int32_t> ft;
    {
        bool fused = g.table_size[0] > 0 && g.table_size[1] > 0 && g.table_size[2] > 0 &&
                     op[QGRU_OP_HH_LINEAR].bits <= 10 && op[QGRU_OP_IH_LINEAR].bits <= 16;
        const auto resc = [](int64_t v, Rescale r) { return (int32_t)rescale64(v, r); };
        int64_t max_zd = 0, max_omz = 0, max_rd = 0, max_nd = 0, max_pre = 0;
        g.k1 = g.one_q - 2 * g.zp_out[ACT_Z];
        if (fused) {
            for (int a = 0; a < 3; ++a) {
                g.ft_off[a] = (int32_t)ft.size();
                for (int q = g.in_lo[a]; q <= g.in_hi[a]; ++q) {
                    const int32_t y = lut_eval(p->lut[a], q, op[in_op[a]], op[out_op[a]]);
                    if (a == ACT_N) {
                        const int32_t nd = resc((int64_t)y - g.zp_out[ACT_N], g.n_to_h);
                        max_nd = std::max<int64_t>(max_nd, std::llabs((long long)nd));
                        ft.push_back(nd);
                    } else {
                        const int32_t d = y - g.zp_out[a];
                        if (a == ACT_Z) {
                            max_zd = std::max<int64_t>(max_zd, std::llabs((long long)d));
                            max_omz = std::max<int64_t>(max_omz, std::llabs((long long)g.k1 - d));
                        } else {
                            max_rd = std::max<int64_t>(max_rd, std::llabs((long long)d));
                        }
                        ft.push_back(d);
                    }
                }
            }
            for (int a = 0; a < 2; ++a) {
                g.ft_off[3 + a] = (int32_t)ft.size();
                for (int v = g.hh_lo; v <= g.hh_hi; ++v) ft.push_back(resc((int64_t)v - g.zp_hh, g.hh_to[a]));
            }
            for (int a = 0; a < 3; ++a)
                for (int64_t v = g.ih_lo; v <= g.ih_hi; v += std::max<int64_t>(1, ((int64_t)g.ih_hi - g.ih_lo))) {
                    // rescale is monotone: the extremes of the range bound every value
                    const int64_t y = (int64_t)resc(v - g.zp_ih, g.ih_to[a]) + g.zp_in[a];
                    max_pre = std::max<int64_t>(max_pre, std::llabs((long long)y));
                }
            g.ft_ih_off = (int32_t)ft.size();
            g.ft_ih_n = 0;
            if (op[QGRU_OP_IH_LINEAR].bits <= 10) {
                g.ft_ih_n = g.ih_hi - g.ih_lo + 1;
                for (int a = 0; a < 3; ++a)
                    for (int v = g.ih_lo; v <= g.ih_hi; ++v)
                        ft.push_back(resc((int64_t)v - g.zp_ih, g.ih_to[a]) + g.zp_in[a]);
            }
            const int64_t max_hd = max_abs_diff(op[QGRU_OP_H]), max_hhd = max_abs_diff(op[QGRU_OP_HH_LINEAR]);
            const int64_t lim = 0x7fffffffll;
            if (max_zd * max_hd + max_omz * max_nd >= lim || max_rd * max_hhd >= lim || max_pre >= lim) fused = false;
            // round-half-up is enough for the cell's two rescales where no operand in range is an exact tie
            const int64_t rh = max_rd * max_hhd, cb = max_zd * max_hd + max_omz * max_nd;
            g.cell_notie = (!rescale_can_tie(g.rh_to_n.mult, g.rh_to_n.shift, -rh, rh) &&
                            !rescale_can_tie(g.uh_to_h.mult, g.uh_to_h.shift, -cb, cb)) ? 1 : 0;
        }
        if (fused) {
            for (int k = 0; k < 3; ++k) {
                g.fi_c[k] = g.ft_off[k] - g.in_lo[k];
                g.fi_lo[k] = g.ft_off[k];
                g.fi_hi[k] = g.ft_off[k] + (g.in_hi[k] - g.in_lo[k]);
            }
            for (int k = 3; k < 5; ++k) {
                g.fi_c[k] = g.zp_hh - g.hh_lo + g.ft_off[k];
                g.fi_lo[k] = g.ft_off[k];
                g.fi_hi[k] = g.ft_off[k] + (g.hh_hi - g.hh_lo);
            }
            g.hn_clo = g.hh_lo - g.zp_hh;
            g.hn_chi = g.hh_hi - g.zp_hh;
        }
        g.fused_ok = fused ? 1 : 0;
        g.ih_pre_bytes = max_pre < 32768 ? 2 : 4;
        if (!fused) ft.clear();
    }
    h->n_ftable = (int)ft.size();

    // storage plan of the 8-bit path
    const auto fits8 = [](const qgru_op &o) { return o.bits <= 8; };
    h->x_uns = op[QGRU_OP_X].bits < 32 && op[QGRU_OP_X].is_unsigned;
    h->h_uns = op[QGRU_OP_H].bits < 32 && op[QGRU_OP_H].is_unsigned;
    const qgru_op &ihop = op[QGRU_OP_IH_LINEAR];
    const bool ih8 = ihop.bits <= 8 && !ihop.is_unsigned;
    const bool ih16 = ihop.bits <= 15 || (ihop.bits == 16 && !ihop.is_unsigned);
    h->ih_bytes = ih8 ? 1 : 2;
    h->fast = fits8(op[QGRU_OP_X]) && fits8(op[QGRU_OP_H]) && fits8(op[QGRU_OP_W]) &&
              !op[QGRU_OP_W].is_unsigned && fits8(op[QGRU_OP_R]) && !op[QGRU_OP_R].is_unsigned &&
              (ih8 || ih16) && (int64_t)std::max(h->I, h->H) * 128 * 255 < (int64_t)0x7fffffff;

    int rc;
    if ((rc = alloc_dev(h, &h->d_gc, 1))) return rc;
    if ((rc = alloc_dev(h, &h->d_tables, tables.size()))) return rc;
    if ((rc = alloc_dev(h, &h->d_ftables, ft.size()))) return rc;
    if (!ft.empty()) CK(cudaMemcpy(h->d_ftables, ft.data(), ft.size() * 4, cudaMemcpyHostToDevice));
    for (int s = 0; s < 2; ++s) {
        if ((rc = alloc_dev(h, &h->d_rs[s], C))) return rc;
        if ((rc = alloc_dev(h, &h->d_brs[s], C))) return rc;
        if ((rc = alloc_dev(h, &h->d_fl[s], C))) return rc;
        if ((rc = alloc_dev(h, &h->d_corr[s], C))) return rc;
        if ((rc = alloc_dev(h, &h->d_wsum[s], C))) return rc;
    }
    for (int k = 0; k < 4; ++k)
        if ((rc = alloc_dev(h, &h->d_wscale[k], C))) return rc;
    CK(cudaMemcpy(h->d_gc, &g, sizeof(g), cudaMemcpyHostToDevice));
    if (!tables.empty())
        CK(cudaMemcpy(h->d_tables, tables.data(), tables.size() * 4, cudaMemcpyHostToDevice));
    CK(cudaMemcpy(h->d_rs[0], rs_x.data(), C * sizeof(Rescale), cudaMemcpyHostToDevice));
    CK(cudaMemcpy(h->d_rs[1], rs_h.data(), C * sizeof(Rescale), cudaMemcpyHostToDevice));
    CK(cudaMemcpy(h->d_brs[0], brs_x.data(), C * sizeof(Rescale), cudaMemcpyHostToDevice));
    CK(cudaMemcpy(h->d_brs[1], brs_h.data(), C * sizeof(Rescale), cudaMemcpyHostToDevice));
    for (int k = 0; k < 4; ++k)
        CK(cudaMemcpy(h->d_wscale[k], wscale[k].data(), C * sizeof(float), cudaMemcpyHostToDevice));
    h->params_set = true;
    h->fs_ready = false;
    return QGRU_OK;
}

}  // extern "C"

namespace {

// Pack int32 weights already resident in h->d_wq[] and derive the per-channel corrections.
int finish_weights(qgru_handle *h, cudaStream_t st) {
    const int C = h->C;
    int rc;
    if (h->fast) {
        // rows are allocated (and zeroed) past 3H so that every 128-row tile load stays inside
        h->w8_rows[0] = (C + 127) / 128 * 128;
        h->w8_rows[1] = C + 256;
        if ((rc = alloc_dev(h, &h->d_w8[0], (size_t)h->w8_rows[0] * h->Ipad))) return rc;
        if ((rc = alloc_dev(h, &h->d_w8[1], (size_t)h->w8_rows[1] * h->Hpad))) return rc;
        CK(cudaMemsetAsync(h->d_w8[0], 0, (size_t)h->w8_rows[0] * h->Ipad, st));
        CK(cudaMemsetAsync(h->d_w8[1], 0, (size_t)h->w8_rows[1] * h->Hpad, st));
    }
    CK(cudaMemsetAsync(h->d_flags, 0, 2 * sizeof(int), st));
    k_pack_weights<<<C, 128, 0, st>>>(h->d_wq[0], h->fast ? h->d_w8[0] : nullptr, h->d_wsum[0], h->I,
                                      h->Ipad, C, h->d_flags);
    k_pack_weights<<<C, 128, 0, st>>>(h->d_wq[1], h->fast ? h->d_w8[1] : nullptr, h->d_wsum[1], h->H,
                                      h->Hpad, C, h->d_flags);
    const int gb = (C + 127) / 128;
    k_channel_consts<<<gb, 128, 0, st>>>(h->d_wq[2], h->d_brs[0], h->d_wsum[0],
                                         h->p.op[QGRU_OP_X].zero_point, h->d_corr[0], h->d_rs[0], h->d_fl[0], C,
                                         (long long)h->I * 128 * 255, h->d_flags, 8);
    k_channel_consts<<<gb, 128, 0, st>>>(h->d_wq[3], h->d_brs[1], h->d_wsum[1],
                                         h->p.op[QGRU_OP_H].zero_point, h->d_corr[1], h->d_rs[1], h->d_fl[1], C,
                                         (long long)h->H * 128 * 255, h->d_flags, 16);
    h->launches += 4;
    CK(cudaGetLastError());
    CK(cudaMemcpyAsync(h->h_flags, h->d_flags, 2 * sizeof(int), cudaMemcpyDeviceToHost, st));
    CK(cudaStreamSynchronize(st));
    if (h->fast && (h->h_flags[0] & 2))
        return fail(h, QGRU_ERR_BAD_ARG, "quantized weight outside the 8-bit range its operator declares");
    h->lin_fits32[0] = !(h->h_flags[0] & 8);
    h->lin_fits32[1] = !(h->h_flags[0] & 16);
    h->lin_notie[0] = !(h->h_flags[0] & 32);
    h->lin_notie[1] = !(h->h_flags[0] & 64);
    h->tc.valid = false;
    h->rec.valid = false;
    h->rec_cl.valid = false;
    h->rec_c64.valid = false;
    h->weights_set = true;
    h->fs_ready = false;
    return QGRU_OK;
}

}  // namespace

extern "C" {

int qgru_set_weights_f32(qgru_handle *h, const float *W, const float *R, const float *bw,
                         const float *br, void *stream) {
    if (!h || !W || !R || !bw || !br) return QGRU_ERR_BAD_ARG;
    if (!h->params_set) return fail(h, QGRU_ERR_NOT_READY, "set_params first");
    CK(cudaSetDevice(h->device));
    cudaStream_t st = (cudaStream_t)stream;
    const int C = h->C;
    const size_t n[4] = {(size_t)h->I * C, (size_t)h->H * C, (size_t)C, (size_t)C};
    const float *src[4] = {W, R, bw, br};
    const int opi[4] = {QGRU_OP_W, QGRU_OP_R, QGRU_OP_BW, QGRU_OP_BR};
    int rc;
    for (int k = 0; k < 4; ++k) {
        if ((rc = alloc_dev(h, &h->d_wq[k], n[k]))) return rc;
        k_quantize_weights<<<grid_for((long long)n[k], 256, h->sm_count), 256, 0, st>>>(
            src[k], h->d_wq[k], (long long)n[k], C, h->d_wscale[k], op_qmin(h->p.op[opi[k]]),
            op_qmax(h->p.op[opi[k]]));
        h->launches++;
    }
    CK(cudaGetLastError());
    return finish_weights(h, st);
}

int qgru_set_weights_i32(qgru_handle *h, const int32_t *W_q, const int32_t *R_q,
                         const int32_t *bw_q, const int32_t *br_q, void *stream) {
    if (!h || !W_q || !R_q || !bw_q || !br_q) return QGRU_ERR_BAD_ARG;
    if (!h->params_set) return fail(h, QGRU_ERR_NOT_READY, "set_params first");
    CK(cudaSetDevice(h->device));
    cudaStream_t st = (cudaStream_t)stream;
    const int C = h->C;
    const size_t n[4] = {(size_t)h->I * C, (size_t)h->H * C, (size_t)C, (size_t)C};
    const int32_t *src[4] = {W_q, R_q, bw_q, br_q};
    int rc;
    for (int k = 0; k < 4; ++k) {
        if ((rc = alloc_dev(h, &h->d_wq[k], n[k]))) return rc;
        CK(cudaMemcpyAsync(h->d_wq[k], src[k], n[k] * 4, cudaMemcpyDeviceToDevice, st));
    }
    return finish_weights(h, st);
}

int qgru_get_weights_i32(qgru_handle *h, int32_t *W_q, int32_t *R_q, int32_t *bw_q, int32_t *br_q,
                         void *stream) {
    if (!h) return QGRU_ERR_BAD_ARG;
    if (!h->weights_set) return fail(h, QGRU_ERR_NOT_READY, "set_weights first");
    CK(cudaSetDevice(h->device));
    cudaStream_t st = (cudaStream_t)stream;
    const int C = h->C;
    const size_t n[4] = {(size_t)h->I * C, (size_t)h->H * C, (size_t)C, (size_t)C};
    int32_t *dst[4] = {W_q, R_q, bw_q, br_q};
    for (int k = 0; k < 4; ++k)
        if (dst[k]) CK(cudaMemcpyAsync(dst[k], h->d_wq[k], n[k] * 4, cudaMemcpyDeviceToDevice, st));
    return QGRU_OK;
}

}  // extern "C"

namespace {

LinearConsts linear_consts(const qgru_handle *h, int side) {
    LinearConsts lc;
    lc.corr = h->d_corr[side];
    lc.rs = h->d_rs[side];
    lc.fl = h->d_fl[side];
    const qgru_op &o = h->p.op[side == 0 ? QGRU_OP_IH_LINEAR : QGRU_OP_HH_LINEAR];
    lc.zp_out = o.zero_point;
    lc.lo = op_qmin(o);
    lc.hi = op_qmax(o);
    lc.fits32 = h->fast && h->lin_fits32[side] ? 1 : 0;
    return lc;
}

bool use_generic(const qgru_handle *h) { return !h->fast || h->opt_rec == 3; }

template <bool HU, typename IhT>
int launch_rec(qgru_handle *h, RecArgs &a, const RecPlan &pl, cudaStream_t st) {
    auto kern = h->gc_host.narrow ? k_recurrence_dp4a<HU, IhT, true> : k_recurrence_dp4a<HU, IhT, false>;
    CK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pl.smem));
    const int grid = pl.G * pl.P;
    if (pl.P > 1) {
        if (!h->coop) return fail(h, QGRU_ERR_UNSUPPORTED, "device lacks cooperative launch");
        int per_sm = 0;
        CK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, 256, pl.smem));
        if ((long long)per_sm * h->sm_count < grid)
            return fail(h, QGRU_ERR_UNSUPPORTED, "recurrence grid cannot be co-resident");
        void *args[] = {&a};
        CK(cudaLaunchCooperativeKernel((void *)kern, dim3(grid), dim3(256), args, pl.smem, st));
    } else {
        kern<<<grid, 256, pl.smem, st>>>(a);
        CK(cudaGetLastError());
    }
    h->launches++;
    return QGRU_OK;
}

// Small-batch form: one CTA per batch row, whole R in shared memory (H <= 256).
size_t gemv_smem(const qgru_handle *h, int n_table) {
    const size_t units = (size_t)(h->H + 31) / 32 * 32;
    return (((size_t)n_table * 4 + 15) & ~size_t(15)) + (size_t)2 * (h->Hpad + 64) + (size_t)3 * units * h->Hpad;
}
bool gemv_fits(const qgru_handle *h) {
    const int n_tab = std::max(h->n_table, h->gc_host.fused_ok ? h->gc_host.ft_ih_off : 0);
    return h->Hpad <= 256 && gemv_smem(h, n_tab) <= (size_t)h->smem_optin;
}

// The register-resident form of the one-CTA-per-row recurrence: the tabulated branch-free cell, Hpad
// 128 or 256 (option gemv_r=smem keeps R in shared memory).
bool gemv_reg_ok(const qgru_handle *h, bool fused) { return fused && h->opt_gemv_r != 1 && (h->Hpad == 128 || h->Hpad == 256); }
size_t gemv_reg_smem(const qgru_handle *h, int n_table) {
    const size_t units = (size_t)(h->H + 31) / 32 * 32;
    return (((size_t)n_table * 4 + 15) & ~size_t(15)) + (size_t)2 * 2 * (h->Hpad / 2 + 16) + 3 * units * sizeof(int) +
           3 * units * sizeof(FastLin);
}

template <bool HU, typename IhT>
int launch_gemv_reg(qgru_handle *h, RecArgs &a, cudaStream_t st) {
    auto kern = h->Hpad == 128 ? k_recurrence_gemv_reg<HU, IhT, 64> : k_recurrence_gemv_reg<HU, IhT, 128>;
    const size_t smem = gemv_reg_smem(h, a.n_table);
    CK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    const int threads = 2 * ((h->H + 31) / 32 * 32);
    kern<<<a.B, threads, smem, st>>>(h->gc_host, a);
    CK(cudaGetLastError());
    h->launches++;
    return QGRU_OK;
}

template <bool HU, typename IhT>
int launch_gemv(qgru_handle *h, RecArgs &a, bool fused, cudaStream_t st) {
    if (gemv_reg_ok(h, fused)) return launch_gemv_reg<HU, IhT>(h, a, st);
    auto kern = fused ? k_recurrence_gemv<HU, IhT, 2>
                      : (h->gc_host.narrow ? k_recurrence_gemv<HU, IhT, 1> : k_recurrence_gemv<HU, IhT, 0>);
    const size_t smem = gemv_smem(h, a.n_table);
    CK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    const int threads = 4 * ((h->H + 31) / 32 * 32);
    kern<<<a.B, threads, smem, st>>>(h->gc_host, a);
    CK(cudaGetLastError());
    h->launches++;
    return QGRU_OK;
}

// Shared tail of the two device entry points, 8-bit path: x8 and the initial state are ready.
int run_fast(qgru_handle *h, int T, int B, int32_t *hq_out, float *hf_out, unsigned flags,
             cudaStream_t st, uint8_t *h8_out = nullptr) {
    const long long N = (long long)T * B;
    const int C = h->C;
    int rc;

    // ---- plan the recurrence first: it decides the form in which W*x+bw is stored
    const int sms = h->opt_sm_limit > 0 ? std::min(h->opt_sm_limit, h->sm_count) : h->sm_count;
    RecPlan pl;
    const bool dp4a_ok = plan_recurrence(h, B, &pl);
    RecMmaPlan mp;
    const int n_tab_mma = std::max(h->n_table, h->gc_host.fused_ok ? h->gc_host.ft_ih_off : 0);
    // two tensor-core forms: state exchanged through distributed shared memory (one cluster per
    // group; H <= 1024) or through global memory with a counter per group (H <= 512)
    RecMmaPlan cp;
    const bool cluster_ok = h->opt_rec != 1 && h->opt_exchange != 1 &&
                            rec_cluster_plan(h->H, h->Hpad, B, sms, h->smem_optin, n_tab_mma, h->opt_r_where, h->opt_mt, h->opt_ng, h->opt_kp, &cp);
    const bool global_ok = h->opt_rec != 1 && rec_mma_plan(h->H, h->Hpad, B, sms, h->smem_optin, n_tab_mma, &mp);
    const bool mma_ok = cluster_ok || global_ok;
    if (h->opt_rec == 2 && !mma_ok)
        return fail(h, QGRU_ERR_UNSUPPORTED, "tensor-core recurrence needs H <= 1024 (H <= 512 with exchange=global)");
    // Tiny batches whose R fits one SM run barrier-free on one CTA per batch row: lower latency
    // than tensor-core tiles of 16 batch columns.
    bool use_mma = mma_ok && (h->opt_rec == 2 || !(dp4a_ok && pl.P == 1 && B <= 4));
    // One CTA per row with the whole R on chip: no synchronisation between CTAs at all.  Taken
    // while the rows fit one wave of SMs (beyond that the tensor-core tiles win on throughput).
    const bool gemv_ok = gemv_fits(h) && h->opt_rec != 1 && h->opt_rec != 2;
    if (h->opt_rec == 4 && !gemv_ok) return fail(h, QGRU_ERR_UNSUPPORTED, "rec=gemv needs H <= 256");
    const bool use_gemv = gemv_ok && (h->opt_rec == 4 || (h->opt_rec == 0 && B <= sms));
    if (use_gemv) use_mma = false;
    const bool use_cluster = use_mma && cluster_ok;
    if (h->opt_exchange == 2 && use_mma && !use_cluster)
        return fail(h, QGRU_ERR_UNSUPPORTED, "cluster exchange does not fit shared memory");
    if (use_cluster) mp = cp;
    if (!use_mma && !use_gemv && !dp4a_ok) return fail(h, QGRU_ERR_UNSUPPORTED, "no recurrence plan fits shared memory");
    // the fused cell needs the GEMM epilogue to pre-rescale W*x+bw: tensor-core GEMM only
    // (the one-CTA-per-row form takes it only in its branch-free shape: every scale shift-free)
    const bool gemv_fused = use_gemv && h->opt_cell == 0 && h->lin_fits32[1] && h->rs_fast[1] &&
                            h->gc_host.rh_to_n.mq != 0 && h->gc_host.uh_to_h.mq != 0;
    const bool fused = (use_mma || gemv_fused) && h->gc_host.fused_ok && h->opt_gemm != 1 && h->opt_cell != 1;
    const int ih_bytes = fused ? h->gc_host.ih_pre_bytes : h->ih_bytes;
    // The 64-units-per-CTA form of the cluster recurrence: only the branch-free tabulated cell, and only
    // on request (option unit_tile=64): measured slower than the 128-unit form so far.
    const bool fast_cell_ok = fused && use_cluster && h->opt_cell != 2 && h->lin_fits32[1] && h->rs_fast[1] &&
                              h->gc_host.rh_to_n.mq != 0 && h->gc_host.uh_to_h.mq != 0;
    RecMmaPlan c64;
    const bool use_c64 = fast_cell_ok && h->opt_ut == 64 && h->opt_ng != 1 && h->opt_mt != 2 && !h->opt_floor && h->opt_r_where != 1 &&
                         rec_c64_plan(h->H, h->Hpad, B, sms, h->smem_optin, h->gc_host.ft_ih_off, h->opt_ut == 64, &c64);
    if (h->opt_ut == 64 && use_mma && !use_c64)
        return fail(h, QGRU_ERR_UNSUPPORTED, "unit_tile=64 needs the fused shift-free cell, H <= 512 and at most 96 rows per cluster");
    if (use_c64) mp = c64;
    PreScale ps{};
    if (fused) {
        ps.enabled = 1;
        ps.H = h->H;
        ps.zp_ih = h->gc_host.zp_ih;
        for (int a = 0; a < 3; ++a) {
            ps.to[a] = h->gc_host.ih_to[a];
            ps.zp_in[a] = h->gc_host.zp_in[a];
        }
        if (h->gc_host.ft_ih_n > 0) {
            ps.table = h->d_ftables + h->gc_host.ft_ih_off;
            ps.table_n = h->gc_host.ft_ih_n;
            ps.lo = h->gc_host.ih_lo;
        }
    }
    // ---- chunks of timesteps (cluster recurrence with the tensor-core GEMM): W*x+bw exists for two
    // chunks at a time instead of the whole sequence, and the GEMM of chunk k+1 runs on a second,
    // low-priority stream beside the recurrence of chunk k, which picks up its initial state where
    // the launch before it left it (RecMmaArgs::write_final).  Automatic where the recurrence
    // leaves at least half of the SMs to the GEMM and the sequence is long enough to pay for the
    // extra launches; one chunk otherwise.
    int Tc = T;
    {
        const bool can_chunk = use_cluster && !use_c64 && !h->opt_floor && h->opt_gemm != 1 && h->Ipad % 128 == 0 &&
                               h->w8_rows[0] >= (long long)(C + 127) / 128 * 128;
        if (can_chunk && h->opt_tchunk > 0) Tc = std::min(T, h->opt_tchunk);
        else if (can_chunk && h->opt_tchunk < 0 && mp.G * mp.P * 2 <= sms && T >= 256) Tc = (T + 7) / 8;
    }
    const int n_chunks = (T + Tc - 1) / Tc;
    const size_t chunk_bytes = ((size_t)Tc * B * C * ih_bytes + 255) & ~size_t(255);
    if ((rc = ensure(h, h->ih, n_chunks > 1 ? 2 * chunk_bytes : (size_t)N * C * ih_bytes))) return rc;
    if (n_chunks > 1 && !h->aux) {
        int lo = 0, hi = 0;
        CK(cudaDeviceGetStreamPriorityRange(&lo, &hi));
        CK(cudaStreamCreateWithPriority(&h->aux, cudaStreamNonBlocking, lo));
        for (int i = 0; i < 2; ++i) {
            CK(cudaEventCreateWithFlags(&h->ev_g[i], cudaEventDisableTiming));
            CK(cudaEventCreateWithFlags(&h->ev_r[i], cudaEventDisableTiming));
        }
        CK(cudaEventCreateWithFlags(&h->ev_fork, cudaEventDisableTiming));
    }
    const bool rev_dir = (flags & QGRU_FLAG_REVERSE) != 0;
    // chunk k covers steps [k*Tc, min(T, (k+1)*Tc)), i.e. timesteps from t_lo(k) on
    auto chunk_T = [&](int k) { return std::min(T, (k + 1) * Tc) - k * Tc; };
    auto chunk_t0 = [&](int k) { return rev_dir ? T - (k * Tc + chunk_T(k)) : k * Tc; };
    auto chunk_ih = [&](int k) { return (void *)((char *)h->ih.p + (n_chunks > 1 ? (size_t)(k & 1) * chunk_bytes : 0)); };

    CK(cudaEventRecord(h->ev[1], st));
    const LinearConsts lcx = linear_consts(h, 0);
    bool used_tc = false;
    // the W*x GEMM of chunk k on stream `gs`
    auto gemm_chunk = [&](int k, cudaStream_t gs) -> int {
        // branch-free epilogue: 32-bit sums and every scale it applies in shift-free form
        // (the launcher also looks at how the second rescale is applied: table or shift-free scale)
        const bool gemm_fast = lcx.fits32 && h->rs_fast[0] && h->opt_cell != 2;
        const long long Nk = (long long)chunk_T(k) * B;
        const int r = tc_gemm_launch(h->tc, (const uint8_t *)h->x8.p, (N + 127) / 128 * 128, h->d_w8[0], h->w8_rows[0],
                                     chunk_ih(k), Nk, C, h->Ipad, h->x_uns, ih_bytes, lcx, ps, gemm_fast,
                                     h->lin_notie[0] && h->opt_tie != 1, h->d_flags + 1, sms, gs, &h->err,
                                     (long long)chunk_t0(k) * B);
        if (r == QGRU_OK) h->launches++;
        return r;
    };
    if (n_chunks > 1) {
        CK(cudaEventRecord(h->ev_fork, st));
        CK(cudaStreamWaitEvent(h->aux, h->ev_fork, 0));
    }
    if (h->opt_gemm != 1) {
        rc = gemm_chunk(0, st);
        if (rc == QGRU_OK) {
            used_tc = true;
        } else if (rc != QGRU_ERR_UNSUPPORTED || h->opt_gemm == 2 || fused || n_chunks > 1) {
            return rc;
        }
    }
    if (!used_tc) {
        dim3 grid((unsigned)((N + 63) / 64), (unsigned)((C + 63) / 64));
        const uint8_t *x8 = (const uint8_t *)h->x8.p;
        if (h->ih_bytes == 1) {
            if (h->x_uns) k_gemm_wx_simt<true, int8_t><<<grid, 256, 0, st>>>(x8, h->d_w8[0], (int8_t *)h->ih.p, N, C, h->Ipad, lcx);
            else k_gemm_wx_simt<false, int8_t><<<grid, 256, 0, st>>>(x8, h->d_w8[0], (int8_t *)h->ih.p, N, C, h->Ipad, lcx);
        } else {
            if (h->x_uns) k_gemm_wx_simt<true, int16_t><<<grid, 256, 0, st>>>(x8, h->d_w8[0], (int16_t *)h->ih.p, N, C, h->Ipad, lcx);
            else k_gemm_wx_simt<false, int16_t><<<grid, 256, 0, st>>>(x8, h->d_w8[0], (int16_t *)h->ih.p, N, C, h->Ipad, lcx);
        }
        CK(cudaGetLastError());
        h->launches++;
    }
    CK(cudaEventRecord(h->ev[2], st));

    const int groups = use_mma ? mp.G : pl.G;
    if (groups > h->bar_groups) {
        if ((rc = alloc_dev(h, &h->d_bar, (size_t)groups * 32))) return rc;
        h->bar_groups = groups;
    }
    CK(cudaMemsetAsync(h->d_bar, 0, (size_t)groups * 32 * sizeof(unsigned), st));
    char buf[400];
    if (use_mma) {
        RecMmaArgs a;
        a.T = T; a.B = B; a.H = h->H; a.Hpad = h->Hpad; a.C = C;
        a.P = mp.P; a.NB = mp.NB; a.b_off = 0; a.b_cnt = B;
        a.reverse = (flags & QGRU_FLAG_REVERSE) ? 1 : 0;
        a.tmem_cols = (uint32_t)mp.tmem_cols;
        a.ih = h->ih.p;
        a.h8 = (uint8_t *)h->h8.p;
        a.hq_out = hq_out;
        a.hf_out = hf_out;
        a.h8_out = h8_out;
        a.lc = linear_consts(h, 1);
        a.tables = fused ? h->d_ftables : h->d_tables;
        a.n_table = fused ? h->gc_host.ft_ih_off : h->n_table;   // the GEMM-side table stays out of smem
        a.bar = h->d_bar;
        a.abort_flag = h->d_flags + 1;
        a.spin_limit = h->spin_limit;
        a.issue_delay = h->opt_issue_delay;
#ifdef QGRU_STAMPS
        a.dbg = h->dbg_stamps;
#endif
        const unsigned long long before = h->rec.launches + h->rec_cl.launches + h->rec_c64.launches;
        // the branch-free fused cell: every scale of the step in shift-free form, 32-bit sums
        const bool fast_cell = fused && use_cluster && h->opt_cell != 2 && a.lc.fits32 && h->rs_fast[1] &&
                               h->gc_host.rh_to_n.mq != 0 && h->gc_host.uh_to_h.mq != 0;
        // round-half-up suffices where no operand in range can be an exact tie (R*h requantization and the
        // cell's two rescales): checked when the weights / parameters were set
        const bool cell_notie = fast_cell && h->lin_notie[1] && h->gc_host.cell_notie != 0 && h->opt_tie != 1;
        if (use_c64)
            rc = rec_c64_launch(h->rec_c64, mp, a, h->gc_host, h->d_w8[1], h->w8_rows[1], (long long)2 * B + 256, h->h_uns,
                                ih_bytes, cell_notie, st, &h->err);
        else if (use_cluster) {
            const size_t BHs = (size_t)B * h->H;
            for (int k = 0; k < n_chunks && rc == QGRU_OK; ++k) {
                if (n_chunks > 1) {
                    // the next chunk's GEMM goes to the second stream first: its buffer is free once the
                    // recurrence of chunk k-1 has read it
                    if (k + 1 < n_chunks) {
                        if (k >= 1) CK(cudaStreamWaitEvent(h->aux, h->ev_r[(k + 1) & 1], 0));
                        if ((rc = gemm_chunk(k + 1, h->aux))) break;
                        CK(cudaEventRecord(h->ev_g[(k + 1) & 1], h->aux));
                    }
                    if (k >= 1) CK(cudaStreamWaitEvent(st, h->ev_g[k & 1], 0));
                    const size_t slot0 = (size_t)chunk_t0(k) * BHs;   // first output slot of the chunk (both directions)
                    a.T = chunk_T(k);
                    a.ih = chunk_ih(k);
                    a.hq_out = hq_out ? hq_out + slot0 : nullptr;
                    a.hf_out = hf_out ? hf_out + slot0 : nullptr;
                    a.h8_out = h8_out ? h8_out + slot0 : nullptr;
                    a.write_final = k + 1 < n_chunks ? 1 : 0;
                }
                rc = rec_cluster_launch(h->rec_cl, mp, a, h->gc_host, h->d_w8[1], h->w8_rows[1], (long long)2 * B + 256,
                                        h->h_uns, ih_bytes, fused ? fast_cell : h->gc_host.narrow != 0, fused, h->opt_floor,
                                        cell_notie, st, &h->err);
                if (n_chunks > 1 && rc == QGRU_OK) CK(cudaEventRecord(h->ev_r[k & 1], st));
            }
        } else
            rc = rec_mma_launch(h->rec, mp, a, h->gc_host, h->d_w8[1], h->w8_rows[1], (long long)2 * B + 256,
                                h->h_uns, ih_bytes, h->gc_host.narrow != 0, fused, h->coop != 0, st, &h->err);
        if (rc) return rc;
        h->launches += h->rec.launches + h->rec_cl.launches + h->rec_c64.launches - before;
        snprintf(buf, sizeof(buf), "path=int8 gemm=%s rec=tcgen05_i8 exchange=%s cell=%s%s UT=%d MT=%d NB=%d NG=%d P=%d G=%d per_launch=%d smem=%zu tmem_cols=%d r_in=%s narrow=%d ih_bytes=%d shiftfree=%d%d%d%d tie_free=%d%d t_chunks=%d",
                 used_tc ? "tcgen05_i8" : "simt_dp4a", use_cluster ? "cluster_dsmem" : "global", fast_cell ? "fused_shiftfree" : fused ? "fused" : "generic", (use_cluster && h->opt_floor) ? "(FLOOR PROBE: no MMAs, no cell)" : "", use_c64 ? 64 : 128, mp.MT, mp.NB, mp.NG, mp.P, mp.G,
                 mp.groups_per_launch, mp.smem, mp.tmem_cols, !use_cluster || mp.tmem_tiles == 0 ? "smem" : ((use_c64 || mp.tmem_tiles == mp.MT * 3 * (h->Hpad / 128)) ? "tmem" : "tmem+smem"),
                 h->gc_host.narrow, ih_bytes, (int)a.lc.fits32,
                 (int)h->rs_fast[1], h->gc_host.rh_to_n.mq != 0, h->gc_host.uh_to_h.mq != 0,
                 (int)(used_tc && h->lin_notie[0] && h->opt_tie != 1), (int)cell_notie, n_chunks);
    } else {
        RecArgs a;
        a.T = T; a.B = B; a.H = h->H; a.Hpad = h->Hpad; a.C = C;
        a.Hs = pl.Hs; a.Bt = pl.Bt; a.P = pl.P;
        a.reverse = (flags & QGRU_FLAG_REVERSE) ? 1 : 0;
        a.r8 = h->d_w8[1];
        a.ih = h->ih.p;
        a.h8 = (uint8_t *)h->h8.p;
        a.hq_out = hq_out;
        a.hf_out = hf_out;
        a.h8_out = h8_out;
        a.lc = linear_consts(h, 1);
        a.gc = h->d_gc;
        a.tables = h->d_tables;
        a.n_table = h->n_table;
        a.bar = h->d_bar;
        a.abort_flag = h->d_flags + 1;
        a.spin_limit = h->spin_limit;
        a.withhold_arrive = h->opt_withhold ? 1 : 0;
        if (use_gemv) {
            if (fused) {
                a.tables = h->d_ftables;
                a.n_table = h->gc_host.ft_ih_off;
            }
            if (ih_bytes == 1) rc = h->h_uns ? launch_gemv<true, int8_t>(h, a, fused, st) : launch_gemv<false, int8_t>(h, a, fused, st);
            else if (ih_bytes == 2) rc = h->h_uns ? launch_gemv<true, int16_t>(h, a, fused, st) : launch_gemv<false, int16_t>(h, a, fused, st);
            else rc = h->h_uns ? launch_gemv<true, int32_t>(h, a, fused, st) : launch_gemv<false, int32_t>(h, a, fused, st);
            if (rc) return rc;
            snprintf(buf, sizeof(buf), "path=int8 gemm=%s rec=gemv cell=%s r_in=%s rows_per_cta=1 ctas=%d smem=%zu narrow=%d ih_bytes=%d",
                     used_tc ? "tcgen05_i8" : "simt_dp4a", fused ? "fused_shiftfree" : "generic",
                     gemv_reg_ok(h, fused) ? "registers" : "smem", B,
                     gemv_reg_ok(h, fused) ? gemv_reg_smem(h, a.n_table) : gemv_smem(h, a.n_table), h->gc_host.narrow, ih_bytes);
        } else {
            if (h->ih_bytes == 1) rc = h->h_uns ? launch_rec<true, int8_t>(h, a, pl, st) : launch_rec<false, int8_t>(h, a, pl, st);
            else rc = h->h_uns ? launch_rec<true, int16_t>(h, a, pl, st) : launch_rec<false, int16_t>(h, a, pl, st);
            if (rc) return rc;
            snprintf(buf, sizeof(buf), "path=int8 gemm=%s rec=dp4a Hs=%d Bt=%d P=%d G=%d smem=%zu narrow=%d ih_bytes=%d",
                     used_tc ? "tcgen05_i8" : "simt_dp4a", pl.Hs, pl.Bt, pl.P, pl.G, pl.smem, h->gc_host.narrow, h->ih_bytes);
        }
    }
    CK(cudaEventRecord(h->ev[3], st));
    h->timing_valid = true;
    h->plan_text = buf;
    return QGRU_OK;
}

// Generic path: int32 operands, 64-bit accumulation, one launch pair per step.
int run_generic(qgru_handle *h, int T, int B, const int32_t *x32, int32_t *hq, int32_t *vq, unsigned flags,
                cudaStream_t st, const qgru_masks *mk = nullptr) {
    const long long N = (long long)T * B;
    const int C = h->C, H = h->H;
    int rc;
    if ((rc = ensure(h, h->ih32, (size_t)N * C * 4))) return rc;
    if ((rc = ensure(h, h->hh32, (size_t)B * C * 4))) return rc;
    CK(cudaEventRecord(h->ev[1], st));
    const LinearConsts lcx = linear_consts(h, 0), lch = linear_consts(h, 1);
    {
        dim3 grid((C + 127) / 128, (unsigned)N);
        k_linear_generic<<<grid, 128, 0, st>>>(h->d_wq[0], x32, (int32_t *)h->ih32.p, N, h->I, C, lcx,
                                               mk ? mk->ih_linear : nullptr);
        h->launches++;
    }
    CK(cudaEventRecord(h->ev[2], st));
    const bool rev = flags & QGRU_FLAG_REVERSE;
    const size_t BH = (size_t)B * H;
    for (int s = 0; s < T; ++s) {
        const int t = rev ? T - 1 - s : s;
        const size_t in_slot = rev ? (size_t)(T - s) : (size_t)s;
        const size_t out_slot = rev ? (size_t)(T - 1 - s) : (size_t)(s + 1);
        dim3 g1((C + 127) / 128, B);
        const size_t row = (size_t)t * B;
        k_linear_generic<<<g1, 128, 0, st>>>(h->d_wq[1], hq + in_slot * BH, (int32_t *)h->hh32.p, B, H, C, lch,
                                             mk && mk->hh_linear ? mk->hh_linear + row * C : nullptr);
        dim3 g2((H + 127) / 128, B);
        if (mk)
            k_gates_train<<<g2, 128, 0, st>>>((const int32_t *)h->ih32.p + row * C, (const int32_t *)h->hh32.p,
                                              hq + in_slot * BH, hq + out_slot * BH, vq + row * 4 * H,
                                              mk->gate_input ? mk->gate_input + row * C : nullptr,
                                              mk->gate_output ? mk->gate_output + row * C : nullptr,
                                              mk->h ? mk->h + row * H : nullptr, B, H, h->d_gc);
        else
        k_gates_generic<<<g2, 128, 0, st>>>((const int32_t *)h->ih32.p + (size_t)t * B * C,
                                            (const int32_t *)h->hh32.p, hq + in_slot * BH,
                                            hq + out_slot * BH, vq ? vq + (size_t)t * B * 4 * H : nullptr, B, H,
                                            h->d_gc, h->d_tables);
        h->launches += 2;
    }
    CK(cudaGetLastError());
    CK(cudaEventRecord(h->ev[3], st));
    h->timing_valid = true;
    h->plan_text = "path=generic_i32 gemm=simt_i64 rec=per_step_i64";
    return QGRU_OK;
}

int check_forward_args(qgru_handle *h, int T, int B) {
    if (T <= 0 || B <= 0) return fail(h, QGRU_ERR_BAD_ARG, "T and B must be positive");
    if (!h->params_set || !h->weights_set) return fail(h, QGRU_ERR_NOT_READY, "set_params and set_weights first");
    if ((long long)T * B * std::max(h->C, h->I) > (1ll << 40)) return fail(h, QGRU_ERR_BAD_ARG, "problem too large");
    return QGRU_OK;
}

}  // namespace

extern "C" {

int qgru_forward_i32(qgru_handle *h, int T, int B, const int32_t *x_q, const int32_t *h0_q,
                     int32_t *h_q, unsigned flags, void *stream) {
    if (!h || !x_q || !h_q) return QGRU_ERR_BAD_ARG;
    int rc = check_forward_args(h, T, B);
    if (rc) return rc;
    CK(cudaSetDevice(h->device));
    cudaStream_t st = (cudaStream_t)stream;
    const long long N = (long long)T * B;
    const qgru_op &xo = h->p.op[QGRU_OP_X], &ho = h->p.op[QGRU_OP_H];
    const long long init_slot = (flags & QGRU_FLAG_REVERSE) ? T : 0;
    h->ev = h->ring[h->calls % qgru_handle::kRing];
    h->calls++;
    CK(cudaEventRecord(h->ev[0], st));
    CK(cudaMemsetAsync(h->d_flags, 0, 2 * sizeof(int), st));
    if (use_generic(h)) {
        k_init_state<<<grid_for((long long)B * h->Hpad, 256, h->sm_count), 256, 0, st>>>(
            h0_q, nullptr, nullptr, h_q, nullptr, nullptr, B, h->H, h->Hpad, init_slot, h->h_scale, ho.zero_point,
            op_qmin(ho), op_qmax(ho), h->d_flags);
        h->launches++;
        return run_generic(h, T, B, x_q, h_q, nullptr, flags, st);
    }
    if ((rc = ensure(h, h->x8, (size_t)((N + 127) / 128 * 128) * h->Ipad))) return rc;
    if ((rc = ensure(h, h->h8, (size_t)(2 * B + 256) * h->Hpad))) return rc;
    k_narrow_rows_i32<<<grid_for(N * (h->Ipad / 4), 256, h->sm_count), 256, 0, st>>>(
        x_q, (uint8_t *)h->x8.p, N, h->I, h->Ipad, op_qmin(xo), op_qmax(xo), h->d_flags);
    CK(cudaMemsetAsync(h->h8.p, 0, (size_t)(2 * B + 256) * h->Hpad, st));
    k_init_state<<<grid_for((long long)B * h->Hpad, 256, h->sm_count), 256, 0, st>>>(
        h0_q, nullptr, (uint8_t *)h->h8.p, h_q, nullptr, nullptr, B, h->H, h->Hpad, init_slot, h->h_scale,
        ho.zero_point, op_qmin(ho), op_qmax(ho), h->d_flags);
    h->launches += 2;
    CK(cudaGetLastError());
    return run_fast(h, T, B, h_q, nullptr, flags, st);
}

int qgru_forward_i32_train(qgru_handle *h, int T, int B, const int32_t *x_q, const int32_t *h0_q,
                           int32_t *h_q, int32_t *v_q, const qgru_masks *masks, unsigned flags,
                           void *stream) {
    if (!h || !x_q || !h_q || !v_q) return QGRU_ERR_BAD_ARG;
    int rc = check_forward_args(h, T, B);
    if (rc) return rc;
    CK(cudaSetDevice(h->device));
    cudaStream_t st = (cudaStream_t)stream;
    const qgru_op &ho = h->p.op[QGRU_OP_H];
    const long long init_slot = (flags & QGRU_FLAG_REVERSE) ? T : 0;
    h->ev = h->ring[h->calls % qgru_handle::kRing];
    h->calls++;
    CK(cudaEventRecord(h->ev[0], st));
    CK(cudaMemsetAsync(h->d_flags, 0, 2 * sizeof(int), st));
    // the step-by-step kernels keep every intermediate the training buffer wants
    k_init_state<<<grid_for((long long)B * h->Hpad, 256, h->sm_count), 256, 0, st>>>(
        h0_q, nullptr, nullptr, h_q, nullptr, nullptr, B, h->H, h->Hpad, init_slot, h->h_scale, ho.zero_point,
        op_qmin(ho), op_qmax(ho), h->d_flags);
    h->launches++;
    return run_generic(h, T, B, x_q, h_q, v_q, flags, st, masks);
}

int qgru_forward_f32(qgru_handle *h, int T, int B, const float *x, const float *h0, float *h_out,
                     int32_t *x_q_out, unsigned flags, void *stream) {
    if (!h || !x || !h_out) return QGRU_ERR_BAD_ARG;
    int rc = check_forward_args(h, T, B);
    if (rc) return rc;
    CK(cudaSetDevice(h->device));
    cudaStream_t st = (cudaStream_t)stream;
    const long long N = (long long)T * B;
    const qgru_op &xo = h->p.op[QGRU_OP_X], &ho = h->p.op[QGRU_OP_H];
    const long long init_slot = (flags & QGRU_FLAG_REVERSE) ? T : 0;
    h->ev = h->ring[h->calls % qgru_handle::kRing];
    h->calls++;
    CK(cudaEventRecord(h->ev[0], st));
    CK(cudaMemsetAsync(h->d_flags, 0, 2 * sizeof(int), st));
    if (use_generic(h)) {
        const size_t nh = (size_t)(T + 1) * B * h->H;
        int32_t *x32 = x_q_out;
        if (!x32) {
            if ((rc = ensure(h, h->x32, (size_t)N * h->I * 4))) return rc;
            x32 = (int32_t *)h->x32.p;
        }
        if ((rc = ensure(h, h->hq32, nh * 4))) return rc;
        k_quantize_f32_i32<<<grid_for(N * h->I, 256, h->sm_count), 256, 0, st>>>(
            x, x32, N * h->I, h->x_scale, xo.zero_point, op_qmin(xo), op_qmax(xo));
        k_init_state<<<grid_for((long long)B * h->Hpad, 256, h->sm_count), 256, 0, st>>>(
            nullptr, h0, nullptr, (int32_t *)h->hq32.p, nullptr, nullptr, B, h->H, h->Hpad, init_slot, h->h_scale,
            ho.zero_point, op_qmin(ho), op_qmax(ho), h->d_flags);
        h->launches += 2;
        if ((rc = run_generic(h, T, B, x32, (int32_t *)h->hq32.p, nullptr, flags, st))) return rc;
        k_dequantize<<<grid_for((long long)nh, 256, h->sm_count), 256, 0, st>>>(
            (const int32_t *)h->hq32.p, h_out, (long long)nh, h->h_scale, ho.zero_point);
        h->launches++;
        CK(cudaGetLastError());
        return QGRU_OK;
    }
    if ((rc = ensure(h, h->x8, (size_t)((N + 127) / 128 * 128) * h->Ipad))) return rc;
    if ((rc = ensure(h, h->h8, (size_t)(2 * B + 256) * h->Hpad))) return rc;
    k_quantize_rows_f32<<<grid_for(N * (h->Ipad / 4), 256, h->sm_count), 256, 0, st>>>(
        x, (uint8_t *)h->x8.p, x_q_out, N, h->I, h->Ipad, h->x_scale, xo.zero_point, op_qmin(xo), op_qmax(xo));
    CK(cudaMemsetAsync(h->h8.p, 0, (size_t)(2 * B + 256) * h->Hpad, st));
    k_init_state<<<grid_for((long long)B * h->Hpad, 256, h->sm_count), 256, 0, st>>>(
        nullptr, h0, (uint8_t *)h->h8.p, nullptr, h_out, nullptr, B, h->H, h->Hpad, init_slot, h->h_scale,
        ho.zero_point, op_qmin(ho), op_qmax(ho), h->d_flags);
    h->launches += 2;
    CK(cudaGetLastError());
    return run_fast(h, T, B, nullptr, h_out, flags, st);
}

int qgru_forward_f32_q8(qgru_handle *h, int T, int B, const float *x, const float *h0, uint8_t *h_q8,
                        unsigned flags, void *stream) {
    if (!h || !x || !h_q8) return QGRU_ERR_BAD_ARG;
    int rc = check_forward_args(h, T, B);
    if (rc) return rc;
    if (use_generic(h))
        return fail(h, QGRU_ERR_UNSUPPORTED, "the 8-bit output needs the 8-bit storage plan (x, h, W, R at most 8 bits)");
    CK(cudaSetDevice(h->device));
    cudaStream_t st = (cudaStream_t)stream;
    const long long N = (long long)T * B;
    const qgru_op &xo = h->p.op[QGRU_OP_X], &ho = h->p.op[QGRU_OP_H];
    const long long init_slot = (flags & QGRU_FLAG_REVERSE) ? T : 0;
    h->ev = h->ring[h->calls % qgru_handle::kRing];
    h->calls++;
    CK(cudaEventRecord(h->ev[0], st));
    CK(cudaMemsetAsync(h->d_flags, 0, 2 * sizeof(int), st));
    if ((rc = ensure(h, h->x8, (size_t)((N + 127) / 128 * 128) * h->Ipad))) return rc;
    if ((rc = ensure(h, h->h8, (size_t)(2 * B + 256) * h->Hpad))) return rc;
    k_quantize_rows_f32<<<grid_for(N * (h->Ipad / 4), 256, h->sm_count), 256, 0, st>>>(
        x, (uint8_t *)h->x8.p, nullptr, N, h->I, h->Ipad, h->x_scale, xo.zero_point, op_qmin(xo), op_qmax(xo));
    CK(cudaMemsetAsync(h->h8.p, 0, (size_t)(2 * B + 256) * h->Hpad, st));
    k_init_state<<<grid_for((long long)B * h->Hpad, 256, h->sm_count), 256, 0, st>>>(
        nullptr, h0, (uint8_t *)h->h8.p, nullptr, nullptr, h_q8, B, h->H, h->Hpad, init_slot, h->h_scale,
        ho.zero_point, op_qmin(ho), op_qmax(ho), h->d_flags);
    h->launches += 2;
    CK(cudaGetLastError());
    return run_fast(h, T, B, nullptr, nullptr, flags, st, h_q8);
}

int qgru_synchronize(qgru_handle *h, void *stream) {
    if (!h) return QGRU_ERR_BAD_ARG;
    CK(cudaSetDevice(h->device));
    cudaStream_t st = (cudaStream_t)stream;
    CK(cudaMemcpyAsync(h->h_flags, h->d_flags, 2 * sizeof(int), cudaMemcpyDeviceToHost, st));
    CK(cudaStreamSynchronize(st));
    CK(cudaGetLastError());
    if (h->h_flags[1]) return fail(h, QGRU_ERR_TIMEOUT, "a per-step barrier wait of the recurrence kernel ran out");
    if (h->h_flags[0] & 1) return fail(h, QGRU_ERR_BAD_ARG, "quantized input outside the range its operator declares");
    return QGRU_OK;
}

int qgru_forward_i32_host(qgru_handle *h, int T, int B, const int32_t *x_q, const int32_t *h0_q,
                          int32_t *h_q, unsigned flags, void *stream) {
    if (!h || !x_q || !h_q) return QGRU_ERR_BAD_ARG;
    int rc = check_forward_args(h, T, B);
    if (rc) return rc;
    CK(cudaSetDevice(h->device));
    cudaStream_t st = (cudaStream_t)stream;
    const size_t nx = (size_t)T * B * h->I * 4, nh = (size_t)(T + 1) * B * h->H * 4, n0 = (size_t)B * h->H * 4;
    if ((rc = ensure(h, h->stage_in, nx))) return rc;
    if ((rc = ensure(h, h->stage_out, nh))) return rc;
    if (h0_q && (rc = ensure(h, h->stage_h0, n0))) return rc;
    CK(cudaMemcpyAsync(h->stage_in.p, x_q, nx, cudaMemcpyHostToDevice, st));
    if (h0_q) CK(cudaMemcpyAsync(h->stage_h0.p, h0_q, n0, cudaMemcpyHostToDevice, st));
    if ((rc = qgru_forward_i32(h, T, B, (const int32_t *)h->stage_in.p,
                               h0_q ? (const int32_t *)h->stage_h0.p : nullptr,
                               (int32_t *)h->stage_out.p, flags, stream)))
        return rc;
    CK(cudaMemcpyAsync(h_q, h->stage_out.p, nh, cudaMemcpyDeviceToHost, st));
    return qgru_synchronize(h, stream);
}

int qgru_forward_f32_host(qgru_handle *h, int T, int B, const float *x, const float *h0,
                          float *h_out, unsigned flags, void *stream) {
    if (!h || !x || !h_out) return QGRU_ERR_BAD_ARG;
    int rc = check_forward_args(h, T, B);
    if (rc) return rc;
    CK(cudaSetDevice(h->device));
    cudaStream_t st = (cudaStream_t)stream;
    const size_t nx = (size_t)T * B * h->I * 4, nh = (size_t)(T + 1) * B * h->H * 4, n0 = (size_t)B * h->H * 4;
    if ((rc = ensure(h, h->stage_in, nx))) return rc;
    if ((rc = ensure(h, h->stage_out, nh))) return rc;
    if (h0 && (rc = ensure(h, h->stage_h0, n0))) return rc;
    CK(cudaMemcpyAsync(h->stage_in.p, x, nx, cudaMemcpyHostToDevice, st));
    if (h0) CK(cudaMemcpyAsync(h->stage_h0.p, h0, n0, cudaMemcpyHostToDevice, st));
    if ((rc = qgru_forward_f32(h, T, B, (const float *)h->stage_in.p,
                               h0 ? (const float *)h->stage_h0.p : nullptr, (float *)h->stage_out.p,
                               nullptr, flags, stream)))
        return rc;
    CK(cudaMemcpyAsync(h_out, h->stage_out.p, nh, cudaMemcpyDeviceToHost, st));
    return qgru_synchronize(h, stream);
}

int qgru_last_timing(qgru_handle *h, float *ms_input_gemm, float *ms_recurrence, float *ms_total) {
    if (!h) return QGRU_ERR_BAD_ARG;
    if (!h->timing_valid) return fail(h, QGRU_ERR_NOT_READY, "no forward has run");
    CK(cudaSetDevice(h->device));
    CK(cudaEventSynchronize(h->ev[3]));
    float a = 0, b = 0, c = 0;
    CK(cudaEventElapsedTime(&a, h->ev[1], h->ev[2]));
    CK(cudaEventElapsedTime(&b, h->ev[2], h->ev[3]));
    CK(cudaEventElapsedTime(&c, h->ev[0], h->ev[3]));
    if (ms_input_gemm) *ms_input_gemm = a;
    if (ms_recurrence) *ms_recurrence = b;
    if (ms_total) *ms_total = c;
    return QGRU_OK;
}

int qgru_timing_window(qgru_handle *h, int *n_calls, float *ms_input_gemm, float *ms_recurrence,
                       float *ms_total) {
    if (!h || !n_calls) return QGRU_ERR_BAD_ARG;
    if (!h->timing_valid) return fail(h, QGRU_ERR_NOT_READY, "no forward has run");
    CK(cudaSetDevice(h->device));
    int n = std::min<long long>(std::min<long long>(*n_calls, qgru_handle::kRing), (long long)h->calls);
    float sa = 0, sb = 0, sc = 0;
    for (int k = 0; k < n; ++k) {
        cudaEvent_t *e = h->ring[(h->calls - 1 - k) % qgru_handle::kRing];
        CK(cudaEventSynchronize(e[3]));
        float a = 0, b = 0, c = 0;
        CK(cudaEventElapsedTime(&a, e[1], e[2]));
        CK(cudaEventElapsedTime(&b, e[2], e[3]));
        CK(cudaEventElapsedTime(&c, e[0], e[3]));
        sa += a; sb += b; sc += c;
    }
    *n_calls = n;
    if (ms_input_gemm) *ms_input_gemm = sa;
    if (ms_recurrence) *ms_recurrence = sb;
    if (ms_total) *ms_total = sc;
    return QGRU_OK;
}

const char *qgru_describe_plan(qgru_handle *h, int T, int B) {
    (void)T;
    (void)B;
    if (!h) return "null handle";
    return h->plan_text.c_str();
}

}  // extern "C"

// ------------------------------------------------------------------------------------------
// Forward without any allocation.
//
// Some callers are not allowed to allocate device memory when they call a forward: a serving
// loop whose memory budget was fixed at start-up, a process whose allocator is owned by another
// framework, code running between the capture and the replay of a CUDA graph, or a real-time
// thread for which cudaMalloc's implicit device synchronisation is not acceptable.  For them
// the workspace of the integer forward (8-bit input rows, the W*x+bw buffer, the ping-pong
// state and the per-group step counters) lives in the array below, which is part of the
// library image: every GPU that loads the library holds these bytes until the process exits.
// ------------------------------------------------------------------------------------------
namespace {

constexpr size_t kStaticWorkspaceBytes = size_t(8) << 20;   // 8 MiB per device
static __device__ __align__(256) unsigned char g_static_workspace[kStaticWorkspaceBytes];

constexpr int kMaxDevices = 64;
std::mutex g_static_mu;
unsigned char *g_static_ptr[kMaxDevices] = {};   // device address of the array, per device

// In host code `g_static_workspace` is only a handle for the runtime, not an address a kernel
// can use: the device address is asked for once per device, with that device current.
int static_workspace(qgru_handle *h, unsigned char **out) {
    if (h->device < 0 || h->device >= kMaxDevices) return fail(h, QGRU_ERR_UNSUPPORTED, "device index too large");
    std::lock_guard<std::mutex> lock(g_static_mu);
    if (!g_static_ptr[h->device]) {
        void *p = nullptr;
        const cudaError_t e = cudaGetSymbolAddress(&p, g_static_workspace);
        if (e != cudaSuccess || !p) {
            h->err = std::string("cudaGetSymbolAddress(static workspace): ") + cudaGetErrorString(e);
            cudaGetLastError();
            return QGRU_ERR_CUDA;
        }
        g_static_ptr[h->device] = static_cast<unsigned char *>(p);
    }
    *out = g_static_ptr[h->device];
    return QGRU_OK;
}

size_t align256(size_t v) { return (v + 255) & ~size_t(255); }

}  // namespace

extern "C" int qgru_forward_i32_static(qgru_handle *h, int T, int B, const int32_t *x_q, const int32_t *h0_q,
                                       int32_t *h_q, unsigned flags, void *stream) {
    if (!h || !x_q || !h_q) return QGRU_ERR_BAD_ARG;
    int rc = check_forward_args(h, T, B);
    if (rc) return rc;
    if (!h->fast) return fail(h, QGRU_ERR_UNSUPPORTED, "the static-workspace forward needs the 8-bit storage plan");
    CK(cudaSetDevice(h->device));
    cudaStream_t st = (cudaStream_t)stream;
    const long long N = (long long)T * B;
    const int C = h->C;

    RecPlan pl;
    if (!plan_recurrence(h, B, &pl)) return fail(h, QGRU_ERR_UNSUPPORTED, "no recurrence plan fits shared memory");
    // carve the array: x8 | ih | h8 (two state buffers) | step counters
    const size_t off_x8 = 0;
    const size_t off_ih = align256(off_x8 + (size_t)N * h->Ipad);
    const size_t off_h8 = align256(off_ih + (size_t)N * C * h->ih_bytes);
    const size_t off_bar = align256(off_h8 + (size_t)2 * B * h->Hpad);
    const size_t need = off_bar + (size_t)pl.G * 32 * sizeof(unsigned);
    if (need > kStaticWorkspaceBytes) {
        char msg[200];
        snprintf(msg, sizeof(msg), "static workspace too small: T=%d B=%d needs %zu bytes, the library holds %zu",
                 T, B, need, kStaticWorkspaceBytes);
        return fail(h, QGRU_ERR_BAD_ARG, msg);
    }
    unsigned char *ws = nullptr;
    if ((rc = static_workspace(h, &ws))) return rc;
    uint8_t *x8 = ws + off_x8;
    void *ih = ws + off_ih;
    uint8_t *h8 = ws + off_h8;
    unsigned *bar = reinterpret_cast<unsigned *>(ws + off_bar);

    const qgru_op &xo = h->p.op[QGRU_OP_X], &ho = h->p.op[QGRU_OP_H];
    const long long init_slot = (flags & QGRU_FLAG_REVERSE) ? T : 0;
    h->ev = h->ring[h->calls % qgru_handle::kRing];
    h->calls++;
    CK(cudaEventRecord(h->ev[0], st));
    CK(cudaMemsetAsync(h->d_flags, 0, 2 * sizeof(int), st));
    // the array keeps what the previous call left: the state buffers' padding columns and the
    // step counters must start at zero
    CK(cudaMemsetAsync(h8, 0, (size_t)2 * B * h->Hpad, st));
    CK(cudaMemsetAsync(bar, 0, (size_t)pl.G * 32 * sizeof(unsigned), st));
    k_narrow_rows_i32<<<grid_for(N * (h->Ipad / 4), 256, h->sm_count), 256, 0, st>>>(
        x_q, x8, N, h->I, h->Ipad, op_qmin(xo), op_qmax(xo), h->d_flags);
    k_init_state<<<grid_for((long long)B * h->Hpad, 256, h->sm_count), 256, 0, st>>>(
        h0_q, nullptr, h8, h_q, nullptr, nullptr, B, h->H, h->Hpad, init_slot, h->h_scale, ho.zero_point, op_qmin(ho),
        op_qmax(ho), h->d_flags);
    CK(cudaEventRecord(h->ev[1], st));
    const LinearConsts lcx = linear_consts(h, 0);
    {
        dim3 grid((unsigned)((N + 63) / 64), (unsigned)((C + 63) / 64));
        if (h->ih_bytes == 1) {
            if (h->x_uns) k_gemm_wx_simt<true, int8_t><<<grid, 256, 0, st>>>(x8, h->d_w8[0], (int8_t *)ih, N, C, h->Ipad, lcx);
            else k_gemm_wx_simt<false, int8_t><<<grid, 256, 0, st>>>(x8, h->d_w8[0], (int8_t *)ih, N, C, h->Ipad, lcx);
        } else {
            if (h->x_uns) k_gemm_wx_simt<true, int16_t><<<grid, 256, 0, st>>>(x8, h->d_w8[0], (int16_t *)ih, N, C, h->Ipad, lcx);
            else k_gemm_wx_simt<false, int16_t><<<grid, 256, 0, st>>>(x8, h->d_w8[0], (int16_t *)ih, N, C, h->Ipad, lcx);
        }
    }
    CK(cudaGetLastError());
    CK(cudaEventRecord(h->ev[2], st));
    RecArgs a;
    a.T = T; a.B = B; a.H = h->H; a.Hpad = h->Hpad; a.C = C;
    a.Hs = pl.Hs; a.Bt = pl.Bt; a.P = pl.P;
    a.reverse = (flags & QGRU_FLAG_REVERSE) ? 1 : 0;
    a.r8 = h->d_w8[1];
    a.ih = ih;
    a.h8 = h8;
    a.hq_out = h_q;
    a.hf_out = nullptr;
    a.lc = linear_consts(h, 1);
    a.gc = h->d_gc;
    a.tables = h->d_tables;
    a.n_table = h->n_table;
    a.bar = bar;
    a.abort_flag = h->d_flags + 1;
    a.spin_limit = h->spin_limit;
    if (h->ih_bytes == 1) rc = h->h_uns ? launch_rec<true, int8_t>(h, a, pl, st) : launch_rec<false, int8_t>(h, a, pl, st);
    else rc = h->h_uns ? launch_rec<true, int16_t>(h, a, pl, st) : launch_rec<false, int16_t>(h, a, pl, st);
    if (rc) return rc;
    h->launches += 3;
    CK(cudaEventRecord(h->ev[3], st));
    h->timing_valid = true;
    h->plan_text = "path=int8 gemm=simt_dp4a rec=dp4a workspace=static";
    return QGRU_OK;
}

#include "qgru_fstorage.cuh"
#include "qgru_train.cuh"
