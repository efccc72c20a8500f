// qgru_rec_mma.cuh - plan and launch interface of the tensor-core recurrence kernel
// (qgru_rec_mma.cu).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include <algorithm>
#include <string>

#include "qgru_internal.h"

namespace qgru {

struct RecMmaArgs {
    int T, B, H, Hpad, C;
    int P;            // CTAs per group (slices of the hidden dimension); set by the launcher
    int NB;           // batch rows per group (multiple of 16); set by the launcher
    int NG = 1;       // cluster kernel: independent sub-groups of NB rows per CTA
    int k_parts = 1;  // cluster kernels: K halves with an issuing warp and accumulators of their own
    int issue_delay = 0;   // cluster kernel: head start (cycles) of the update gate's MMAs over the reset gate's, and of those over the new gate's
    int b_off, b_cnt; // batch rows [b_off, b_off + b_cnt) are handled by this launch
    int reverse;
    int h_unsigned;   // the state h is stored as uint8 (else int8)
    uint32_t tmem_cols;
    int r_tmem_col;   // first tensor-memory column of the R tiles kept there
    int tmem_tiles;   // cluster kernel: R tiles [0, tmem_tiles) live in tensor memory, the rest in shared memory
    int r_slots;      // cluster kernel: 16 KB shared-memory tile slots for R
    const void *ih;         // [T*B][3H]: raw W*x+bw (int8/int16) or pre-rescaled for the fused cell (int16/int32)
    uint8_t *h8;            // [2][B][Hpad] ping-pong state (+ slack rows)
    int32_t *hq_out;        // [(T+1)][B][H] or null
    float *hf_out;          // [(T+1)][B][H] or null
    uint8_t *h8_out = nullptr;   // [(T+1)][B][H] or null: the quantized state in its 8-bit container
    int write_final = 0;    // cluster kernel: the last step also writes its state to h8 (rows [B][Hpad]), where the
                            // launch over the next chunk of timesteps picks it up as its initial state
    LinearConsts lc;        // R*h + br epilogue
    const int32_t *tables;  // activation tables (table_off) or, fused, the fused-cell tables (ft_off)
    int n_table;
    unsigned *bar;          // one counter per group, 32 words apart, zeroed before the launch
    int *abort_flag;
    unsigned spin_limit;
#ifdef QGRU_STAMPS
    long long *dbg = nullptr;   // development builds only: [T][2 sub-groups][8] clock stamps of CTA 0
#endif
    // float-storage forward (cluster kernel, generic-cell instantiation only): the float cell of
    // the reference's quantGRUForwardFP instead of the integer one
    int fs_on = 0;
    const float *fs_chan = nullptr;   // [3][C]: offset, bias term, scale ratio of R*h + br per channel
    FsConsts fs{};
};

struct RecMmaPlan {
    int MT = 1, P = 1, NB = 16, NG = 1, G = 1, tmem_cols = 32, groups_per_launch = 1;
    int r_tmem_col = 0, tmem_tiles = 0, r_slots = 0, k_parts = 1;
    size_t smem = 0;
};

struct RecMmaState {
    bool valid = false;
    const void *r8 = nullptr, *h8 = nullptr;
    long long r_rows = 0, h_rows = 0;
    int Hpad = 0, NB = 0;
    unsigned long long launches = 0;
    alignas(64) unsigned char map_r[128];
    alignas(64) unsigned char map_h[128];
};

// False when the shape cannot use this kernel (the slice of R for 128 hidden units must fit
// one SM's shared memory: H <= 512 with 8-bit weights).
bool rec_mma_plan(int H, int Hpad, int B, int sms, int smem_optin, int n_table, RecMmaPlan *out);

int rec_mma_launch(RecMmaState &s, const RecMmaPlan &pl, RecMmaArgs a, const GateConsts &gc_host,
                   const int8_t *r8, long long r_rows_alloc,
                   long long h_rows_alloc, bool h_unsigned, int ih_bytes, bool narrow, bool fused, bool have_coop,
                   cudaStream_t stream, std::string *err);

// The same kernel with the P CTAs of a group as one thread-block cluster exchanging h_t through
// distributed shared memory (qgru_rec_cluster.cu).  Same plan fields; no cooperative launch.
bool rec_cluster_plan(int H, int Hpad, int B, int sms, int smem_optin, int n_table, int r_where,
                      int mt_opt, int ng_opt, int kp_opt, RecMmaPlan *out);

int rec_cluster_launch(RecMmaState &s, const RecMmaPlan &pl, RecMmaArgs a, const GateConsts &gc_host,
                       const int8_t *r8, long long r_rows_alloc, long long h_rows_alloc, bool h_unsigned,
                       int ih_bytes, bool narrow, bool fused, bool floor, bool notie, cudaStream_t stream,
                       std::string *err);

// The cluster kernel's low-latency form: 64 hidden units per CTA, two sub-groups, the branch-free
// tabulated cell only (qgru_rec_c64.cu).  The plan fails where it does not apply (H > 512, or - unless
// `force` - where a cluster would hold more than 64 rows or fewer than 3 CTAs).
bool rec_c64_plan(int H, int Hpad, int B, int sms, int smem_optin, int n_table, bool force, RecMmaPlan *out);

int rec_c64_launch(RecMmaState &s, const RecMmaPlan &pl, RecMmaArgs a, const GateConsts &gc_host, const int8_t *r8,
                   long long r_rows_alloc, long long h_rows_alloc, bool h_unsigned, int ih_bytes, bool notie,
                   cudaStream_t stream, std::string *err);

}  // namespace qgru
