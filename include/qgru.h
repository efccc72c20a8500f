/*
 * qgru.h - C ABI of the B200-native integer quantized GRU forward.
 *
 * This is the boundary a maintainer of CX9898/quant-gru-pytorch binds in place of the
 * library's own `ForwardPassQuant` machinery: plain pointers, sizes and status codes,
 * no C++ or torch types.  Each entry point names the reference interface it replaces
 * (paths are relative to the reference project's root).
 *
 * Conventions shared by every entry point
 *   - Layouts are the reference's "haste" layouts: W [I,3H], R [H,3H], bw/br [3H],
 *     gate order along 3H is (update z, reset r, new n); x [T,B,I]; h [(T+1),B,H] with the
 *     initial state in slot 0 (include/gru_interface.h:389-413).
 *   - Quantized tensors crossing the boundary are int32 containers whose values are
 *     already clamped to the operator's bit width, exactly as in the reference.
 *   - `stream` is a cudaStream_t passed as void*; NULL means the legacy default stream.
 *     Calls are asynchronous with respect to the host unless stated otherwise.
 *   - Every function returns a qgru_status; no exception crosses this boundary.
 *   - Nothing here falls back to a CPU path: without a CUDA device the device entry
 *     points return QGRU_ERR_CUDA.
 */
#ifndef QGRU_H_
#define QGRU_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(_WIN32)
#define QGRU_API
#else
#define QGRU_API __attribute__((visibility("default")))
#endif

/* ------------------------------------------------------------------ status */
typedef enum qgru_status {
    QGRU_OK = 0,
    QGRU_ERR_BAD_ARG = 1,      /* null pointer, non-positive size, mismatched shape   */
    QGRU_ERR_CUDA = 2,         /* a CUDA runtime/driver call failed (see last_error)   */
    QGRU_ERR_TIMEOUT = 3,      /* a bounded device-side wait ran out                   */
    QGRU_ERR_UNSUPPORTED = 4,  /* bit width / shape outside what the kernels implement */
    QGRU_ERR_NOT_READY = 5,    /* params or weights were not set before a forward      */
    QGRU_ERR_NOMEM = 6,        /* device or host allocation failed                     */
    QGRU_ERR_RANGE = 7         /* a scale cannot be encoded (<=0, shift outside int8)  */
} qgru_status;

/* ------------------------------------------------------------- data model */

/* Operator order of `qgru_params.op[]`.  One entry per quantized operator of
 * include/quantize_param_types.h:100-146 (GRUQuantParams) and
 * include/quantize_bitwidth_config.h:68-75 (OperatorQuantConfig). */
enum {
    QGRU_OP_X = 0,
    QGRU_OP_H = 1,
    QGRU_OP_W = 2,   /* per-channel scales live in the scale_W array  */
    QGRU_OP_R = 3,
    QGRU_OP_BW = 4,
    QGRU_OP_BR = 5,
    QGRU_OP_IH_LINEAR = 6,  /* weight_ih_linear = W*x + bw */
    QGRU_OP_HH_LINEAR = 7,  /* weight_hh_linear = R*h + br */
    QGRU_OP_UPDATE_IN = 8,
    QGRU_OP_UPDATE_OUT = 9,
    QGRU_OP_RESET_IN = 10,
    QGRU_OP_RESET_OUT = 11,
    QGRU_OP_NEW_IN = 12,
    QGRU_OP_NEW_OUT = 13,
    QGRU_OP_MUL_RESET_HIDDEN = 14,   /* calibrated and exported, unused by the datapath */
    QGRU_OP_MUL_NEW_CONTRIB = 15,    /* idem */
    QGRU_OP_MUL_OLD_CONTRIB = 16,    /* idem */
    QGRU_NUM_OPS = 17
};

enum { QGRU_PER_TENSOR = 0, QGRU_PER_GATE = 1, QGRU_PER_CHANNEL = 2 };
enum { QGRU_LUT_UPDATE = 0, QGRU_LUT_RESET = 1, QGRU_LUT_NEW = 2 };
#define QGRU_LUT_SEGMENTS 16

/* QuantParam + QuantBitWidth + symmetric flag of one operator
 * (include/quantize_param_types.h:63-66, include/quantize_bitwidth_config.h:6-22). */
typedef struct qgru_op {
    float scale;          /* authoritative scale: continuous (M+shift mode) or 2^-n (POT2) */
    int32_t zero_point;
    int8_t bits;          /* 1..32 */
    uint8_t is_unsigned;
    uint8_t symmetric;
    uint8_t reserved;
} qgru_op;

/* One SegmentParams (include/quantize_lut_types.h:31-36). */
typedef struct qgru_lut_segment {
    int32_t q_b;
    int32_t n_bx;        /* reference stores int8; widened, same value */
    int32_t term_c;
    int32_t threshold;
} qgru_lut_segment;

/* The part of SigmoidLUT the datapath reads (include/quantize_lut_types.h:47-55). */
typedef struct qgru_lut {
    qgru_lut_segment seg[QGRU_LUT_SEGMENTS];
    int32_t zp_x;
    int32_t reserved[3];
} qgru_lut;

/* Everything of GRUQuantParams except the four per-channel scale arrays. */
typedef struct qgru_params {
    int32_t hidden;
    int32_t use_pot2;                 /* OperatorQuantConfig::usePOT2_ */
    qgru_op op[QGRU_NUM_OPS];
    int32_t granularity[4];           /* W, R, bw, br: QGRU_PER_* (informational) */
    qgru_lut lut[3];                  /* update, reset, new */
} qgru_params;

/* GRUQuantizationRanges (include/gru_quantization_ranges.h:20-71) as a POD.
 * Scalars are indexed by the QGRU_OP_* ids (W/R/BW/BR slots unused); per-channel
 * ranges are caller-owned arrays of 3H floats. */
typedef struct qgru_ranges {
    int32_t hidden;
    int32_t reserved;
    float min_v[QGRU_NUM_OPS];
    float max_v[QGRU_NUM_OPS];
    float *min_W, *max_W, *min_R, *max_R, *min_bw, *max_bw, *min_br, *max_br; /* [3H] host */
} qgru_ranges;

typedef struct qgru_handle qgru_handle;

/* ----------------------------------------------------------- host helpers */
/* Pure host functions: no CUDA call is made, they work without a GPU. */

QGRU_API const char *qgru_status_string(int status);
QGRU_API const char *qgru_version(void);

/* encodeMShift (include/quantize_ops_helper.h:245-264): scale ~= M * 2^-shift, M in
 * [32768, 65535].  Returns QGRU_ERR_RANGE where the reference throws. */
QGRU_API int qgru_encode_mshift(float scale, uint16_t *multiplier, int8_t *shift);

/* decode_effective_scale of the reference's binding (pytorch/lib/gru_interface_binding.cc:
 * 1285-1296): the scale the kernels really apply for a stored scale - multiplier * 2^-shift of
 * its 16-bit fixed-point encoding, or 2^-shift in POT2 mode.  QGRU_ERR_BAD_ARG for scale <= 0. */
QGRU_API int qgru_decode_effective_scale(float scale, int use_pot2, float *effective);

/* rshift_round(int64) (include/quantize_ops_helper.h:183-206). */
QGRU_API int64_t qgru_rshift_round(int64_t x, int n);

/* applyRescale (include/quantize_ops_helper.h:228-230) for a 32-bit operand, computed by the
 * very routine the kernels use: rshift_round(x * multiplier, shift), through the shift-free
 * form (one 32x32->64 multiply by the left-aligned multiplier, rounding on the high word) for
 * shifts 17..48 (2..33 when multiplier is 1), else through 64-bit shifts. */
QGRU_API int32_t qgru_apply_rescale(int32_t x, uint16_t multiplier, int shift);
/* No counterpart in the reference.  Can x * multiplier / 2^shift be an exact tie (remainder
 * exactly one half) for some integer x in [lo, hi]?  Where it cannot, rounding half up gives what
 * the reference's round-half-even gives, and the kernels drop the tie rule (option "tie_rule").
 * qgru_apply_rescale_half_up is that cheaper rounding, through the kernels' shift-free form. */
QGRU_API int qgru_rescale_can_tie(uint16_t multiplier, int shift, int64_t lo, int64_t hi);
QGRU_API int32_t qgru_apply_rescale_half_up(int32_t x, uint16_t multiplier, int shift);

/* Evaluate one LUT the way piecewise_linear does (include/quantize_ops_helper.h:600-606). */
QGRU_API int32_t qgru_lut_eval(const qgru_lut *lut, int32_t q_x, const qgru_op *in_bw,
                               const qgru_op *out_bw);

/* generate_piecewise_linear_lut_to_params (src/quantize_ops.cu:21-52): fills p->lut[0..2]
 * from the six gate input/output operators of p. */
QGRU_API int qgru_generate_luts(qgru_params *p);

/* calculateGRUQuantitativeParameters (src/gru_interface.cc:51-158), MinMax path:
 * ranges + bit-width config (the bits/is_unsigned/symmetric/granularity/use_pot2 fields
 * of `p`) -> scales, zero points and LUTs.  scale_* are host arrays of 3H floats. */
QGRU_API int qgru_calc_params_from_ranges(const qgru_ranges *ranges, qgru_params *p,
                                          float *scale_W, float *scale_R, float *scale_bw,
                                          float *scale_br);

/* --------------------------------------------------------------- lifecycle */

/* One handle per (device, direction).  Replaces the per-call construction of
 * gru::ForwardPassQuant (src/gru_forward_gpu_quant.cu:412-442): streams, events and the
 * workspace live as long as the handle and grow on demand. */
QGRU_API int qgru_create(qgru_handle **out, int device, int input_size, int hidden_size);
QGRU_API void qgru_destroy(qgru_handle *h);
QGRU_API const char *qgru_last_error(const qgru_handle *h);

/* ForwardPassQuant::setRescaleParam (src/gru_forward_gpu_quant.cu:672-748): derives every
 * execution-time rescale from the (scale, zero_point) seeds and uploads the tables.
 * Host pointers.  Must precede set_weights and forward. */
QGRU_API int qgru_set_params(qgru_handle *h, const qgru_params *p, const float *scale_W,
                             const float *scale_R, const float *scale_bw,
                             const float *scale_br);

/* quantitativeWeight<false> (src/gru_interface.cc:294-328): per-channel quantize of the
 * float master weights (device pointers) and packing into the kernels' layout.  The
 * packed copy is kept until the next set_weights/set_params call. */
QGRU_API int qgru_set_weights_f32(qgru_handle *h, const float *W, const float *R,
                                  const float *bw, const float *br, void *stream);

/* Same, for weights that are already quantized (the W_q/R_q/bw_q/br_q arguments of
 * quantGRUForwardInt32, include/gru_interface.h:389). Device pointers. */
QGRU_API int qgru_set_weights_i32(qgru_handle *h, const int32_t *W_q, const int32_t *R_q,
                                  const int32_t *bw_q, const int32_t *br_q, void *stream);

/* Copy the quantized weights out as int32 containers (the W_q_out..br_q_out outputs of
 * quantGRUForwardInt, include/gru_interface.h:266-299).  Any pointer may be NULL. */
QGRU_API int qgru_get_weights_i32(qgru_handle *h, int32_t *W_q, int32_t *R_q, int32_t *bw_q,
                                  int32_t *br_q, void *stream);

/* ----------------------------------------------------------------- forward */

#define QGRU_FLAG_REVERSE 1u /* consume x and produce h in reversed time order */

/* quantGRUForwardInt32 (src/gru_interface.cc:551-603), inference mode.
 *   x_q  [T,B,I] int32 device, h0_q [B,H] int32 device or NULL (-> zero point of h),
 *   h_q  [(T+1),B,H] int32 device out.
 * With QGRU_FLAG_REVERSE timestep s of the recurrence reads x_q[T-1-s] and writes
 * h_q[T-1-s]; slot T holds the initial state, slots 0..T-1 the outputs in input time order
 * and slot 0 is h_n.  This equals the reference's
 * flip -> forward -> flip for the reverse direction (pytorch/quant_gru.py:2143-2158)
 * without the two copies. */
QGRU_API int qgru_forward_i32(qgru_handle *h, int T, int B, const int32_t *x_q,
                              const int32_t *h0_q, int32_t *h_q, unsigned flags, void *stream);

/* quantGRUForwardInt32 with is_training = true and v_q given (src/gru_interface.cc:551-603;
 * buffer written at src/gru_forward_gpu_quant.cu:318-330, src/gru_forward_cpu_quant.cc:199-205):
 * the same h_q plus v_q [T,B,4H] int32 device out = quantized update, reset and new gate outputs
 * and the R*h + br row of the new gate, per timestep of x (with QGRU_FLAG_REVERSE, slot t of
 * v_q belongs to x_q[t]).  Runs on the step-by-step int32 kernels, which keep those
 * intermediates.
 * masks (may be NULL, and so may each member): the five clamp masks of the reference's training
 * mode (include/gru_interface.h:380-402; src/gru_forward_gpu_quant.cu:168-178, :318-348), uint8
 * device out, 1 = the value was inside its range before the clamp (the backward pass keeps the
 * gradient), 0 = it was clamped; rows are indexed like v_q (row t*B + b belongs to x_q[t]). */
typedef struct qgru_masks {
    uint8_t *ih_linear;   /* [T*B, 3H] W*x + bw */
    uint8_t *hh_linear;   /* [T*B, 3H] R*h + br */
    uint8_t *gate_input;  /* [T*B, 3H] gate inputs (z, r, n) */
    uint8_t *gate_output; /* [T*B, 3H] gate outputs (z, r, n) */
    uint8_t *h;           /* [T*B, H]  new state */
} qgru_masks;
QGRU_API int qgru_forward_i32_train(qgru_handle *h, int T, int B, const int32_t *x_q,
                                    const int32_t *h0_q, int32_t *h_q, int32_t *v_q,
                                    const qgru_masks *masks, unsigned flags, void *stream);

/* quantGRUForwardFP (src/gru_interface.cc:894-995, src/gru_forward_gpu_quant_fp.cu), inference
 * mode: the float-storage quantized forward that QuantGRU.forward runs by default and that QAT
 * trains against.  Tensors hold quantized values, the requantization between operators is
 * float arithmetic (round(x * scale_ratio)) and the gates are the real sigmoid / tanh of the
 * dequantized gate inputs, not the piecewise-linear tables.  x [T,B,I], h0 [B,H] or NULL,
 * h_out [(T+1),B,H] (dequantized, slot layout as qgru_forward_i32), x_q_out [T,B,I] or NULL
 * (the quantized input as floats): device fp32.  Needs 8-bit W, R, x and h (else
 * QGRU_ERR_UNSUPPORTED); weights as set by qgru_set_weights_f32 / _i32.  The matrix products
 * are exact integer sums; the reference's are fp32 sums of the same integers, exact below
 * 2^24, and every float operation after them is the reference's, in its order. */
QGRU_API int qgru_forward_fstorage(qgru_handle *h, int T, int B, const float *x, const float *h0,
                                   float *h_out, float *x_q_out, unsigned flags, void *stream);

/* quantGRUForwardFP with is_training = true: the float-storage forward that also returns what
 * the masked backward needs.  v_out [T,B,4H]: dequantized update, reset and new gate outputs and
 * R*h + br row of the new gate.  masks (may be NULL, and so may each member): uint8 device out,
 * 1 = not clamped; the six input masks x [T*B,I], h0 [B,H], W [I,3H], R [H,3H], bw, br [3H]
 * (W..br: the float master weights, device, needed only for these four) and the five
 * computation masks of qgru_masks.  Runs on exact int32 sums and a per-step kernel (two launches
 * per step); h_out equals qgru_forward_fstorage's. */
typedef struct qgru_train_masks {
    uint8_t *x, *h0, *W, *R, *bw, *br;
    uint8_t *ih_linear, *hh_linear, *gate_input, *gate_output, *h;
} qgru_train_masks;
QGRU_API int qgru_forward_fstorage_train(qgru_handle *h, int T, int B, const float *W, const float *R,
                                         const float *bw, const float *br, const float *x, const float *h0,
                                         float *h_out, float *v_out, float *x_q_out,
                                         const qgru_train_masks *masks, unsigned flags, void *stream);

/* quantGRUForwardInt with is_training = true (src/gru_interface.cc:610-725): the integer forward
 * with float interface that also returns what the masked backward needs.  Same arguments as
 * qgru_forward_fstorage_train, except x_q_out [T,B,I] int32 (may be NULL); v_out holds the
 * dequantized gate buffer of the integer path (piecewise-linear gates).  Runs on the
 * step-by-step int32 kernels. */
QGRU_API int qgru_forward_f32_train(qgru_handle *h, int T, int B, const float *W, const float *R,
                                    const float *bw, const float *br, const float *x, const float *h0,
                                    float *h_out, float *v_out, int32_t *x_q_out,
                                    const qgru_train_masks *masks, unsigned flags, void *stream);

/* dequantizeGRUWeights (include/gru_interface.h:141): the quantized weights the handle holds,
 * times their per-channel scales, as device fp32 (W [I,3H], R [H,3H], bw, br [3H]; NULL = skip).
 * These are the weights the masked backward differentiates through. */
QGRU_API int qgru_get_weights_dequantized(qgru_handle *h, float *W, float *R, float *bw, float *br,
                                          void *stream);
/* dequantize_f (include/quantize_ops_helper.h:510-512) for operator `op` (QGRU_OP_*) of the
 * handle's parameters on n float-stored quantized values: out = (q - zero_point) * scale. */
QGRU_API int qgru_dequantize_f32(qgru_handle *h, int op, const float *q, float *out, long long n,
                                 void *stream);

/* hasteGRUBackward (src/gru_interface.cc:215-240) and quantGRUBackward (:246-290): backward pass
 * through T steps from the forward's saved h [(T+1),B,H] and v [T,B,4H] (float mode:
 * qgru_forward_float's v; quantized training: the dequantized training buffer).  All device fp32.
 * In: W_t [3H,I], R_t [3H,H], x_t [I,T*B] (the transposes, as the reference takes them),
 * dh_new [(T+1),B,H] (gradient of every output state; slot 0 unused).  In/out, accumulated like
 * the reference does: dW [I,3H], dR [H,3H], dbw [3H], dbr [3H] (+=), dh [B,H] (in: gradient
 * arriving at the last state from outside the sequence, normally zeros; out: gradient of h0).
 * Out: dx [T*B,I].  masks: NULL for the float backward; else the straight-through masks of
 * the quantized training forward (1 = gradient kept, 0 = the forward clamped there), each
 * member may be NULL: x [T*B,I], h0 [B,H], W [I,3H], R [H,3H], bw [3H], br [3H], and the five
 * masks of qgru_masks. */
typedef struct qgru_bwd_masks {
    const uint8_t *x, *h0, *W, *R, *bw, *br;
    const uint8_t *ih_linear, *hh_linear, *gate_input, *gate_output, *h;
} qgru_bwd_masks;
QGRU_API int qgru_backward(qgru_handle *h, int T, int B, const float *W_t, const float *R_t,
                           const float *x_t, const float *dh_new, const float *h_all, const float *v,
                           float *dx, float *dW, float *dR, float *dbw, float *dbr, float *dh,
                           const qgru_bwd_masks *masks, void *stream);

/* quantGRUForwardInt (src/gru_interface.cc:610-725), inference mode: float in, float out.
 *   x [T,B,I] f32 device, h0 [B,H] f32 device or NULL, h [(T+1),B,H] f32 device out,
 *   x_q_out [T,B,I] int32 device or NULL. */
QGRU_API int qgru_forward_f32(qgru_handle *h, int T, int B, const float *x, const float *h0,
                              float *h_out, int32_t *x_q_out, unsigned flags, void *stream);

/* No counterpart in the reference (its outputs are fp32 or int32 containers).  qgru_forward_f32
 * with the output left in its native width: h_q8 [(T+1),B,H] holds the quantized states as 8-bit
 * values (int8, or uint8 when the h operator is unsigned; slot layout as qgru_forward_i32), a
 * quarter of the fp32 output's bytes for a caller whose link to the result is the bottleneck
 * (a host behind PCIe).  The caller dequantizes with (q - zero_point) * scale of the h operator
 * (scale as qgru_decode_effective_scale gives it): exactly the value qgru_forward_f32 writes.
 * Needs the 8-bit storage plan (else QGRU_ERR_UNSUPPORTED). */
QGRU_API int qgru_forward_f32_q8(qgru_handle *h, int T, int B, const float *x, const float *h0,
                                 uint8_t *h_q8, unsigned flags, void *stream);

/* No counterpart in the reference.  The same result as qgru_forward_i32 for callers that must
 * not allocate device memory at call time (a serving loop with a fixed memory budget, a process
 * whose allocator belongs to another framework, a real-time thread that cannot tolerate the
 * implicit synchronisation of cudaMalloc).  The whole workspace is a fixed array of 8 MiB inside
 * the library image - every GPU that loads the library holds it until the process exits - so the
 * call makes no cudaMalloc / cudaFree and grows nothing.  Problems whose workspace
 * (a256(T*B*Kpad(I)) + a256(T*B*3H*b) + a256(2*B*Kpad(H)) + 128*G bytes; Kpad rounds up to 128,
 * a256 to 256, b = 1 or 2 bytes per W*x+bw value, G = batch groups of the recurrence, at most the
 * SM count) does not fit
 * are rejected with QGRU_ERR_BAD_ARG and a message naming both sizes.  It needs the 8-bit
 * storage plan (x, h, W, R at most 8 bits) and runs the SIMT GEMM and the dp4a recurrence.
 * The first call on a device looks up the array's device address (cudaGetSymbolAddress); make
 * that first call before any stream capture.  All handles and calls on one GPU share the array
 * and it keeps the previous call's contents (what must start at zero is cleared by the call
 * itself), so two calls that overlap on the GPU - different streams or handles - race: serialise
 * them. */
QGRU_API int qgru_forward_i32_static(qgru_handle *h, int T, int B, const int32_t *x_q,
                                     const int32_t *h0_q, int32_t *h_q, unsigned flags,
                                     void *stream);

/* The same two calls for callers that hold HOST buffers (pinned or pageable): the library
 * stages x to the device, runs the forward and copies h back, all on `stream`; returns
 * after the stream has been synchronised. */
QGRU_API int qgru_forward_i32_host(qgru_handle *h, int T, int B, const int32_t *x_q,
                                   const int32_t *h0_q, int32_t *h_q, unsigned flags,
                                   void *stream);
QGRU_API int qgru_forward_f32_host(qgru_handle *h, int T, int B, const float *x,
                                   const float *h0, float *h_out, unsigned flags,
                                   void *stream);

/* Blocks until the work queued on `stream` by this handle is done and reports a device-side
 * bounded-wait expiry (QGRU_ERR_TIMEOUT) or CUDA error, as the reference's
 * cudaDeviceSynchronize + cudaGetLastError + throw does (src/gru_interface.cc:594-602).
 * The device-side status words belong to the handle and every forward clears them when it starts:
 * the call reports on the LAST forward queued before it.  A caller that queues several forwards
 * on one handle without synchronising in between learns the status of the last one only; call
 * this after each forward whose status matters (the host-buffer entry points do). */
QGRU_API int qgru_synchronize(qgru_handle *h, void *stream);

/* Timing of the two kernels of the most recent forward, measured with CUDA events on the
 * launching stream (milliseconds; synchronises).  Any pointer may be NULL. */
QGRU_API int qgru_last_timing(qgru_handle *h, float *ms_input_gemm, float *ms_recurrence,
                              float *ms_total);

/* Sums of the same three durations over the last `n_calls` forwards of this handle (at most
 * 64 are remembered), so a benchmark can queue steps back to back and read per-kernel time
 * afterwards.  *n_calls returns how many calls were summed.  Synchronises. */
QGRU_API int qgru_timing_window(qgru_handle *h, int *n_calls, float *ms_input_gemm,
                                float *ms_recurrence, float *ms_total);

/* Number of kernels launched by this handle since creation. */
QGRU_API uint64_t qgru_launch_count(const qgru_handle *h);

/* Which implementation the next forward will use, as a short human-readable string
 * ("gemm=tcgen05_i8 rec=mma ..."), for benchmarks and tests. */
QGRU_API const char *qgru_describe_plan(qgru_handle *h, int T, int B);

/* No counterpart in the reference (it has no tensor-core code).  Measurement aid: runs `mmas` (a multiple of 8)
 * back-to-back tcgen05.mma kind::i8 instructions of shape M x N x 32 (M 128 with N a multiple of
 * 16, or M 64 with N a multiple of 8; N <= 256) on `ctas` CTAs, one per SM, operands resident in
 * shared memory (or A in tensor memory), rotating over `accumulators` accumulators; no loads, no
 * epilogue.  Returns the SM clock cycles one MMA takes in that chain (slowest CTA) and the
 * aggregate rate in 1e12 int8 operations per second (2*M*N*32 per MMA, CUDA-event time).  The
 * large-N figure is the measured peak of the int8 tensor pipe that benchmark lines quote the
 * W*x GEMM against; the small-N figures are the cost model of the recurrence kernels. */
QGRU_API int qgru_probe_mma_i8(int device, int M, int N, int a_in_tmem, int accumulators, int mmas,
                               int ctas, double *cycles_per_mma, double *tera_ops);
/* The same with `issuers` (1..4) warps issuing `mmas` MMAs each into accumulators of their own, and
 * `spinners` further warps beside them that (neighbour_mode 0) poll an mbarrier as a kernel's waiting
 * warps do, (1) run integer arithmetic back to back or (2) run dependent shared-memory loads, as its
 * busy warps do, (3) drain accumulators with 16-column tensor-memory loads or (4) write 128-bit words
 * into shared memory, (6) follow the first issuer's periodic commits with suspending barrier waits,
 * as an epilogue follows its accumulator barrier, (7) stream global memory (read, add, write back):
 * cycles_per_mma is the slowest issuer's chain time divided by `mmas`, tera_ops
 * counts all issuers.  neighbour_mode + 1024 (N <= 128): every MMA of a pass of eight reads operand
 * tiles of its own, spread over 128 KB of shared memory, as a GEMM that streams its operands does
 * (without it the four K steps of one tile pair repeat); + 512: all 32 lanes of an issuing warp stay
 * in the loop and an elected lane issues.  neighbour_mode + 256 fills the shared-memory operands with pseudo-random bytes
 * instead of zeros: same instruction stream, the multipliers toggle as in a real product, which
 * shows what part of the zero-operand peak survives the board's power limit. */
QGRU_API int qgru_probe_mma_i8_ex(int device, int M, int N, int a_in_tmem, int accumulators, int mmas,
                                  int ctas, int issuers, int spinners, int neighbour_mode,
                                  double *cycles_per_mma, double *tera_ops);
/* The same with a tcgen05.commit after every `commit_every` (0, 4 or 8) MMAs of each issuer, as a GEMM
 * main loop commits to hand its operand stages back. */
QGRU_API int qgru_probe_mma_i8_commits(int device, int M, int N, int a_in_tmem, int accumulators, int mmas,
                                       int ctas, int issuers, int spinners, int neighbour_mode,
                                       int commit_every, double *cycles_per_mma, double *tera_ops);

/* neighbour_mode 5 of the probes above: the first neighbour warp keeps four 16 KB bulk copies from
 * global memory into shared memory in flight, as a GEMM's operand loads do.  This returns the bytes
 * per SM clock that the copies of CTA 0 moved during the last such probe of this process. */
QGRU_API double qgru_probe_last_bulk_rate(void);

/* Restrict or force kernel choices (testing).  Names and values:
 *   "gemm"     auto | simt | tcgen05        W*x kernel
 *   "gemm_order" auto | stream | w_stationary  tile order of the tcgen05 W*x kernel: W and x slabs
 *                                           stream per tile (auto), or a CTA keeps one slice of W
 *                                           in tensor memory for the whole launch (slower; kept
 *                                           as a measured alternative)
 *   "gemv_r"   auto | smem                  one-CTA-per-row recurrence: R held in registers for all
 *                                           steps (auto, tabulated cell, H <= 256) or in shared memory
 *   "t_chunk"  auto | 0 | N                 cluster recurrence: W*x+bw is computed and consumed N
 *                                           timesteps at a time (two chunk buffers instead of the
 *                                           whole sequence; the next chunk's GEMM runs on a second
 *                                           stream beside this chunk's recurrence).  0: one chunk;
 *                                           auto: eight chunks where the recurrence leaves half of
 *                                           the SMs free and T >= 256
 *   "rec"      auto | dp4a | mma | generic  recurrence kernel (generic = int32 storage path)
 *   "exchange" auto | global | cluster      how the CTAs of a batch group exchange h_t
 *   "cell"     auto | fused | generic       gate datapath: tabulated (auto also allows its
 *                                           shift-free form), or the reference's step by step
 *   "r_resident" auto | smem | tmem       where the cluster recurrence keeps its slice of R
 *   "tiles_per_cta" 1 | 2                 cluster recurrence at 128 < H <= 256: 128-unit tiles per CTA
 *   "subgroups" auto | 1 | 2              cluster recurrence: independent batch sub-groups per CTA (with 2,
 *                                         the MMAs of one overlap the cells of the other)
 *   "tie_rule" auto | always              auto: kernels round half up where the library has proved that no value
 *                                         in range is an exact tie (same result as round-half-even, fewer
 *                                         instructions); always: every rescale applies the tie rule
 *   "k_parts" 1 | 2                       cluster recurrence: 1 = one MMA-issuing warp per gate, 2 = one per K half
 *   "issue_delay" n                       cluster recurrence: SM cycles by which the reset gate's MMAs start after
 *                                         the update gate's, and the new gate's after the reset gate's
 *   "unit_tile" auto | 64 | 128           cluster recurrence: hidden units per CTA (auto = 128; 64: update and
 *                                         reset rows share one MMA tile, H <= 512, tabulated cell only)
 *   "probe_floor" 0 | 1                   measurement aid: the cluster recurrence runs with its MMAs and
 *                                         cells left out (results are meaningless); the recurrence time of
 *                                         qgru_last_timing is then the per-step synchronisation floor
 *   "sm_limit" n   use at most n SMs (0 = all);  "spin_limit" n   bound of the group barrier
 *   "test_withhold_arrive" 0 | 1          failure-path test: with the dp4a recurrence on several CTAs per group,
 *                                         CTA 0 leaves out one arrival, the group's bounded wait runs out and the
 *                                         forward reports QGRU_ERR_TIMEOUT; nothing faults or hangs
 * Unknown names or values return QGRU_ERR_BAD_ARG. */
QGRU_API int qgru_set_option(qgru_handle *h, const char *name, const char *value);

/* ------------------------------------------------------- float mode / calibration */

/* hasteGRUForward (src/gru_interface.cc:173-207): unquantized fp32 GRU.
 *   h [(T+1),B,H] f32 out; v [T,B,4H] f32 out or NULL (z, r, n, Rh_n+br_n as the
 *   reference's training buffer). */
QGRU_API int qgru_forward_float(qgru_handle *h, int T, int B, const float *W, const float *R,
                                const float *bw, const float *br, const float *x,
                                const float *h0, float *h_out, float *v_out, void *stream);

/* forwardWithCalibrationGPU, MinMax branch (src/gru_interface.cc:1283-1372 with
 * updateGRUQuantizationRangesGPU, src/calibration_gpu.cu:1847-1953): float forward, then
 * fold the batch's min/max of every operator into `ranges` (host, in/out).  Synchronous.
 *   h_out [(T+1),B,H] f32 device or NULL. */
QGRU_API int qgru_calibrate_minmax(qgru_handle *h, int T, int B, const float *W,
                                   const float *R, const float *bw, const float *br,
                                   const float *x, const float *h0, qgru_ranges *ranges,
                                   float *h_out, void *stream);

/* ---- histogram calibration (Percentile / SQNR) ----
 * A qgru_hist holds one 2048-bin (or fewer) histogram with range growth per operator, as
 * GRUGPUHistogramCollectors does (include/histogram_gpu.cuh; collectors of
 * src/calibration_gpu.cu:820-1039).  Index space:
 *   QGRU_OP_* ids           the 13 activation operators; QGRU_OP_W/R/BW/BR: per-tensor weights
 *   QGRU_HIST_GATE0 + 3*k+g per-gate weight histograms (k: 0 W, 1 R, 2 bw, 3 br; g: z, r, n)
 *   QGRU_HIST_CHANNEL0 + k*3H + c   per-channel weight histograms
 * Counts live on the device; ranges and totals on the host. */
typedef struct qgru_hist qgru_hist;
#define QGRU_HIST_GATE0 17
#define QGRU_HIST_CHANNEL0 29

QGRU_API int qgru_hist_create(qgru_hist **out, int device, int hidden_size, int num_bins);
QGRU_API void qgru_hist_destroy(qgru_hist *hs);
QGRU_API int qgru_hist_reset(qgru_hist *hs);
QGRU_API int qgru_hist_count(const qgru_hist *hs);
QGRU_API const char *qgru_hist_last_error(const qgru_hist *hs);

/* GPUHistogramCollector::collect (src/calibration_gpu.cu:820-876) for one collector: fold n
 * device floats into histogram `index` (first call fixes the range, later calls grow it and
 * redistribute the old counts).  Synchronous. */
QGRU_API int qgru_hist_collect(qgru_hist *hs, int index, const float *data, long long n,
                               void *stream);

/* Copy one histogram out (counts: host array of num_bins floats, may be NULL) or in. */
QGRU_API int qgru_hist_export(const qgru_hist *hs, int index, float *counts, float *min_val,
                              float *max_val, int64_t *total_count);
QGRU_API int qgru_hist_import(qgru_hist *hs, int index, const float *counts, float min_val,
                              float max_val, int64_t total_count);

/* forwardWithCalibrationGPU, histogram branch (src/gru_interface.cc:1283-1372 with
 * collectAllHistogramsGPU, src/histogram_calibration_utils.cu:18-123): float forward of one
 * batch, then every operator's values are folded into `hs`.  granularity[4]: QGRU_PER_* of
 * W, R, bw, br (per-channel weight histograms are built once).  Synchronous. */
QGRU_API int qgru_calibrate_hist(qgru_handle *h, qgru_hist *hs, int T, int B, const float *W,
                                 const float *R, const float *bw, const float *br,
                                 const float *x, const float *h0, const int32_t *granularity,
                                 void *stream);

/* calculateGRUQuantitativeParametersFromHistograms (src/gru_interface.cc:1079-1153):
 * histograms + bit-width config (fields of `p` as for qgru_calc_params_from_ranges) ->
 * scales, zero points and LUTs, by Percentile (use_percentile != 0; percentile e.g. 99.99)
 * or by the SQNR search (calibrateSqnr, include/pot_sqnr_calibrator.h:246-381). */
QGRU_API int qgru_calc_params_from_hist(const qgru_hist *hs, int use_percentile, float percentile,
                                        qgru_params *p, float *scale_W, float *scale_R,
                                        float *scale_bw, float *scale_br);

/* The same derivation for one histogram given as host arrays (pure host function):
 * calibrateContinuousScaleFromHistogram + encodeScaleResult
 * (include/pot_sqnr_calibrator.h:526-544, 451-524).  In: op->bits / is_unsigned / symmetric;
 * out: op->scale, op->zero_point. */
QGRU_API int qgru_calibrate_from_histogram(const float *counts, int num_bins, float min_val,
                                           float max_val, int64_t total_count, int use_pot2,
                                           int use_percentile, float percentile, qgru_op *op);

/* Initialise a qgru_ranges to "empty" (min=+FLT_MAX, max=-FLT_MAX), as
 * GRUQuantizationRanges::reset does (include/gru_quantization_ranges.h:75-123). */
QGRU_API void qgru_ranges_reset(qgru_ranges *r, int hidden);

#ifdef __cplusplus
}
#endif
#endif /* QGRU_H_ */
