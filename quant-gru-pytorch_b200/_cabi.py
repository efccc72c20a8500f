"""ctypes view of include/qgru.h and loader of libqgru_b200.so.

There is no CPU fallback: if the shared library has not been built, ``lib()`` raises.
"""
import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libqgru_b200.so")

QGRU_OK, QGRU_ERR_BAD_ARG, QGRU_ERR_CUDA, QGRU_ERR_TIMEOUT = 0, 1, 2, 3
QGRU_ERR_UNSUPPORTED, QGRU_ERR_NOT_READY, QGRU_ERR_NOMEM, QGRU_ERR_RANGE = 4, 5, 6, 7

OPS = ["x", "h", "W", "R", "bw", "br", "weight_ih_linear", "weight_hh_linear",
       "update_gate_input", "update_gate_output", "reset_gate_input", "reset_gate_output",
       "new_gate_input", "new_gate_output", "mul_reset_hidden", "mul_new_contribution",
       "mul_old_contribution"]
OP_INDEX = {n: i for i, n in enumerate(OPS)}
NUM_OPS = 17
PER_TENSOR, PER_GATE, PER_CHANNEL = 0, 1, 2
FLAG_REVERSE = 1


class Op(C.Structure):
    _fields_ = [("scale", C.c_float), ("zero_point", C.c_int32), ("bits", C.c_int8),
                ("is_unsigned", C.c_uint8), ("symmetric", C.c_uint8), ("reserved", C.c_uint8)]


class LutSegment(C.Structure):
    _fields_ = [("q_b", C.c_int32), ("n_bx", C.c_int32), ("term_c", C.c_int32),
                ("threshold", C.c_int32)]


class Lut(C.Structure):
    _fields_ = [("seg", LutSegment * 16), ("zp_x", C.c_int32), ("reserved", C.c_int32 * 3)]


class Params(C.Structure):
    _fields_ = [("hidden", C.c_int32), ("use_pot2", C.c_int32), ("op", Op * NUM_OPS),
                ("granularity", C.c_int32 * 4), ("lut", Lut * 3)]


class Masks(C.Structure):
    """qgru_masks: the five clamp masks of the training-mode integer forward (device pointers)."""
    _fields_ = [("ih_linear", C.c_void_p), ("hh_linear", C.c_void_p), ("gate_input", C.c_void_p),
                ("gate_output", C.c_void_p), ("h", C.c_void_p)]


class BwdMasks(C.Structure):
    """qgru_bwd_masks: straight-through masks of the quantized backward (device pointers, 0 = absent)."""
    _fields_ = [(n, C.c_void_p) for n in ("x", "h0", "W", "R", "bw", "br", "ih_linear", "hh_linear",
                                          "gate_input", "gate_output", "h")]


class Ranges(C.Structure):
    _fields_ = [("hidden", C.c_int32), ("reserved", C.c_int32),
                ("min_v", C.c_float * NUM_OPS), ("max_v", C.c_float * NUM_OPS),
                ("min_W", C.POINTER(C.c_float)), ("max_W", C.POINTER(C.c_float)),
                ("min_R", C.POINTER(C.c_float)), ("max_R", C.POINTER(C.c_float)),
                ("min_bw", C.POINTER(C.c_float)), ("max_bw", C.POINTER(C.c_float)),
                ("min_br", C.POINTER(C.c_float)), ("max_br", C.POINTER(C.c_float))]


# every symbol include/qgru.h declares: name -> (restype, argtypes)
_P = C.c_void_p
_F = C.POINTER(C.c_float)
SYMBOLS = {
    "qgru_status_string": (C.c_char_p, [C.c_int]),
    "qgru_version": (C.c_char_p, []),
    "qgru_decode_effective_scale": (C.c_int, [C.c_float, C.c_int, C.POINTER(C.c_float)]),
    "qgru_encode_mshift": (C.c_int, [C.c_float, C.POINTER(C.c_uint16), C.POINTER(C.c_int8)]),
    "qgru_rshift_round": (C.c_int64, [C.c_int64, C.c_int]),
    "qgru_apply_rescale": (C.c_int32, [C.c_int32, C.c_uint16, C.c_int]),
    "qgru_rescale_can_tie": (C.c_int, [C.c_uint16, C.c_int, C.c_int64, C.c_int64]),
    "qgru_apply_rescale_half_up": (C.c_int32, [C.c_int32, C.c_uint16, C.c_int]),
    "qgru_lut_eval": (C.c_int32, [C.POINTER(Lut), C.c_int32, C.POINTER(Op), C.POINTER(Op)]),
    "qgru_generate_luts": (C.c_int, [C.POINTER(Params)]),
    "qgru_calc_params_from_ranges": (C.c_int, [C.POINTER(Ranges), C.POINTER(Params), _F, _F, _F, _F]),
    "qgru_create": (C.c_int, [C.POINTER(_P), C.c_int, C.c_int, C.c_int]),
    "qgru_destroy": (None, [_P]),
    "qgru_last_error": (C.c_char_p, [_P]),
    "qgru_set_params": (C.c_int, [_P, C.POINTER(Params), _F, _F, _F, _F]),
    "qgru_set_weights_f32": (C.c_int, [_P, _P, _P, _P, _P, _P]),
    "qgru_set_weights_i32": (C.c_int, [_P, _P, _P, _P, _P, _P]),
    "qgru_get_weights_i32": (C.c_int, [_P, _P, _P, _P, _P, _P]),
    "qgru_forward_i32": (C.c_int, [_P, C.c_int, C.c_int, _P, _P, _P, C.c_uint, _P]),
    "qgru_forward_f32_train": (C.c_int, [_P, C.c_int, C.c_int] + [_P] * 10 + [C.c_uint, _P]),
    "qgru_forward_fstorage_train": (C.c_int, [_P, C.c_int, C.c_int] + [_P] * 10 + [C.c_uint, _P]),
    "qgru_get_weights_dequantized": (C.c_int, [_P] * 6),
    "qgru_dequantize_f32": (C.c_int, [_P, C.c_int, _P, _P, C.c_longlong, _P]),
    "qgru_backward": (C.c_int, [_P, C.c_int, C.c_int] + [_P] * 14),
    "qgru_forward_fstorage": (C.c_int, [_P, C.c_int, C.c_int, _P, _P, _P, _P, C.c_uint, _P]),
    "qgru_forward_i32_train": (C.c_int, [_P, C.c_int, C.c_int, _P, _P, _P, _P, _P, C.c_uint, _P]),
    "qgru_forward_i32_static": (C.c_int, [_P, C.c_int, C.c_int, _P, _P, _P, C.c_uint, _P]),
    "qgru_forward_f32": (C.c_int, [_P, C.c_int, C.c_int, _P, _P, _P, _P, C.c_uint, _P]),
    "qgru_forward_f32_q8": (C.c_int, [_P, C.c_int, C.c_int, _P, _P, _P, C.c_uint, _P]),
    "qgru_forward_i32_host": (C.c_int, [_P, C.c_int, C.c_int, _P, _P, _P, C.c_uint, _P]),
    "qgru_forward_f32_host": (C.c_int, [_P, C.c_int, C.c_int, _P, _P, _P, C.c_uint, _P]),
    "qgru_synchronize": (C.c_int, [_P, _P]),
    "qgru_last_timing": (C.c_int, [_P, _F, _F, _F]),
    "qgru_timing_window": (C.c_int, [_P, C.POINTER(C.c_int), _F, _F, _F]),
    "qgru_launch_count": (C.c_uint64, [_P]),
    "qgru_describe_plan": (C.c_char_p, [_P, C.c_int, C.c_int]),
    "qgru_set_option": (C.c_int, [_P, C.c_char_p, C.c_char_p]),
    "qgru_probe_mma_i8": (C.c_int, [C.c_int] * 7 + [C.POINTER(C.c_double), C.POINTER(C.c_double)]),
    "qgru_probe_mma_i8_commits": (C.c_int, [C.c_int] * 11 + [C.POINTER(C.c_double), C.POINTER(C.c_double)]),
    "qgru_probe_last_bulk_rate": (C.c_double, []),
    "qgru_probe_mma_i8_ex": (C.c_int, [C.c_int] * 10 + [C.POINTER(C.c_double), C.POINTER(C.c_double)]),
    "qgru_forward_float": (C.c_int, [_P, C.c_int, C.c_int, _P, _P, _P, _P, _P, _P, _P, _P, _P]),
    "qgru_calibrate_minmax": (C.c_int, [_P, C.c_int, C.c_int, _P, _P, _P, _P, _P, _P,
                                        C.POINTER(Ranges), _P, _P]),
    "qgru_ranges_reset": (None, [C.POINTER(Ranges), C.c_int]),
    "qgru_hist_create": (C.c_int, [C.POINTER(_P), C.c_int, C.c_int, C.c_int]),
    "qgru_hist_destroy": (None, [_P]),
    "qgru_hist_reset": (C.c_int, [_P]),
    "qgru_hist_count": (C.c_int, [_P]),
    "qgru_hist_last_error": (C.c_char_p, [_P]),
    "qgru_hist_collect": (C.c_int, [_P, C.c_int, _P, C.c_longlong, _P]),
    "qgru_hist_export": (C.c_int, [_P, C.c_int, _F, _F, _F, C.POINTER(C.c_int64)]),
    "qgru_hist_import": (C.c_int, [_P, C.c_int, _F, C.c_float, C.c_float, C.c_int64]),
    "qgru_calibrate_hist": (C.c_int, [_P, _P, C.c_int, C.c_int, _P, _P, _P, _P, _P, _P,
                                      C.POINTER(C.c_int32), _P]),
    "qgru_calc_params_from_hist": (C.c_int, [_P, C.c_int, C.c_float, C.POINTER(Params), _F, _F, _F, _F]),
    "qgru_calibrate_from_histogram": (C.c_int, [_F, C.c_int, C.c_float, C.c_float, C.c_int64, C.c_int,
                                                C.c_int, C.c_float, C.POINTER(Op)]),
}
HIST_GATE0 = 17
HIST_CHANNEL0 = 29

_lib = None


def lib():
    """Load libqgru_b200.so once; raise if it is missing (no fallback exists)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with __graft_entry__.build() "
                "(nvcc, sm_100a). There is no CPU or PyTorch fallback for this path.")
        L = C.CDLL(LIB_PATH)
        for name, (res, args) in SYMBOLS.items():
            fn = getattr(L, name)
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


class QgruError(RuntimeError):
    """A C-ABI call returned a status other than QGRU_OK."""

    def __init__(self, status, where, detail=""):
        self.status = status
        msg = lib().qgru_status_string(status).decode()
        super().__init__(f"{where}: {msg}" + (f" ({detail})" if detail else ""))


def check(status, where, handle=None):
    if status != QGRU_OK:
        detail = lib().qgru_last_error(handle).decode() if handle else ""
        if status in (QGRU_ERR_BAD_ARG,):
            raise ValueError(f"{where}: {detail or 'bad argument'}")
        raise QgruError(status, where, detail)
