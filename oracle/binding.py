"""TEST INFRASTRUCTURE: ctypes bindings of the two checkers.

``Oracle``    libqgru_oracle.so - the plain-C restatement (oracle/qgru_oracle.c)
``Reference`` _ref/libqgru_ref.so - the unmodified reference sources + oracle/ref_shim.cc

Both expose the same method names so a test can run either.  Only tests/, the smoke test and
the CPU-baseline leg of bench.py may import this module; the product never does.
"""
import ctypes as C
import os
import subprocess
import sys

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_ROOT = os.path.dirname(_HERE)
# the reference project's tree: QGRU_REF_ROOT, else a checkout named "reference" beside this repository
REF_ROOT = os.environ.get("QGRU_REF_ROOT") or os.path.join(os.path.dirname(_ROOT), "reference")


def _pkg():
    sys.path.insert(0, _ROOT) if _ROOT not in sys.path else None
    from __graft_entry__ import load_package
    return load_package()


def _f(a):
    return a.ctypes.data_as(C.POINTER(C.c_float))


def _i(a):
    return a.ctypes.data_as(C.POINTER(C.c_int32))


def build_oracle():
    so = os.path.join(_HERE, "libqgru_oracle.so")
    src = os.path.join(_HERE, "qgru_oracle.c")
    if not os.path.exists(so) or os.path.getmtime(so) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE, "oracle"], check=True, capture_output=True)
    return so


def build_ref():
    """Compile the reference where it lies; returns None if the tree is absent (GPU box)."""
    so = os.path.join(_HERE, "_ref", "libqgru_ref.so")
    if os.path.isdir(os.path.join(REF_ROOT, "src")):
        subprocess.run(["make", "-C", _HERE, "-j8", "ref", "REF_ROOT=" + REF_ROOT], check=True,
                       capture_output=True)
        # the reference-signature binding of the product library and its test driver
        subprocess.run(["make", "-C", _HERE, "shimtest", "REF_ROOT=" + REF_ROOT], check=True,
                       capture_output=True)
    return so if os.path.exists(so) else None


class _Checker:
    prefix = ""

    def __init__(self, path):
        self.cabi = _pkg()._cabi
        self.lib = C.CDLL(path)
        # getattr caches the function object (CDLL.__getitem__ would make a new one per use)
        self._fn("rshift_round").restype = C.c_int64
        self._fn("rshift_round").argtypes = [C.c_int64, C.c_int]
        self._fn("lut_eval").restype = C.c_int32

    def _fn(self, name):
        return getattr(self.lib, self.prefix + name)

    def rshift_round(self, x, n):
        return int(self._fn("rshift_round")(int(x), int(n)))

    def encode_mshift(self, scale):
        m, s = C.c_uint16(), C.c_int8()
        rc = self._fn("encode_mshift")(C.c_float(scale), C.byref(m), C.byref(s))
        return None if rc else (m.value, s.value)

    def lut_eval(self, lut, q, in_op, out_op):
        return int(self._fn("lut_eval")(C.byref(lut), C.c_int32(int(q)), C.byref(in_op), C.byref(out_op)))

    def generate_luts(self, params):
        rc = self._fn("generate_luts")(C.byref(params))
        if rc:
            raise RuntimeError("generate_luts failed")

    def calc_params_from_ranges(self, ranges, params):
        """ranges: params.Ranges-like object with .struct(); returns the 4 scale arrays."""
        Cn = 3 * ranges.hidden
        sc = [np.zeros(Cn, np.float32) for _ in range(4)]
        rs = ranges.struct()
        rc = self._fn("calc_params_from_ranges")(C.byref(rs), C.byref(params), *[_f(a) for a in sc])
        if rc:
            raise RuntimeError("calc_params_from_ranges failed")
        return sc

    def quantize_weights(self, I, H, W, R, bw, br, params, sc):
        Cn = 3 * H
        out = [np.zeros((I, Cn), np.int32), np.zeros((H, Cn), np.int32), np.zeros(Cn, np.int32),
               np.zeros(Cn, np.int32)]
        rc = self._fn("quantize_weights")(I, H, _f(W), _f(R), _f(bw), _f(br), C.byref(params),
                                          *[_f(a) for a in sc], *[_i(a) for a in out])
        if rc:
            raise RuntimeError("quantize_weights failed")
        return out

    def quantize(self, x, params, op):
        x = np.ascontiguousarray(x, np.float32)
        out = np.zeros(x.shape, np.int32)
        rc = self._fn("quantize")(_f(x), _i(out), C.c_size_t(x.size), C.byref(params), int(op))
        if rc:
            raise RuntimeError("quantize failed")
        return out

    def dequantize(self, q, params, op):
        q = np.ascontiguousarray(q, np.int32)
        out = np.zeros(q.shape, np.float32)
        rc = self._fn("dequantize")(_i(q), _f(out), C.c_size_t(q.size), C.byref(params), int(op))
        if rc:
            raise RuntimeError("dequantize failed")
        return out

    def calibrate_from_histogram(self, counts, min_val, max_val, total, op, pot2, use_percentile,
                                 percentile=99.99):
        """One histogram -> (scale, zero_point) for the operator described by `op` (bits,
        is_unsigned, symmetric); None where the checker reports a failure."""
        counts = np.ascontiguousarray(counts, np.float32)
        o = self.cabi.Op(0.0, 0, op.bits, op.is_unsigned, op.symmetric, 0)
        rc = self._fn("calibrate_from_histogram")(
            _f(counts), int(counts.size), C.c_float(min_val), C.c_float(max_val), C.c_int64(int(total)),
            int(bool(pot2)), int(bool(use_percentile)), C.c_float(percentile), C.byref(o))
        return None if rc else (float(np.float32(o.scale)), int(o.zero_point))

    def hist_new(self, bins=2048):
        f = self._fn("hist_new")
        f.restype = C.c_void_p
        return _Hist(self, C.c_void_p(f(int(bins))), bins)

    def forward_i32(self, T, B, I, H, wq, x_q, h0_q, params, sc, threads=1):
        x_q = np.ascontiguousarray(x_q, np.int32)
        h = np.zeros((T + 1, B, H), np.int32)
        h0p = _i(np.ascontiguousarray(h0_q, np.int32)) if h0_q is not None else None
        args = [T, B, I, H, *[_i(np.ascontiguousarray(a, np.int32)) for a in wq], _i(x_q), h0p,
                C.byref(params), *[_f(a) for a in sc], _i(h)]
        if threads > 1:
            rc = self._fn("forward_i32_mt")(*args, int(threads))
        else:
            rc = self._fn("forward_i32")(*args)
        if rc:
            raise RuntimeError("forward_i32 failed")
        return h

    def forward_i32_v(self, T, B, I, H, wq, x_q, h0_q, params, sc):
        """Training-mode forward: (h_q [(T+1),B,H], v_q [T,B,4H])."""
        x_q = np.ascontiguousarray(x_q, np.int32)
        h = np.zeros((T + 1, B, H), np.int32)
        v = np.zeros((T, B, 4 * H), np.int32)
        h0p = _i(np.ascontiguousarray(h0_q, np.int32)) if h0_q is not None else None
        rc = self._fn("forward_i32_v")(T, B, I, H, *[_i(np.ascontiguousarray(w, np.int32)) for w in wq], _i(x_q),
                                       h0p, C.byref(params), *[_f(s) for s in sc], _i(h), _i(v))
        if rc:
            raise RuntimeError("forward_i32_v failed")
        return h, v

    def forward_i32_train(self, T, B, I, H, wq, x_q, h0_q, params, sc):
        """Training-mode forward with the five clamp masks (oracle only: the reference's CPU path
        has none): (h_q, v_q, [ih, hh, gate_in, gate_out (each [T*B,3H]), h [T*B,H]] uint8)."""
        x_q = np.ascontiguousarray(x_q, np.int32)
        h = np.zeros((T + 1, B, H), np.int32)
        v = np.zeros((T, B, 4 * H), np.int32)
        ms = [np.zeros((T * B, 3 * H), np.uint8) for _ in range(4)] + [np.zeros((T * B, H), np.uint8)]
        mptr = (C.c_void_p * 5)(*[m.ctypes.data for m in ms])
        h0p = _i(np.ascontiguousarray(h0_q, np.int32)) if h0_q is not None else None
        rc = self._fn("forward_i32_train")(T, B, I, H, *[_i(np.ascontiguousarray(w, np.int32)) for w in wq],
                                           _i(x_q), h0p, C.byref(params), *[_f(s) for s in sc], _i(h), _i(v),
                                           mptr)
        if rc:
            raise RuntimeError("forward_i32_train failed")
        return h, v, ms

    def forward_f32(self, T, B, I, H, wq, x, h0, params, sc):
        x = np.ascontiguousarray(x, np.float32)
        h = np.zeros((T + 1, B, H), np.float32)
        h0p = _f(np.ascontiguousarray(h0, np.float32)) if h0 is not None else None
        rc = self._fn("forward_f32")(T, B, I, H, *[_i(np.ascontiguousarray(a, np.int32)) for a in wq],
                                     _f(x), h0p, C.byref(params), *[_f(a) for a in sc], _f(h))
        if rc:
            raise RuntimeError("forward_f32 failed")
        return h


class _Hist:
    """One histogram collector of a checker (oracle: the GPU collector's rules on the CPU;
    reference: its CPU HistogramCollector)."""

    def __init__(self, chk, handle, bins):
        self.chk, self.h, self.bins = chk, handle, bins

    def collect(self, data):
        data = np.ascontiguousarray(data, np.float32).ravel()
        rc = self.chk._fn("hist_collect")(self.h, _f(data), C.c_size_t(data.size))
        if rc:
            raise RuntimeError("hist_collect failed")

    def get(self):
        counts = np.zeros(self.bins, np.float32)
        mn, mx, tot = C.c_float(), C.c_float(), C.c_int64()
        self.chk._fn("hist_get")(self.h, _f(counts), C.byref(mn), C.byref(mx), C.byref(tot))
        return counts, float(mn.value), float(mx.value), int(tot.value)

    def __del__(self):
        try:
            f = self.chk._fn("hist_free")
            f.argtypes = [C.c_void_p]
            f(self.h)
        except Exception:
            pass


class Oracle(_Checker):
    prefix = "orc_"
    kind = "port"

    def __init__(self):
        super().__init__(build_oracle())

    def forward_float(self, T, B, I, H, W, R, bw, br, x, h0=None, ranges=None, want_v=False):
        """fp32 GRU; optionally folds the MinMax ranges (orc_forward_float)."""
        h = np.zeros((T + 1, B, H), np.float32)
        v = np.zeros((T, B, 4 * H), np.float32) if want_v else None
        rs = ranges.struct() if ranges is not None else None
        rc = self.lib.orc_forward_float(
            T, B, I, H, _f(W), _f(R), _f(bw), _f(br), _f(np.ascontiguousarray(x, np.float32)),
            _f(np.ascontiguousarray(h0, np.float32)) if h0 is not None else None, _f(h),
            _f(v) if v is not None else None, C.byref(rs) if rs is not None else None)
        if rc:
            raise RuntimeError("forward_float failed")
        if ranges is not None:
            ranges.load(rs)
        return (h, v) if want_v else h


    def forward_fstorage(self, T, B, I, H, wq, x, h0, params, sc):
        """Float-storage quantized forward (orc_forward_fstorage): (h dequantized, x_q floats)."""
        x = np.ascontiguousarray(x, np.float32)
        h = np.zeros((T + 1, B, H), np.float32)
        xq = np.zeros((T, B, I), np.float32)
        h0p = _f(np.ascontiguousarray(h0, np.float32)) if h0 is not None else None
        rc = self.lib.orc_forward_fstorage(T, B, I, H, *[_i(np.ascontiguousarray(a, np.int32)) for a in wq],
                                           _f(x), h0p, C.byref(params), *[_f(a) for a in sc], _f(h), _f(xq))
        if rc:
            raise RuntimeError("forward_fstorage failed")
        return h, xq


class Reference(_Checker):
    prefix = "ref_"
    kind = "reference"

    def __init__(self):
        so = build_ref()
        if so is None:
            raise FileNotFoundError("oracle/_ref/libqgru_ref.so has not been built")
        super().__init__(so)


class ReferenceGpu:
    """The reference's own GPU paths (ref_gpu_* of oracle/ref_shim.cc): host arrays in and out,
    run on the current CUDA device.  Only meaningful on a machine with a GPU."""
    prefix = "ref_gpu_"
    kind = "reference-gpu"

    def __init__(self, ref):
        self.lib, self.cabi, self.ref = ref.lib, ref.cabi, ref
        self.lib.ref_last_error.restype = C.c_char_p

    def _fn(self, name):
        return getattr(self.lib, self.prefix + name)

    def _check(self, rc, what):
        if rc:
            raise RuntimeError(f"{what}: {self.lib.ref_last_error().decode(errors='replace')}")

    def device_count(self):
        return int(self._fn("device_count")())

    def forward_i32(self, T, B, I, H, wq, x_q, h0_q, params, sc, training=False, masks=False):
        """quantGRUForwardInt32 on the GPU: h_q, and in training mode (v_q, the 5 clamp masks)."""
        x_q = np.ascontiguousarray(x_q, np.int32)
        h = np.zeros((T + 1, B, H), np.int32)
        v = np.zeros((T, B, 4 * H), np.int32) if training else None
        ms = None
        mptr = None
        if masks:
            ms = [np.zeros((T * B, 3 * H), np.uint8) for _ in range(4)] + [np.zeros((T * B, H), np.uint8)]
            mptr = (C.c_void_p * 5)(*[m.ctypes.data for m in ms])
        h0p = _i(np.ascontiguousarray(h0_q, np.int32)) if h0_q is not None else None
        rc = self._fn("forward_i32")(int(training), T, B, I, H,
                                     *[_i(np.ascontiguousarray(w, np.int32)) for w in wq], _i(x_q), h0p,
                                     C.byref(params), *[_f(s) for s in sc], _i(h),
                                     _i(v) if v is not None else None, mptr)
        self._check(rc, "ref_gpu_forward_i32")
        return (h, v, ms) if training else h

    def time_forward_i32(self, T, B, I, H, wq, x_q, params, sc, warmup=2, iters=5):
        """Milliseconds per call of quantGRUForwardInt32 (inference) with resident inputs."""
        ms = C.c_float()
        rc = self._fn("time_forward_i32")(T, B, I, H, *[_i(np.ascontiguousarray(w, np.int32)) for w in wq],
                                          _i(np.ascontiguousarray(x_q, np.int32)), C.byref(params),
                                          *[_f(s) for s in sc], int(warmup), int(iters), C.byref(ms))
        self._check(rc, "ref_gpu_time_forward_i32")
        return float(ms.value)

    def time_forward_fstorage(self, T, B, I, H, W, R, bw, br, x, params, sc, warmup=1, iters=3):
        """Milliseconds per call of quantGRUForwardFP (inference) with resident inputs."""
        ms = C.c_float()
        rc = self._fn("time_forward_fstorage")(T, B, I, H, _f(W), _f(R), _f(bw), _f(br),
                                               _f(np.ascontiguousarray(x, np.float32)), C.byref(params),
                                               *[_f(s) for s in sc], int(warmup), int(iters), C.byref(ms))
        self._check(rc, "ref_gpu_time_forward_fstorage")
        return float(ms.value)

    def forward_float(self, T, B, I, H, W, R, bw, br, x, h0=None, want_v=False):
        h = np.zeros((T + 1, B, H), np.float32)
        v = np.zeros((T, B, 4 * H), np.float32) if want_v else None
        rc = self._fn("forward_float")(T, B, I, H, _f(W), _f(R), _f(bw), _f(br),
                                       _f(np.ascontiguousarray(x, np.float32)),
                                       _f(np.ascontiguousarray(h0, np.float32)) if h0 is not None else None,
                                       _f(h), _f(v) if v is not None else None)
        self._check(rc, "ref_gpu_forward_float")
        return (h, v) if want_v else h

    def forward_fstorage(self, T, B, I, H, W, R, bw, br, x, h0, params, sc):
        """quantGRUForwardFP, inference: (h dequantized, x_q as floats, [W_q, R_q, bw_q, br_q] as
        floats)."""
        h = np.zeros((T + 1, B, H), np.float32)
        xq = np.zeros((T, B, I), np.float32)
        wq = [np.zeros((I, 3 * H), np.float32), np.zeros((H, 3 * H), np.float32),
              np.zeros(3 * H, np.float32), np.zeros(3 * H, np.float32)]
        rc = self._fn("forward_fstorage")(T, B, I, H, _f(W), _f(R), _f(bw), _f(br),
                                          _f(np.ascontiguousarray(x, np.float32)),
                                          _f(np.ascontiguousarray(h0, np.float32)) if h0 is not None else None,
                                          C.byref(params), *[_f(a) for a in sc], _f(h), _f(xq),
                                          *[_f(a) for a in wq])
        self._check(rc, "ref_gpu_forward_fstorage")
        return h, xq, wq

    def forward_fstorage_train(self, T, B, I, H, W, R, bw, br, x, h0, params, sc, int_storage=False):
        """quantGRUForwardFP (or, with int_storage, quantGRUForwardInt) in training mode:
        (h, v dequantized, dict of the eleven masks)."""
        from oracle.backward_np import MASK_NAMES
        h = np.zeros((T + 1, B, H), np.float32)
        v = np.zeros((T, B, 4 * H), np.float32)
        shapes = {"x": (T * B, I), "h0": (B, H), "W": (I, 3 * H), "R": (H, 3 * H), "bw": (3 * H,), "br": (3 * H,),
                  "ih_linear": (T * B, 3 * H), "hh_linear": (T * B, 3 * H), "gate_input": (T * B, 3 * H),
                  "gate_output": (T * B, 3 * H), "h": (T * B, H)}
        ms = {n: np.zeros(shapes[n], np.uint8) for n in MASK_NAMES}
        mptr = (C.c_void_p * 11)(*[ms[n].ctypes.data for n in MASK_NAMES])
        rc = self._fn("forward_int_train" if int_storage else "forward_fstorage_train")(T, B, I, H, _f(W), _f(R), _f(bw), _f(br),
                                                _f(np.ascontiguousarray(x, np.float32)),
                                                _f(np.ascontiguousarray(h0, np.float32)), C.byref(params),
                                                *[_f(a) for a in sc], _f(h), _f(v), mptr)
        self._check(rc, "ref_gpu_forward_fstorage_train")
        return h, v, ms

    def backward(self, T, B, I, H, W, R, bw, br, x, dh_new, h, v, masks=None):
        """hasteGRUBackward, or quantGRUBackward when `masks` (dict of all eleven uint8 arrays,
        names as oracle/backward_np.MASK_NAMES) is given: (dx, dW, dR, dbw, dbr, dh)."""
        from oracle.backward_np import MASK_NAMES
        f32 = lambda a: np.ascontiguousarray(a, np.float32)  # noqa: E731
        W_t, R_t = f32(np.asarray(W).T), f32(np.asarray(R).T)
        x_t = f32(np.asarray(x).transpose(2, 0, 1))
        outs = [np.zeros((T, B, I), np.float32), np.zeros((I, 3 * H), np.float32), np.zeros((H, 3 * H), np.float32),
                np.zeros(3 * H, np.float32), np.zeros(3 * H, np.float32), np.zeros((B, H), np.float32)]
        mptr, keep = None, []
        if masks is not None:
            keep = [np.ascontiguousarray(masks[n], np.uint8) for n in MASK_NAMES]
            mptr = (C.c_void_p * 11)(*[m.ctypes.data for m in keep])
        rc = self._fn("backward")(T, B, I, H, _f(W_t), _f(R_t), _f(f32(bw)), _f(f32(br)), _f(x_t), _f(f32(dh_new)),
                                  _f(f32(h)), _f(f32(v)), int(masks is not None), mptr, *[_f(o) for o in outs])
        self._check(rc, "ref_gpu_backward")
        return tuple(outs)

    def calibrate_minmax(self, T, B, I, H, W, R, bw, br, x, ranges):
        """forwardWithCalibrationGPU(MINMAX): folds one batch into `ranges`; returns h."""
        h = np.zeros((T + 1, B, H), np.float32)
        rs = ranges.struct()
        rc = self._fn("calibrate_minmax")(T, B, I, H, _f(W), _f(R), _f(bw), _f(br),
                                          _f(np.ascontiguousarray(x, np.float32)), C.byref(rs), _f(h))
        self._check(rc, "ref_gpu_calibrate_minmax")
        ranges.load(rs)
        return h

    def hist_new(self, bins=2048):
        f = self._fn("hist_new")
        f.restype = C.c_void_p
        return _Hist(self, C.c_void_p(f(int(bins))), bins)

    def histset_new(self, hidden, bins=2048):
        return _GpuHistSet(self, hidden, bins)


class _GpuHistSet:
    """GRUGPUHistogramCollectors of the reference, filled by its calibration forward."""

    def __init__(self, gpu, hidden, bins):
        f = gpu._fn("histset_new")
        f.restype = C.c_void_p
        self.gpu, self.hidden, self.bins = gpu, hidden, bins
        self.h = C.c_void_p(f(int(hidden), int(bins)))
        if not self.h:
            raise RuntimeError("ref_gpu_histset_new failed")

    def calibrate(self, T, B, I, H, W, R, bw, br, x, params, use_percentile):
        rc = self.gpu._fn("histset_calibrate")(self.h, T, B, I, H, _f(W), _f(R), _f(bw), _f(br),
                                               _f(np.ascontiguousarray(x, np.float32)), C.byref(params),
                                               int(use_percentile))
        self.gpu._check(rc, "ref_gpu_histset_calibrate")

    def sync(self):
        self.gpu._check(self.gpu._fn("histset_sync")(self.h), "ref_gpu_histset_sync")

    def get(self, index):
        """(counts, min, max, total) of histogram `index` (qgru_hist layout), or None if empty."""
        counts = np.zeros(self.bins, np.float32)
        mn, mx, tot, valid = C.c_float(), C.c_float(), C.c_int64(), C.c_int()
        rc = self.gpu._fn("histset_get")(self.h, int(index), _f(counts), C.byref(mn), C.byref(mx),
                                         C.byref(tot), C.byref(valid))
        self.gpu._check(rc, "ref_gpu_histset_get")
        if not valid.value:
            return None
        return counts, float(mn.value), float(mx.value), int(tot.value)

    def params(self, params, use_percentile, percentile=99.99):
        """calculateGRUQuantitativeParametersFromHistograms on the collected set; fills `params`
        in place and returns the four per-channel scale arrays."""
        sc = [np.zeros(3 * self.hidden, np.float32) for _ in range(4)]
        rc = self.gpu._fn("histset_params")(self.h, C.byref(params), int(use_percentile),
                                            C.c_float(percentile), *[_f(a) for a in sc])
        self.gpu._check(rc, "ref_gpu_histset_params")
        return sc

    def __del__(self):
        try:
            f = self.gpu._fn("histset_free")
            f.argtypes = [C.c_void_p]
            f(self.h)
        except Exception:
            pass


class ShimTest:
    """The reference-signature entry points of quant-gru-pytorch_b200/shim/gru_interface_b200.cc
    (quantGRUForwardInt32 / Int / IntIO), called with host arrays through oracle/shim_driver.cc.
    Needs oracle/_ref/libqgru_shimtest.so (built where the reference's headers are) and a GPU."""

    def __init__(self):
        self.lib = C.CDLL(os.path.join(_HERE, "_ref", "libqgru_shimtest.so"))
        self.lib.shimtest_last_error.restype = C.c_char_p

    def _check(self, rc, what):
        if rc:
            raise (ValueError if rc == 2 else RuntimeError)(f"{what}: {self.lib.shimtest_last_error().decode()}")

    def forward_i32(self, T, B, I, H, wq, x_q, h0_q, params, sc, training=False):
        h = np.zeros((T + 1, B, H), np.int32)
        v = np.zeros((T, B, 4 * H), np.int32) if training else None
        masks = [np.zeros((T * B, 3 * H), np.uint8) for _ in range(4)] + [np.zeros((T * B, H), np.uint8)] \
            if training else None
        mp = (C.c_void_p * 5)(*[m.ctypes.data for m in masks]) if training else None
        h0p = _i(np.ascontiguousarray(h0_q, np.int32)) if h0_q is not None else None
        rc = self.lib.shimtest_forward_i32(int(training), T, B, I, H, *[_i(np.ascontiguousarray(a, np.int32)) for a in wq],
                                           _i(np.ascontiguousarray(x_q, np.int32)), h0p, C.byref(params),
                                           *[_f(a) for a in sc], _i(h), _i(v) if training else None, mp)
        self._check(rc, "quantGRUForwardInt32 (shim)")
        return (h, v, masks) if training else h

    def forward_f32(self, T, B, I, H, W, R, bw, br, x, h0, params, sc):
        h = np.zeros((T + 1, B, H), np.float32)
        q = [np.zeros((I, 3 * H), np.int32), np.zeros((H, 3 * H), np.int32), np.zeros(3 * H, np.int32),
             np.zeros(3 * H, np.int32), np.zeros((T, B, I), np.int32)]
        h0p = _f(np.ascontiguousarray(h0, np.float32)) if h0 is not None else None
        rc = self.lib.shimtest_forward_f32(T, B, I, H, *[_f(np.ascontiguousarray(a, np.float32)) for a in (W, R, bw, br, x)],
                                           h0p, C.byref(params), *[_f(a) for a in sc], _f(h), *[_i(a) for a in q])
        self._check(rc, "quantGRUForwardInt (shim)")
        return h, q[:4], q[4]

    def forward_intio(self, T, B, I, H, W, R, bw, br, x_q, h0_q, params, sc):
        h = np.zeros((T + 1, B, H), np.int32)
        h0p = _i(np.ascontiguousarray(h0_q, np.int32)) if h0_q is not None else None
        rc = self.lib.shimtest_forward_intio(T, B, I, H, *[_f(np.ascontiguousarray(a, np.float32)) for a in (W, R, bw, br)],
                                             _i(np.ascontiguousarray(x_q, np.int32)), h0p, C.byref(params),
                                             *[_f(a) for a in sc], _i(h))
        self._check(rc, "quantGRUForwardIntIO (shim)")
        return h


def reference_or_none():
    try:
        return Reference()
    except (FileNotFoundError, OSError, subprocess.CalledProcessError):
        return None
