"""Python host side of the C ABI, shaped like the reference's ``gru_ops`` pybind module.

``Handle`` is a thin object over ``qgru_handle``.  The module-level functions keep the names,
argument order and return conventions of the reference binding for the integer path
(pytorch/lib/gru_interface_binding.cc): ``forward_quant_int_storage`` (:436),
``forward_quantized_int_io`` (:573), ``forward_fp`` (:629), ``forward_calibrate`` (:683) and
``calculate_gru_quantitative_parameters`` (:209).  Tensors are torch CUDA tensors; torch is
used for device memory and streams only - every computation happens in libqgru_b200.so.
"""
import ctypes as C

import torch

from . import _cabi
from .params import Histograms, GRUQuantParams, OperatorQuantConfig, Ranges, WEIGHT_OPS  # noqa: F401


def _ptr(t):
    return C.c_void_p(t.data_ptr()) if t is not None else None


def _stream(device):
    return C.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def _check_tensor(t, name, dtype, shape=None, cuda=True):
    if not isinstance(t, torch.Tensor):
        raise TypeError(f"{name} must be a torch.Tensor")
    if cuda and not t.is_cuda:
        raise ValueError(f"{name} must be CUDA {dtype} tensor")
    if t.dtype != dtype:
        raise ValueError(f"{name} must be CUDA {dtype} tensor")
    if shape is not None and tuple(t.shape) != tuple(shape):
        raise ValueError(f"{name} must have shape {list(shape)}, got {list(t.shape)}")
    return t.contiguous()


class Handle:
    """One (device, direction) instance of the integer GRU forward.

    Owns the packed weights, the derived rescale tables and a growing device workspace, so
    repeated forwards allocate nothing and never synchronise the device."""

    def __init__(self, input_size, hidden_size, device=0):
        self._lib = _cabi.lib()
        self.input_size, self.hidden_size, self.device = input_size, hidden_size, int(device)
        h = C.c_void_p()
        st = self._lib.qgru_create(C.byref(h), self.device, input_size, hidden_size)
        if st != _cabi.QGRU_OK:
            raise _cabi.QgruError(st, "qgru_create", "no usable CUDA device" if st == 2 else "")
        self._h = h
        self._tdev = torch.device("cuda", self.device)

    # -- lifecycle
    def close(self):
        if getattr(self, "_h", None):
            self._lib.qgru_destroy(self._h)
            self._h = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _ck(self, st, where):
        _cabi.check(st, where, self._h)

    # -- configuration
    def set_option(self, name, value):
        self._ck(self._lib.qgru_set_option(self._h, name.encode(), str(value).encode()), "qgru_set_option")

    def set_params(self, params):
        fp = C.POINTER(C.c_float)
        self._params = params
        self._ck(self._lib.qgru_set_params(self._h, C.byref(params.c),
                                           *[params.scales[n].ctypes.data_as(fp) for n in WEIGHT_OPS]),
                 "qgru_set_params")

    def set_weights_f32(self, W, R, bw, br):
        I, H = self.input_size, self.hidden_size
        W = _check_tensor(W, "W", torch.float32, (I, 3 * H))
        R = _check_tensor(R, "R", torch.float32, (H, 3 * H))
        bw = _check_tensor(bw, "bw", torch.float32, (3 * H,))
        br = _check_tensor(br, "br", torch.float32, (3 * H,))
        self._ck(self._lib.qgru_set_weights_f32(self._h, _ptr(W), _ptr(R), _ptr(bw), _ptr(br),
                                                _stream(self._tdev)), "qgru_set_weights_f32")

    def set_weights_i32(self, W_q, R_q, bw_q, br_q):
        I, H = self.input_size, self.hidden_size
        W_q = _check_tensor(W_q, "W_q", torch.int32, (I, 3 * H))
        R_q = _check_tensor(R_q, "R_q", torch.int32, (H, 3 * H))
        bw_q = _check_tensor(bw_q, "bw_q", torch.int32, (3 * H,))
        br_q = _check_tensor(br_q, "br_q", torch.int32, (3 * H,))
        self._ck(self._lib.qgru_set_weights_i32(self._h, _ptr(W_q), _ptr(R_q), _ptr(bw_q), _ptr(br_q),
                                                _stream(self._tdev)), "qgru_set_weights_i32")

    def get_weights_i32(self):
        I, H = self.input_size, self.hidden_size
        o = dict(dtype=torch.int32, device=self._tdev)
        out = [torch.empty((I, 3 * H), **o), torch.empty((H, 3 * H), **o),
               torch.empty(3 * H, **o), torch.empty(3 * H, **o)]
        self._ck(self._lib.qgru_get_weights_i32(self._h, *[_ptr(t) for t in out], _stream(self._tdev)),
                 "qgru_get_weights_i32")
        return out

    def _out_buffer(self, out, name, dtype, shape):
        """A caller-supplied result tensor is written through its raw pointer: it must be a
        contiguous tensor of exactly this shape and type on this handle's device."""
        if out is None:
            return torch.empty(shape, dtype=dtype, device=self._tdev)
        if not isinstance(out, torch.Tensor) or not out.is_cuda or out.device != self._tdev:
            raise ValueError(f"{name} must be a CUDA tensor on {self._tdev}")
        if out.dtype != dtype or tuple(out.shape) != tuple(shape) or not out.is_contiguous():
            raise ValueError(f"{name} must be a contiguous {dtype} tensor of shape {list(shape)}")
        return out

    # -- forward (device tensors)
    def forward_i32(self, x_q, h0_q=None, reverse=False, out=None, sync=True):
        """x_q [T,B,I] int32 -> h_q [(T+1),B,H] int32 (slot layout as in include/qgru.h)."""
        x_q = _check_tensor(x_q, "x_q", torch.int32)
        if x_q.dim() != 3 or x_q.shape[2] != self.input_size:
            raise ValueError("x_q must have shape [time_steps, batch_size, input_size]")
        T, B = int(x_q.shape[0]), int(x_q.shape[1])
        if h0_q is not None:
            h0_q = _check_tensor(h0_q, "h0_q", torch.int32, (B, self.hidden_size))
        h_q = self._out_buffer(out, "out", torch.int32, (T + 1, B, self.hidden_size))
        self._ck(self._lib.qgru_forward_i32(self._h, T, B, _ptr(x_q), _ptr(h0_q), _ptr(h_q),
                                            _cabi.FLAG_REVERSE if reverse else 0, _stream(self._tdev)),
                 "qgru_forward_i32")
        if sync:
            self.synchronize()
        return h_q

    def forward_i32_train(self, x_q, h0_q=None, reverse=False, want_masks=False):
        """Training-mode integer forward: (h_q [(T+1),B,H], v_q [T,B,4H]) int32; v_q holds the
        quantized update / reset / new gate outputs and the R*h + br row of the new gate.
        With want_masks also the five uint8 clamp masks (1 = not clamped) as a third result:
        [W*x+bw [T*B,3H], R*h+br [T*B,3H], gate inputs [T*B,3H], gate outputs [T*B,3H],
        h [T*B,H]]."""
        T, B = int(x_q.shape[0]), int(x_q.shape[1])
        H = self.hidden_size
        x_q = _check_tensor(x_q, "x_q", torch.int32, (T, B, self.input_size))
        if h0_q is not None:
            h0_q = _check_tensor(h0_q, "h0_q", torch.int32, (B, H))
        h = torch.empty((T + 1, B, H), dtype=torch.int32, device=self._tdev)
        v = torch.empty((T, B, 4 * H), dtype=torch.int32, device=self._tdev)
        masks, mk = None, None
        if want_masks:
            masks = [torch.empty((T * B, 3 * H), dtype=torch.uint8, device=self._tdev) for _ in range(4)]
            masks.append(torch.empty((T * B, H), dtype=torch.uint8, device=self._tdev))
            mk = _cabi.Masks(*[m.data_ptr() for m in masks])
        self._ck(self._lib.qgru_forward_i32_train(self._h, T, B, _ptr(x_q), _ptr(h0_q), _ptr(h), _ptr(v),
                                                  C.byref(mk) if mk is not None else None,
                                                  _cabi.FLAG_REVERSE if reverse else 0, _stream(self._tdev)),
                 "qgru_forward_i32_train")
        self.synchronize()
        return (h, v, masks) if want_masks else (h, v)

    def forward_i32_static(self, x_q, h0_q=None, reverse=False, out=None, sync=True):
        """forward_i32 for callers that may not allocate device memory at call time: the
        workspace is a fixed 8 MiB array inside the library (shared by every call on the GPU, so
        overlapping calls race); sizes that do not fit raise ValueError.  Pass `out` to avoid
        the allocation of the result tensor too."""
        x_q = _check_tensor(x_q, "x_q", torch.int32)
        if x_q.dim() != 3 or x_q.shape[2] != self.input_size:
            raise ValueError("x_q must have shape [time_steps, batch_size, input_size]")
        T, B = int(x_q.shape[0]), int(x_q.shape[1])
        if h0_q is not None:
            h0_q = _check_tensor(h0_q, "h0_q", torch.int32, (B, self.hidden_size))
        h_q = self._out_buffer(out, "out", torch.int32, (T + 1, B, self.hidden_size))
        self._ck(self._lib.qgru_forward_i32_static(self._h, T, B, _ptr(x_q), _ptr(h0_q), _ptr(h_q),
                                                   _cabi.FLAG_REVERSE if reverse else 0,
                                                   _stream(self._tdev)), "qgru_forward_i32_static")
        if sync:
            self.synchronize()
        return h_q

    def forward_f32(self, x, h0=None, reverse=False, want_x_q=False, out=None, sync=True):
        x = _check_tensor(x, "x", torch.float32)
        if x.dim() != 3 or x.shape[2] != self.input_size:
            raise ValueError("x must have shape [time_steps, batch_size, input_size]")
        T, B = int(x.shape[0]), int(x.shape[1])
        if h0 is not None:
            h0 = _check_tensor(h0, "h0", torch.float32, (B, self.hidden_size))
        h = self._out_buffer(out, "out", torch.float32, (T + 1, B, self.hidden_size))
        x_q = torch.empty((T, B, self.input_size), dtype=torch.int32, device=self._tdev) if want_x_q else None
        self._ck(self._lib.qgru_forward_f32(self._h, T, B, _ptr(x), _ptr(h0), _ptr(h), _ptr(x_q),
                                            _cabi.FLAG_REVERSE if reverse else 0, _stream(self._tdev)),
                 "qgru_forward_f32")
        if sync:
            self.synchronize()
        return (h, x_q) if want_x_q else h

    def forward_f32_q8(self, x, h0=None, reverse=False, out=None, sync=True):
        """forward_f32 with the result left in 8 bits: returns the quantized states
        [(T+1),B,H] as torch.int8 (torch.uint8 when the h operator is unsigned).  Dequantize
        with ``h_quant_meta()``: (q - zero_point) * scale is what forward_f32 returns."""
        x = _check_tensor(x, "x", torch.float32)
        if x.dim() != 3 or x.shape[2] != self.input_size:
            raise ValueError("x must have shape [time_steps, batch_size, input_size]")
        T, B = int(x.shape[0]), int(x.shape[1])
        if h0 is not None:
            h0 = _check_tensor(h0, "h0", torch.float32, (B, self.hidden_size))
        dtype = torch.uint8 if self.h_quant_meta()[2] else torch.int8
        h = self._out_buffer(out, "out", dtype, (T + 1, B, self.hidden_size))
        self._ck(self._lib.qgru_forward_f32_q8(self._h, T, B, _ptr(x), _ptr(h0), _ptr(h),
                                               _cabi.FLAG_REVERSE if reverse else 0, _stream(self._tdev)),
                 "qgru_forward_f32_q8")
        if sync:
            self.synchronize()
        return h

    def h_quant_meta(self):
        """(scale, zero_point, is_unsigned) of the state h: the decoded scale the kernels use."""
        o = self._params.c.op[_cabi.OP_INDEX["h"]]
        return decode_effective_scale(float(o.scale), bool(self._params.c.use_pot2)), int(o.zero_point), \
            bool(o.is_unsigned) and o.bits < 32

    def forward_fstorage(self, x, h0=None, reverse=False, want_x_q=False, sync=True):
        """Float-storage quantized forward (the reference's forward_quant_float_storage, inference):
        float requantization and real sigmoid / tanh on quantized tensors.  x [T,B,I] fp32 ->
        h [(T+1),B,H] fp32 dequantized; with want_x_q also the quantized x as floats."""
        x = _check_tensor(x, "x", torch.float32)
        if x.dim() != 3 or x.shape[2] != self.input_size:
            raise ValueError("x must have shape [time_steps, batch_size, input_size]")
        T, B = int(x.shape[0]), int(x.shape[1])
        if h0 is not None:
            h0 = _check_tensor(h0, "h0", torch.float32, (B, self.hidden_size))
        h = torch.empty((T + 1, B, self.hidden_size), dtype=torch.float32, device=self._tdev)
        x_q = torch.empty((T, B, self.input_size), dtype=torch.float32, device=self._tdev) if want_x_q else None
        self._ck(self._lib.qgru_forward_fstorage(self._h, T, B, _ptr(x), _ptr(h0), _ptr(h), _ptr(x_q),
                                                 _cabi.FLAG_REVERSE if reverse else 0, _stream(self._tdev)),
                 "qgru_forward_fstorage")
        if sync:
            self.synchronize()
        return (h, x_q) if want_x_q else h

    def get_weights_dequantized(self):
        """The handle's quantized weights times their scales: (W [I,3H], R [H,3H], bw, br) fp32."""
        I, H = self.input_size, self.hidden_size
        outs = [torch.empty(s, dtype=torch.float32, device=self._tdev) for s in ((I, 3 * H), (H, 3 * H), (3 * H,), (3 * H,))]
        self._ck(self._lib.qgru_get_weights_dequantized(self._h, *[_ptr(o) for o in outs], _stream(self._tdev)),
                 "qgru_get_weights_dequantized")
        return outs

    def dequantize_f32(self, q, op_name):
        """Float-stored quantized values of operator `op_name` -> real values."""
        q = _check_tensor(q, "q", torch.float32)
        out = torch.empty_like(q)
        self._ck(self._lib.qgru_dequantize_f32(self._h, _cabi.OP_INDEX[op_name], _ptr(q), _ptr(out), q.numel(),
                                               _stream(self._tdev)), "qgru_dequantize_f32")
        return out

    MASK_NAMES = ("x", "h0", "W", "R", "bw", "br", "ih_linear", "hh_linear", "gate_input", "gate_output", "h")

    def forward_fstorage_train(self, W, R, bw, br, x, h0=None, reverse=False, int_storage=False):
        """Training mode of the float-storage forward: (h [(T+1),B,H], v [T,B,4H] dequantized,
        x_q [T,B,I] as floats, masks: dict of the eleven uint8 clamp masks, 1 = not clamped).
        W..br are the float master weights the handle was loaded with (set_weights_f32).
        int_storage: the integer forward in training mode instead (quantGRUForwardInt:
        piecewise-linear gates, x_q as int32)."""
        x = _check_tensor(x, "x", torch.float32)
        T, B = int(x.shape[0]), int(x.shape[1])
        I, H = self.input_size, self.hidden_size
        ws = [_check_tensor(t, n, torch.float32) for t, n in ((W, "W"), (R, "R"), (bw, "bw"), (br, "br"))]
        if h0 is not None:
            h0 = _check_tensor(h0, "h0", torch.float32, (B, H))
        dev = self._tdev
        h = torch.empty((T + 1, B, H), dtype=torch.float32, device=dev)
        v = torch.empty((T, B, 4 * H), dtype=torch.float32, device=dev)
        x_q = torch.empty((T, B, I), dtype=torch.int32 if int_storage else torch.float32, device=dev)
        shapes = {"x": (T * B, I), "h0": (B, H), "W": (I, 3 * H), "R": (H, 3 * H), "bw": (3 * H,), "br": (3 * H,),
                  "ih_linear": (T * B, 3 * H), "hh_linear": (T * B, 3 * H), "gate_input": (T * B, 3 * H),
                  "gate_output": (T * B, 3 * H), "h": (T * B, H)}
        masks = {n: torch.ones(shapes[n], dtype=torch.uint8, device=dev) for n in self.MASK_NAMES}
        mk = _cabi.BwdMasks(*[masks[n].data_ptr() for n in self.MASK_NAMES])
        fn = self._lib.qgru_forward_f32_train if int_storage else self._lib.qgru_forward_fstorage_train
        self._ck(fn(self._h, T, B, *[_ptr(t) for t in ws], _ptr(x), _ptr(h0), _ptr(h), _ptr(v), _ptr(x_q),
                    C.byref(mk), _cabi.FLAG_REVERSE if reverse else 0, _stream(dev)),
                 "qgru_forward_f32_train" if int_storage else "qgru_forward_fstorage_train")
        self.synchronize()
        return h, v, x_q, masks

    def backward(self, W, R, x, dh_new, h, v, masks=None, dh_last=None):
        """Backward pass through the saved forward (hasteGRUBackward; with `masks`, a dict of
        uint8 tensors named as in qgru_bwd_masks, quantGRUBackward).  W [I,3H], R [H,3H],
        x [T,B,I], dh_new / h [(T+1),B,H], v [T,B,4H]: CUDA fp32.  Returns
        (dx [T,B,I], dW, dR, dbw, dbr, dh [B,H])."""
        T, B = int(x.shape[0]), int(x.shape[1])
        I, H = self.input_size, self.hidden_size
        x = _check_tensor(x, "x", torch.float32, (T, B, I))
        W = _check_tensor(W, "W", torch.float32, (I, 3 * H))
        R = _check_tensor(R, "R", torch.float32, (H, 3 * H))
        dh_new = _check_tensor(dh_new, "dh_new", torch.float32, (T + 1, B, H))
        h = _check_tensor(h, "h", torch.float32, (T + 1, B, H))
        v = _check_tensor(v, "v", torch.float32, (T, B, 4 * H))
        x_t = x.permute(2, 0, 1).contiguous()        # [I, T*B]
        W_t, R_t = W.t().contiguous(), R.t().contiguous()
        dev = self._tdev
        dx = torch.empty((T, B, I), dtype=torch.float32, device=dev)
        dW = torch.zeros((I, 3 * H), dtype=torch.float32, device=dev)
        dR = torch.zeros((H, 3 * H), dtype=torch.float32, device=dev)
        dbw = torch.zeros(3 * H, dtype=torch.float32, device=dev)
        dbr = torch.zeros(3 * H, dtype=torch.float32, device=dev)
        dh = torch.zeros((B, H), dtype=torch.float32, device=dev) if dh_last is None else \
            _check_tensor(dh_last, "dh_last", torch.float32, (B, H)).clone()
        mk, keep = None, []
        if masks:
            mk = _cabi.BwdMasks()
            for name, t in masks.items():
                if t is not None:
                    keep.append(_check_tensor(t, name, torch.uint8))   # alive until the call has run
                    setattr(mk, name, keep[-1].data_ptr())
        self._ck(self._lib.qgru_backward(self._h, T, B, _ptr(W_t), _ptr(R_t), _ptr(x_t), _ptr(dh_new), _ptr(h),
                                         _ptr(v), _ptr(dx), _ptr(dW), _ptr(dR), _ptr(dbw), _ptr(dbr), _ptr(dh),
                                         C.byref(mk) if mk is not None else None, _stream(dev)), "qgru_backward")
        self.synchronize()
        return dx, dW, dR, dbw, dbr, dh

    # -- forward (host tensors; copies are part of the call)
    def forward_i32_host(self, x_q, h0_q=None, reverse=False, out=None):
        x_q = _check_tensor(x_q, "x_q", torch.int32, cuda=False)
        T, B = int(x_q.shape[0]), int(x_q.shape[1])
        h_q = out if out is not None else torch.empty((T + 1, B, self.hidden_size), dtype=torch.int32)
        self._ck(self._lib.qgru_forward_i32_host(self._h, T, B, _ptr(x_q), _ptr(h0_q), _ptr(h_q),
                                                 _cabi.FLAG_REVERSE if reverse else 0,
                                                 _stream(self._tdev)), "qgru_forward_i32_host")
        return h_q

    def forward_f32_host(self, x, h0=None, reverse=False, out=None):
        x = _check_tensor(x, "x", torch.float32, cuda=False)
        T, B = int(x.shape[0]), int(x.shape[1])
        h = out if out is not None else torch.empty((T + 1, B, self.hidden_size), dtype=torch.float32)
        self._ck(self._lib.qgru_forward_f32_host(self._h, T, B, _ptr(x), _ptr(h0), _ptr(h),
                                                 _cabi.FLAG_REVERSE if reverse else 0,
                                                 _stream(self._tdev)), "qgru_forward_f32_host")
        return h

    # -- float mode / calibration
    def forward_float(self, W, R, bw, br, x, h0=None, want_v=False):
        T, B = int(x.shape[0]), int(x.shape[1])
        H = self.hidden_size
        h = torch.empty((T + 1, B, H), dtype=torch.float32, device=self._tdev)
        v = torch.empty((T, B, 4 * H), dtype=torch.float32, device=self._tdev) if want_v else None
        args = [_check_tensor(t, n, torch.float32) for t, n in
                ((W, "W"), (R, "R"), (bw, "bw"), (br, "br"), (x, "x"))]
        if h0 is not None:
            h0 = _check_tensor(h0, "h0", torch.float32, (B, H))
        self._ck(self._lib.qgru_forward_float(self._h, T, B, *[_ptr(t) for t in args], _ptr(h0),
                                              _ptr(h), _ptr(v), _stream(self._tdev)), "qgru_forward_float")
        self.synchronize()
        return (h, v) if want_v else h

    def calibrate_minmax(self, W, R, bw, br, x, ranges, h0=None, want_h=False):
        """Float forward + fold of this batch's min/max into ``ranges`` (in place)."""
        T, B = int(x.shape[0]), int(x.shape[1])
        H = self.hidden_size
        args = [_check_tensor(t, n, torch.float32) for t, n in
                ((W, "W"), (R, "R"), (bw, "bw"), (br, "br"), (x, "x"))]
        if h0 is not None:
            h0 = _check_tensor(h0, "h0", torch.float32, (B, H))
        h = torch.empty((T + 1, B, H), dtype=torch.float32, device=self._tdev) if want_h else None
        rs = ranges.struct()
        self._ck(self._lib.qgru_calibrate_minmax(self._h, T, B, *[_ptr(t) for t in args], _ptr(h0),
                                                 C.byref(rs), _ptr(h), _stream(self._tdev)),
                 "qgru_calibrate_minmax")
        ranges.load(rs)
        return h

    def calibrate_hist(self, W, R, bw, br, x, hist, granularity, h0=None):
        """Float forward + fold of every operator's values of this batch into ``hist``
        (a params.Histograms); granularity = QGRU_PER_* of W, R, bw, br."""
        T, B = int(x.shape[0]), int(x.shape[1])
        H = self.hidden_size
        args = [_check_tensor(t, n, torch.float32) for t, n in
                ((W, "W"), (R, "R"), (bw, "bw"), (br, "br"), (x, "x"))]
        if h0 is not None:
            h0 = _check_tensor(h0, "h0", torch.float32, (B, H))
        gran = (C.c_int32 * 4)(*[int(g) for g in granularity])
        self._ck(self._lib.qgru_calibrate_hist(self._h, hist._h, T, B, *[_ptr(t) for t in args], _ptr(h0),
                                               gran, _stream(self._tdev)), "qgru_calibrate_hist")

    # -- introspection
    def synchronize(self):
        self._ck(self._lib.qgru_synchronize(self._h, _stream(self._tdev)), "qgru_synchronize")

    def last_timing(self):
        a, b, c = C.c_float(), C.c_float(), C.c_float()
        self._ck(self._lib.qgru_last_timing(self._h, C.byref(a), C.byref(b), C.byref(c)), "qgru_last_timing")
        return {"input_gemm_ms": a.value, "recurrence_ms": b.value, "total_ms": c.value}

    def timing_window(self, n_calls):
        """Sums of the per-kernel durations over the last n_calls forwards (<= 64)."""
        n, a, b, c = C.c_int(int(n_calls)), C.c_float(), C.c_float(), C.c_float()
        self._ck(self._lib.qgru_timing_window(self._h, C.byref(n), C.byref(a), C.byref(b), C.byref(c)),
                 "qgru_timing_window")
        return {"calls": n.value, "input_gemm_ms": a.value, "recurrence_ms": b.value, "total_ms": c.value}

    def launch_count(self):
        return int(self._lib.qgru_launch_count(self._h))

    def describe_plan(self):
        return self._lib.qgru_describe_plan(self._h, 0, 0).decode()


# --------------------------------------------------------------------------------------
# Functions with the reference binding's names.  A small cache keeps one Handle per
# (device, I, H, slot) so that, unlike the reference, repeated calls reuse packed weights'
# storage, streams and workspace.  `slot` separates the two directions.
# --------------------------------------------------------------------------------------
_handles = {}


def _handle_for(device, I, H, slot=0):
    key = (int(device), int(I), int(H), slot)
    hd = _handles.get(key)
    if hd is None:
        hd = _handles[key] = Handle(I, H, device=device)
    return hd


def release_handles():
    for hd in _handles.values():
        hd.close()
    _handles.clear()


def init_gru_cublas():
    """Kept for drop-in compatibility; the integer path uses no cuBLAS handle."""
    return None


def calculate_gru_quantitative_parameters(quant_ranges, bitwidth_config):
    """MinMax ranges + bit-width config -> GRUQuantParams with LUTs (binding :209-231)."""
    return GRUQuantParams.from_ranges(quant_ranges, bitwidth_config)


def calculate_gru_quantitative_parameters_from_histograms(hist_collectors, bitwidth_config,
                                                          use_percentile=False, percentile_value=99.99):
    """Histograms + bit-width config -> GRUQuantParams with LUTs (binding :233-262): Percentile
    (use_percentile) or SQNR."""
    return GRUQuantParams.from_histograms(hist_collectors, bitwidth_config, use_percentile, percentile_value)


def forward_quant_int_storage(is_training, time_steps, batch_size, input_size, hidden_size,
                              W, R, bw, br, x, h0, quant_params, slot=0, reverse=False):
    """Integer forward with float interface (binding :436-571).

    Returns the reference's 18-tuple (h [(T+1),B,H] f32, v, W_q, R_q, bw_q, br_q, x_q (int32), then
    the eleven clamp masks in the order of Handle.MASK_NAMES); in inference mode v and the
    masks are empty tensors."""
    x = _check_tensor(x, "x", torch.float32, (time_steps, batch_size, input_size))
    hd = _handle_for(x.device.index or 0, input_size, hidden_size, slot)
    hd.set_params(quant_params)
    hd.set_weights_f32(W, R, bw, br)
    h0 = h0 if (h0 is not None and h0.numel() > 0) else None
    W_q, R_q, bw_q, br_q = hd.get_weights_i32()
    if is_training:
        h, v, x_q, m = hd.forward_fstorage_train(W, R, bw, br, x, h0, reverse=reverse, int_storage=True)
        return (h, v, W_q, R_q, bw_q, br_q, x_q) + tuple(m[n] for n in Handle.MASK_NAMES)
    h, x_q = hd.forward_f32(x, h0, reverse=reverse, want_x_q=True)
    e = torch.empty(0, dtype=torch.uint8, device=x.device)
    v = torch.empty(0, dtype=torch.float32, device=x.device)
    return (h, v, W_q, R_q, bw_q, br_q, x_q) + (e,) * 11


def forward_quant_float_storage(is_training, time_steps, batch_size, input_size, hidden_size,
                                W, R, bw, br, x, h0, quant_params, slot=0, reverse=False):
    """Float-storage quantized forward (binding :283-423): quantized values kept as floats, float
    requantization, real sigmoid / tanh.

    Returns the reference's 18-tuple (h [(T+1),B,H] f32, v, W_q, R_q, bw_q, br_q, x_q, x_mask,
    h0_mask, W_mask, R_mask, bw_mask, br_mask, weight_ih_linear_mask, weight_hh_linear_mask,
    gate_input_mask, gate_output_mask, h_mask) with the quantized tensors as float32; in
    inference mode v and the masks are empty tensors."""
    x = _check_tensor(x, "x", torch.float32, (time_steps, batch_size, input_size))
    hd = _handle_for(x.device.index or 0, input_size, hidden_size, slot)
    hd.set_params(quant_params)
    hd.set_weights_f32(W, R, bw, br)
    h0 = h0 if (h0 is not None and h0.numel() > 0) else None
    W_q, R_q, bw_q, br_q = [t.to(torch.float32) for t in hd.get_weights_i32()]
    if is_training:
        h, v, x_q, m = hd.forward_fstorage_train(W, R, bw, br, x, h0, reverse=reverse)
        return (h, v, W_q, R_q, bw_q, br_q, x_q) + tuple(m[n] for n in Handle.MASK_NAMES)
    h, x_q = hd.forward_fstorage(x, h0, reverse=reverse, want_x_q=True)
    e = torch.empty(0, dtype=torch.uint8, device=x.device)
    v = torch.empty(0, dtype=torch.float32, device=x.device)
    return (h, v, W_q, R_q, bw_q, br_q, x_q) + (e,) * 11


def backward_fp(time_steps, batch_size, input_size, hidden_size, W, R, bw, br, x, dh_new, h, v):
    """Float backward (binding :945-1020): returns (dx, dW, dR, dbw, dbr, dh)."""
    hd = _handle_for(x.device.index or 0, input_size, hidden_size, "fp")
    return hd.backward(W, R, x, dh_new, h, v)


def decode_effective_scale(scale, use_pot2):
    """The scale the kernels really apply for a stored scale (binding :1285-1296)."""
    out = C.c_float()
    _cabi.check(_cabi.lib().qgru_decode_effective_scale(float(scale), int(bool(use_pot2)), C.byref(out)),
                "qgru_decode_effective_scale")
    return float(out.value)


def backward_quant_float_storage(time_steps, batch_size, input_size, hidden_size, W_q, R_q, bw_q, br_q, x_q,
                                 dh_new, h, v, quant_params, x_mask=None, h0_mask=None, W_mask=None, R_mask=None,
                                 bw_mask=None, br_mask=None, weight_ih_linear_mask=None,
                                 weight_hh_linear_mask=None, gate_input_mask=None, gate_output_mask=None,
                                 h_mask=None):
    """Backward of the quantized training forward with its straight-through masks (binding
    :763-900): W_q .. x_q are the float-stored quantized tensors the forward returned; they are
    dequantized here (per-channel weight scales, the scale and zero point of x), then
    quantGRUBackward's arithmetic runs.  Returns (dx, dW, dR, dbw, dbr, dh)."""
    c = quant_params.c
    pot2 = bool(c.use_pot2)
    dev = x_q.device

    def chan(name):
        return torch.tensor([decode_effective_scale(s, pot2) for s in quant_params.scales[name]],
                            dtype=torch.float32, device=dev)

    W = W_q.to(torch.float32) * chan("W")
    R = R_q.to(torch.float32) * chan("R")
    xo = c.op[_cabi.OP_INDEX["x"]]
    x = (x_q.to(torch.float32) - float(xo.zero_point)) * decode_effective_scale(xo.scale, pot2)
    hd = _handle_for(dev.index or 0, input_size, hidden_size, "fp")
    masks = {"x": x_mask, "h0": h0_mask, "W": W_mask, "R": R_mask, "bw": bw_mask, "br": br_mask,
             "ih_linear": weight_ih_linear_mask, "hh_linear": weight_hh_linear_mask,
             "gate_input": gate_input_mask, "gate_output": gate_output_mask, "h": h_mask}
    masks = {k: (m if (m is not None and m.numel() > 0) else None) for k, m in masks.items()}
    return hd.backward(W, R, x, dh_new, h, v, masks=masks)


def forward_quantized_int_io(time_steps, batch_size, input_size, hidden_size, W, R, bw, br, x_q,
                             h0_q, quant_params, slot=0, reverse=False):
    """int32 in / int32 out inference (binding :573-618): returns (output_q [T,B,H], h_n_q [1,B,H])."""
    x_q = _check_tensor(x_q, "x_q", torch.int32, (time_steps, batch_size, input_size))
    hd = _handle_for(x_q.device.index or 0, input_size, hidden_size, slot)
    hd.set_params(quant_params)
    hd.set_weights_f32(W, R, bw, br)
    h0_q = h0_q if (h0_q is not None and h0_q.numel() > 0) else None
    h_q = hd.forward_i32(x_q, h0_q, reverse=reverse)
    if reverse:
        return h_q[:time_steps].contiguous(), h_q[0:1].contiguous()
    return h_q[1:].contiguous(), h_q[time_steps:time_steps + 1].contiguous()


def forward_fp(is_training, time_steps, batch_size, input_size, hidden_size, W, R, bw, br, x, h0):
    """Unquantized fp32 GRU (binding :629-681): returns (h [(T+1),B,H], v [T,B,4H])."""
    x = _check_tensor(x, "x", torch.float32, (time_steps, batch_size, input_size))
    hd = _handle_for(x.device.index or 0, input_size, hidden_size, "fp")
    h0 = h0 if (h0 is not None and h0.numel() > 0) else None
    return hd.forward_float(W, R, bw, br, x, h0, want_v=True)


def forward_calibrate(is_training, time_steps, batch_size, input_size, hidden_size, W, R, bw, br,
                      x, h0, calib_method_str, bitwidth_config, quant_ranges=None,
                      hist_collectors=None):
    """Calibration forward (binding :683-790): a float forward whose operator statistics are
    folded in place into ``quant_ranges`` (method 'minmax') or into ``hist_collectors``
    (methods 'sqnr' and 'percentile'); returns (h, v)."""
    method = calib_method_str.lower()
    if method in ("sqnr", "percentile", "histogram"):
        if hist_collectors is None:
            raise ValueError("hist_collectors is required for histogram calibration")
        x = _check_tensor(x, "x", torch.float32, (time_steps, batch_size, input_size))
        hd = _handle_for(x.device.index or 0, input_size, hidden_size, "fp")
        h0 = h0 if (h0 is not None and h0.numel() > 0) else None
        hd.calibrate_hist(W, R, bw, br, x, hist_collectors, bitwidth_config.granularity_list(), h0)
        h = hd.forward_float(W, R, bw, br, x, h0)
        return h, torch.empty(0, dtype=torch.float32, device=x.device)
    if method != "minmax":
        raise ValueError(f"unknown calibration method {calib_method_str!r}")
    if quant_ranges is None:
        raise ValueError("quant_ranges is required for minmax calibration")
    x = _check_tensor(x, "x", torch.float32, (time_steps, batch_size, input_size))
    hd = _handle_for(x.device.index or 0, input_size, hidden_size, "fp")
    h0 = h0 if (h0 is not None and h0.numel() > 0) else None
    h = hd.calibrate_minmax(W, R, bw, br, x, quant_ranges, h0, want_h=True)
    v = torch.empty(0, dtype=torch.float32, device=x.device)
    return h, v


def probe_mma_i8(M=128, N=256, a_in_tmem=False, accumulators=1, mmas=16384, ctas=148, device=0, issuers=1,
                 spinners=3, neighbour_mode=0, commit_every=0):
    """Issue rate of tcgen05.mma kind::i8 for one shape (qgru_probe_mma_i8_ex): returns
    (SM cycles per MMA in a back-to-back chain of one issuing thread, aggregate 1e12 int8 ops/s
    over `ctas` SMs and `issuers` issuing warps); `spinners` neighbour warps wait (mode 0), compute (1) or
    load from shared memory (2), drain tensor memory (3), store to shared memory (4) or keep bulk
    copies from global into shared memory in flight (5; `probe_last_bulk_rate()` then gives their
    bytes per clock) beside them; + 256: pseudo-random operand bytes instead of zeros."""
    cyc, tops = C.c_double(), C.c_double()
    st = _cabi.lib().qgru_probe_mma_i8_commits(int(device), int(M), int(N), int(bool(a_in_tmem)), int(accumulators),
                                               int(mmas), int(ctas), int(issuers), int(spinners), int(neighbour_mode),
                                               int(commit_every), C.byref(cyc), C.byref(tops))
    _cabi.check(st, "qgru_probe_mma_i8_commits")
    return cyc.value, tops.value


def probe_last_bulk_rate():
    """Bytes per SM clock the bulk copies of CTA 0 moved in the last neighbour_mode 5 probe."""
    return float(_cabi.lib().qgru_probe_last_bulk_rate())
