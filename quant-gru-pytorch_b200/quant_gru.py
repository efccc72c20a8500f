"""``QuantGRU``: the nn.GRU-compatible module of the reference (pytorch/quant_gru.py:1060-2400),
restricted to the inference hot path and running on libqgru_b200.so.

What is kept, with the reference's names and meaning: the constructor signature and parameter
names (``weight_ih_l0`` ... in PyTorch's (r, z, n) gate order), ``batch_first``,
``bidirectional``, ``use_quantization``, ``calibrating`` + ``finalize_calibration`` (MinMax),
``load_bitwidth_config`` / ``set_all_bitwidth``, ``forward`` (float mode, calibration mode,
quantized mode with ``quant_storage_dtype="int32"``: the integer path, or ``"float32"``: the
float-storage path with real sigmoid / tanh, both in eval mode), ``forward_quantized`` (int32 in / out),
``export_quant_params`` / ``load_quant_params``.

What differs by design: each direction owns a ``gru_ops.Handle`` whose packed weights are
re-quantized only when a parameter tensor or the quant params change (the reference
re-quantizes weights and regenerates LUTs on every call); the reverse direction runs on the
same input with reversed time indexing instead of two ``flip`` copies; the two directions
are queued on two CUDA streams.  Training: in train() mode with gradients enabled, forward
runs through an autograd function whose backward is qgru_backward - the fp32 GRU in float mode,
and with use_quantization the quantized forward in training mode (float-storage path, or the
integer path with quant_storage_dtype="int32") with its clamp masks as straight-through
estimators (QAT).  ONNX and AIMET hooks are not
built.
"""
import json
import math

import torch
from torch import nn

from . import gru_ops
from .params import GRUQuantParams, Histograms, OperatorQuantConfig, Ranges


def reorder_weights_pytorch_to_haste(w):
    """(r, z, n) -> (z, r, n) along dim 0 (pytorch/quant_gru.py:617-639); self-inverse."""
    h3 = w.shape[0] // 3
    return torch.cat([w[h3:2 * h3], w[:h3], w[2 * h3:]], 0).contiguous()


def convert_weights_to_haste_format(weight_ih, weight_hh, bias_ih, bias_hh, hidden_size, device):
    """[3H, I] / [3H, H] PyTorch weights -> W [I, 3H], R [H, 3H], bw, br [3H] in (z, r, n) order
    (pytorch/quant_gru.py:661-712); missing biases become zeros."""
    W = reorder_weights_pytorch_to_haste(weight_ih.detach().to(device, torch.float32)).t().contiguous()
    R = reorder_weights_pytorch_to_haste(weight_hh.detach().to(device, torch.float32)).t().contiguous()
    if bias_ih is not None and bias_hh is not None:
        bw = reorder_weights_pytorch_to_haste(bias_ih.detach().to(device, torch.float32))
        br = reorder_weights_pytorch_to_haste(bias_hh.detach().to(device, torch.float32))
    else:
        bw = torch.zeros(3 * hidden_size, device=device, dtype=torch.float32)
        br = torch.zeros(3 * hidden_size, device=device, dtype=torch.float32)
    return W, R, bw, br


class _FloatGRUFunction(torch.autograd.Function):
    """One direction of the fp32 GRU with its backward pass (the reference's GRUFunction,
    pytorch/quant_gru.py:760-1058, float mode): forward keeps h and the gate buffer v, backward
    is qgru_backward.  Inputs in haste layout: x [T,B,I], W [I,3H], R [H,3H], bw, br [3H],
    h0 [B,H]; returns h [(T+1),B,H] (slot 0 = h0)."""

    @staticmethod
    def forward(ctx, handle, x, W, R, bw, br, h0):
        h, v = handle.forward_float(W, R, bw, br, x, h0, want_v=True)
        ctx.handle = handle
        ctx.save_for_backward(x, W, R, h, v)
        return h

    @staticmethod
    def backward(ctx, dh_all):
        x, W, R, h, v = ctx.saved_tensors
        dh_all = dh_all.contiguous()
        # the gradient of slot 0 (h0 passed through as an output) is added to what flows back to h0
        dx, dW, dR, dbw, dbr, dh0 = ctx.handle.backward(W, R, x, dh_all, h, v)
        return None, dx, dW, dR, dbw, dbr, dh0 + dh_all[0]


class _QuantGRUFunction(torch.autograd.Function):
    """One direction of quantization-aware training (the reference's GRUFunction with
    use_quantization and float32 storage, pytorch/quant_gru.py:826-1050): forward is the
    float-storage quantized forward in training mode (gate buffer and clamp masks kept),
    backward differentiates through the dequantized quantized tensors with the masks as
    straight-through estimators (qgru_backward)."""

    @staticmethod
    def forward(ctx, handle, qp, int_storage, x, W, R, bw, br, h0):
        handle.set_params(qp)
        handle.set_weights_f32(W, R, bw, br)
        # float32 storage: float requantization, real sigmoid / tanh; int32 storage: the integer
        # path (piecewise-linear gates) in training mode
        h, v, x_q, masks = handle.forward_fstorage_train(W, R, bw, br, x, h0, int_storage=int_storage)
        Wd, Rd, _, _ = handle.get_weights_dequantized()
        xd = handle.dequantize_f32(x_q.to(torch.float32), "x")
        ctx.handle, ctx.masks = handle, masks
        ctx.save_for_backward(xd, Wd, Rd, h, v)
        return h

    @staticmethod
    def backward(ctx, dh_all):
        xd, Wd, Rd, h, v = ctx.saved_tensors
        dh_all = dh_all.contiguous()
        dx, dW, dR, dbw, dbr, dh0 = ctx.handle.backward(Wd, Rd, xd, dh_all, h, v, masks=ctx.masks)
        return None, None, None, dx, dW, dR, dbw, dbr, dh0 + dh_all[0]


class _Direction:
    """Per-direction run-time state: handle, haste-layout weights, what the handle holds."""

    def __init__(self):
        self.handle = None
        self.weights = None
        self.weights_key = None
        self.loaded_key = None
        self.stream = None


class QuantGRU(nn.Module):
    def __init__(self, input_size, hidden_size, num_layers=1, bias=True, batch_first=False,
                 dropout=0.0, bidirectional=False, use_quantization=False, use_pot2_scale=False,
                 quant_storage_dtype="float32"):
        super().__init__()
        if num_layers != 1:
            raise NotImplementedError("only num_layers=1 is supported")
        if dropout > 0:
            raise NotImplementedError("dropout is not supported")
        if quant_storage_dtype not in ("float32", "int32"):
            raise ValueError(f"quant_storage_dtype must be 'float32' or 'int32', got {quant_storage_dtype}")
        self.input_size, self.hidden_size, self.num_layers = input_size, hidden_size, num_layers
        self.bias, self.batch_first, self.dropout = bias, batch_first, dropout
        self.bidirectional = bidirectional
        self.num_directions = 2 if bidirectional else 1
        self.use_quantization = use_quantization
        self.quant_storage_dtype = quant_storage_dtype
        suffixes = [""] + (["_reverse"] if bidirectional else [])
        for s in suffixes:
            setattr(self, "weight_ih_l0" + s, nn.Parameter(torch.empty(3 * hidden_size, input_size)))
            setattr(self, "weight_hh_l0" + s, nn.Parameter(torch.empty(3 * hidden_size, hidden_size)))
            if bias:
                setattr(self, "bias_ih_l0" + s, nn.Parameter(torch.empty(3 * hidden_size)))
                setattr(self, "bias_hh_l0" + s, nn.Parameter(torch.empty(3 * hidden_size)))
            else:
                self.register_parameter("bias_ih_l0" + s, None)
                self.register_parameter("bias_hh_l0" + s, None)
        self.reset_parameters()
        self._bitwidth_config = OperatorQuantConfig()
        self._bitwidth_config.use_pot2 = bool(use_pot2_scale)
        self.calibration_method = "minmax"
        self.percentile_value = 100.0
        self.calibrating = False
        self.quant_ranges = self.quant_params = None
        self.quant_ranges_reverse = self.quant_params_reverse = None
        self.hist_collectors = self.hist_collectors_reverse = None
        self._quant_params_dirty = False
        self._dirs = [_Direction() for _ in suffixes]

    # ------------------------------------------------------------------ configuration
    @property
    def use_pot2_scale(self):
        return self._bitwidth_config.use_pot2

    @use_pot2_scale.setter
    def use_pot2_scale(self, v):
        self._bitwidth_config.use_pot2 = bool(v)
        self._quant_params_dirty = True

    def reset_parameters(self):
        stdv = 1.0 / math.sqrt(self.hidden_size)
        for p in self.parameters():
            nn.init.uniform_(p, -stdv, stdv)

    def load_bitwidth_config(self, config_file, verbose=False):
        if self.is_calibrated():
            return  # as the reference: ignored once params exist (pytorch/quant_gru.py:1389-1397)
        cfg = OperatorQuantConfig.from_json(config_file)
        self.use_quantization = not cfg.disable_quantization
        self._bitwidth_config = cfg
        self._quant_params_dirty = True

    def set_all_bitwidth(self, bitwidth=8, is_symmetric=True, verbose=False):
        self._bitwidth_config.set_all_bitwidth(bitwidth, is_symmetric)
        self._quant_params_dirty = True

    def is_calibrated(self):
        if self.bidirectional:
            return self.quant_params is not None and self.quant_params_reverse is not None
        return self.quant_params is not None

    def reset_calibration(self):
        self.quant_ranges = self.quant_params = None
        self.quant_ranges_reverse = self.quant_params_reverse = None
        self.hist_collectors = self.hist_collectors_reverse = None
        self._quant_params_dirty = False

    def _check_method(self):
        if self.calibration_method not in ("minmax", "sqnr", "percentile"):
            raise ValueError(f"calibration_method must be 'minmax', 'sqnr' or 'percentile', "
                             f"got {self.calibration_method!r}")

    def finalize_calibration(self, verbose=False):
        """Ranges (minmax) or histograms (sqnr / percentile) -> quant params and LUTs
        (pytorch/quant_gru.py finalize_calibration)."""
        self._check_method()
        if self.calibration_method == "minmax":
            if self.quant_ranges is None or (self.bidirectional and self.quant_ranges_reverse is None):
                raise RuntimeError("no calibration data: set calibrating=True and call forward() first")
            self.quant_params = gru_ops.calculate_gru_quantitative_parameters(self.quant_ranges, self._bitwidth_config)
            if self.bidirectional:
                self.quant_params_reverse = gru_ops.calculate_gru_quantitative_parameters(
                    self.quant_ranges_reverse, self._bitwidth_config)
        else:
            if self.hist_collectors is None or (self.bidirectional and self.hist_collectors_reverse is None):
                raise RuntimeError("no calibration data: set calibrating=True and call forward() first")
            pct = self.calibration_method == "percentile"
            self.quant_params = gru_ops.calculate_gru_quantitative_parameters_from_histograms(
                self.hist_collectors, self._bitwidth_config, pct, self.percentile_value)
            if self.bidirectional:
                self.quant_params_reverse = gru_ops.calculate_gru_quantitative_parameters_from_histograms(
                    self.hist_collectors_reverse, self._bitwidth_config, pct, self.percentile_value)
        self._quant_params_dirty = False

    # ---------------------------------------------------------- quant-param JSON files
    def export_quant_params(self, path):
        """Write the reference's quant-param JSON layout (pytorch/quant_gru.py:4252-4330)."""
        if not self.is_calibrated():
            raise RuntimeError("QuantGRU not calibrated")
        doc = {"model_info": {"input_size": self.input_size, "hidden_size": self.hidden_size,
                              "bias": self.bias, "batch_first": self.batch_first,
                              "bidirectional": self.bidirectional,
                              "use_pot2_scale": bool(self._bitwidth_config.use_pot2)},
               "operators": self.quant_params.to_export_dict()}
        if self.bidirectional:
            doc["operators_reverse"] = self.quant_params_reverse.to_export_dict()
        with open(path, "w", encoding="utf-8") as f:
            json.dump(doc, f, indent=2)

    def load_quant_params(self, path):
        with open(path, "r", encoding="utf-8") as f:
            doc = json.load(f)
        info = doc.get("model_info", {})
        if info.get("hidden_size", self.hidden_size) != self.hidden_size or \
                info.get("input_size", self.input_size) != self.input_size:
            raise ValueError("quant-param file was exported for a different input/hidden size")
        if bool(info.get("bidirectional", False)) != self.bidirectional:   # pytorch/quant_gru.py:4379-4383
            raise ValueError(f"bidirectional mismatch: file {info.get('bidirectional')}, module {self.bidirectional}")
        if "operators" not in doc:
            raise ValueError(f"unsupported quant-param file: no 'operators' (has {list(doc)})")
        pot2 = bool(info.get("use_pot2_scale", False))
        self.quant_params = GRUQuantParams.from_export_dict(doc["operators"], self.hidden_size, pot2)
        if self.bidirectional:
            if "operators_reverse" not in doc:
                raise ValueError("bidirectional module needs 'operators_reverse' in the file")
            self.quant_params_reverse = GRUQuantParams.from_export_dict(doc["operators_reverse"],
                                                                        self.hidden_size, pot2)
            # both directions quantize the same input (pytorch/quant_gru.py:4428-4433)
            fi, ri = doc["operators"].get("input", {}), doc["operators_reverse"].get("input", {})
            for field in ("multiplier", "shift", "zero_point"):
                if (field in fi or field in ri) and fi.get(field) != ri.get(field):
                    raise ValueError(f"operators.input and operators_reverse.input differ in {field}")
        self._bitwidth_config = self.quant_params.config()
        self.use_quantization = True
        self._quant_params_dirty = False

    # ----------------------------------------------------------------- run-time plumbing
    def _params_of(self, d):
        suffix = "_reverse" if d == 1 else ""
        return [getattr(self, n + suffix) for n in ("weight_ih_l0", "weight_hh_l0", "bias_ih_l0", "bias_hh_l0")]

    def _direction(self, d, device):
        st = self._dirs[d]
        if st.handle is None or st.handle.device != (device.index or 0):
            st.handle = gru_ops.Handle(self.input_size, self.hidden_size, device=device.index or 0)
            st.stream = torch.cuda.Stream(device=device)
            if self.bidirectional:
                # the two directions run side by side: each persistent kernel takes half the SMs
                sms = torch.cuda.get_device_properties(device).multi_processor_count
                st.handle.set_option("sm_limit", max(1, sms // 2))
            st.weights_key = st.loaded_key = None
        ps = self._params_of(d)
        key = tuple((p.data_ptr(), p._version) if p is not None else None for p in ps)
        if key != st.weights_key:
            st.weights = convert_weights_to_haste_format(*ps, self.hidden_size, device)
            st.weights_key = key
            st.loaded_key = None
        return st

    def _ready_quant(self, d, device):
        st = self._direction(d, device)
        qp = self.quant_params_reverse if d == 1 else self.quant_params
        key = (st.weights_key, id(qp), qp.to_bytes())
        if key != st.loaded_key:
            st.handle.set_params(qp)
            st.handle.set_weights_f32(*st.weights)
            st.loaded_key = key
        return st

    def _split_h0(self, hx, batch, device, dtype):
        if hx is None:
            return [None] * self.num_directions
        want = (self.num_directions, batch, self.hidden_size)
        if tuple(hx.shape) != want:
            raise ValueError(f"hx must have shape {list(want)}, got {list(hx.shape)}")
        hx = hx.to(device=device, dtype=dtype)
        return [hx[d].contiguous() for d in range(self.num_directions)]

    def _has_calibration_data(self):
        have = self.quant_ranges if self.calibration_method == "minmax" else self.hist_collectors
        have_r = self.quant_ranges_reverse if self.calibration_method == "minmax" else self.hist_collectors_reverse
        return have is not None and (not self.bidirectional or have_r is not None)

    def _ensure_quant_ready(self):
        """Quant params are (re)derived whenever calibration data or the bit-width configuration
        changed since they were last computed, as the reference's forward does
        (pytorch/quant_gru.py:2106-2125): the documented flow `calibrating=True; forward();
        calibrating=False; forward()` needs no explicit finalize_calibration() for any method."""
        if self._quant_params_dirty and self._has_calibration_data():
            self.finalize_calibration()
        elif not self.is_calibrated():
            if self.quant_ranges is not None or self.hist_collectors is not None:
                self.finalize_calibration()   # raises if the data of the chosen method is missing
            else:
                raise RuntimeError("quantization is enabled but the module is not calibrated: set "
                                   "calibrating=True, run forward() on calibration data, then "
                                   "calibrating=False")

    def _combine(self, outs, T):
        """outs[d] = h [(T+1),B,H]; forward slots 1..T are the outputs, reverse slots 0..T-1."""
        of = outs[0][1:]
        hn = outs[0][T:T + 1]
        if not self.bidirectional:
            return of.contiguous(), hn.contiguous()
        orv = outs[1][:T]
        return torch.cat([of, orv], dim=-1), torch.cat([hn, outs[1][0:1]], dim=0)

    def _run_directions(self, fn, device):
        """Queue fn(d, state) for each direction on its own stream, then join."""
        cur = torch.cuda.current_stream(device)
        outs = []
        for d in range(self.num_directions):
            st = self._dirs[d]
            st.stream.wait_stream(cur)
            with torch.cuda.stream(st.stream):
                outs.append(fn(d, st))
        for d in range(self.num_directions):
            cur.wait_stream(self._dirs[d].stream)
        for d in range(self.num_directions):
            self._dirs[d].handle.synchronize()
        return outs

    def _forward_float_train(self, input, hx):
        """Float mode and QAT with autograd: every tensor operation outside the two library calls is a
        torch operation, so gradients reach the module's parameters in their PyTorch layout."""
        x = input.transpose(0, 1) if self.batch_first else input
        device = x.device
        x = x.to(torch.float32).contiguous()
        T, B, _ = x.shape
        H = self.hidden_size
        outs, hns = [], []
        for d in range(self.num_directions):
            st = self._direction(d, device)
            w_ih, w_hh, b_ih, b_hh = self._params_of(d)
            W = reorder_weights_pytorch_to_haste(w_ih.to(torch.float32)).t().contiguous()
            R = reorder_weights_pytorch_to_haste(w_hh.to(torch.float32)).t().contiguous()
            if b_ih is not None and b_hh is not None:
                bw = reorder_weights_pytorch_to_haste(b_ih.to(torch.float32))
                br = reorder_weights_pytorch_to_haste(b_hh.to(torch.float32))
            else:
                bw = torch.zeros(3 * H, device=device)
                br = torch.zeros(3 * H, device=device)
            h0 = hx[d].to(torch.float32).contiguous() if hx is not None else torch.zeros(B, H, device=device)
            xd = x.flip(0).contiguous() if d == 1 else x
            if self.use_quantization:
                qp = self.quant_params_reverse if d == 1 else self.quant_params
                h = _QuantGRUFunction.apply(st.handle, qp, self.quant_storage_dtype == "int32", xd, W, R, bw, br, h0)
                st.loaded_key = None        # the handle was reloaded outside the module's cache
            else:
                h = _FloatGRUFunction.apply(st.handle, xd, W, R, bw, br, h0)
            outs.append(h[1:].flip(0) if d == 1 else h[1:])
            hns.append(h[T:T + 1])
        output = torch.cat(outs, dim=-1) if self.bidirectional else outs[0]
        h_n = torch.cat(hns, dim=0)
        if self.batch_first:
            output = output.transpose(0, 1).contiguous()
        return output, h_n

    # --------------------------------------------------------------------------- forward
    def forward(self, input, hx=None):
        needs_grad = torch.is_grad_enabled() and (input.requires_grad or (hx is not None and hx.requires_grad) or
                                                  any(p.requires_grad for p in self.parameters()))
        if needs_grad and self.training and not self.calibrating:
            if self.use_quantization:
                self._ensure_quant_ready()
            if not input.is_cuda:
                raise ValueError("input must be a CUDA tensor")
            want = (self.num_directions, input.shape[0 if self.batch_first else 1], self.hidden_size)
            if hx is not None and tuple(hx.shape) != want:
                raise ValueError(f"hx must have shape {list(want)}, got {list(hx.shape)}")
            return self._forward_float_train(input, hx)
        with torch.no_grad():
            return self._forward_impl(input, hx)

    def _forward_impl(self, input, hx=None):
        if self.batch_first:
            input = input.transpose(0, 1)
        device = input.device if input.is_cuda else torch.device("cuda", torch.cuda.current_device())
        x = input.to(device=device, dtype=torch.float32).contiguous()
        T, B, _ = x.shape
        h0 = self._split_h0(hx, B, device, torch.float32)

        if self.calibrating:
            self._check_method()
            outs = []
            for d in range(self.num_directions):
                st = self._direction(d, device)
                xd = x.flip(0).contiguous() if d == 1 else x
                if self.calibration_method == "minmax":
                    rng_name = "quant_ranges_reverse" if d == 1 else "quant_ranges"
                    if getattr(self, rng_name) is None:
                        setattr(self, rng_name, Ranges(self.hidden_size))
                    h = st.handle.calibrate_minmax(*st.weights, xd, getattr(self, rng_name), h0[d], want_h=True)
                else:
                    name = "hist_collectors_reverse" if d == 1 else "hist_collectors"
                    if getattr(self, name) is None:
                        setattr(self, name, Histograms(self.hidden_size, device.index or 0))
                    st.handle.calibrate_hist(*st.weights, xd, getattr(self, name),
                                             self._bitwidth_config.granularity_list(), h0[d])
                    h = st.handle.forward_float(*st.weights, xd, h0[d])
                outs.append(torch.cat([h[1:].flip(0), h[0:1]], 0) if d == 1 else h)
            self._quant_params_dirty = True
        elif self.use_quantization:
            self._ensure_quant_ready()
            for d in range(self.num_directions):
                self._ready_quant(d, device)
            if self.quant_storage_dtype == "int32":
                run = lambda d, st: st.handle.forward_f32(x, h0[d], reverse=(d == 1), sync=False)  # noqa: E731
            else:
                run = lambda d, st: st.handle.forward_fstorage(x, h0[d], reverse=(d == 1), sync=False)  # noqa: E731
            outs = self._run_directions(run, device)
        else:
            outs = []
            for d in range(self.num_directions):
                st = self._direction(d, device)
                xd = x.flip(0).contiguous() if d == 1 else x
                h = st.handle.forward_float(*st.weights, xd, h0[d])
                outs.append(torch.cat([h[1:].flip(0), h[0:1]], 0) if d == 1 else h)
        output, h_n = self._combine(outs, T)
        if self.batch_first:
            output = output.transpose(0, 1).contiguous()
        return output, h_n

    @torch.no_grad()
    def forward_quantized(self, input, hx=None):
        """int32 in / int32 out inference (pytorch/quant_gru.py:2318-2380)."""
        if not self.is_calibrated() or self.quant_params is None:
            raise RuntimeError("QuantGRU not calibrated")
        if input.is_floating_point():
            raise TypeError("forward_quantized only accepts already quantized integer input "
                            f"(int in / int out); got dtype={input.dtype}")
        if self.batch_first:
            input = input.transpose(0, 1)
        device = input.device if input.is_cuda else torch.device("cuda", torch.cuda.current_device())
        x_q = input.to(device=device, dtype=torch.int32).contiguous()
        T, B, _ = x_q.shape
        h0 = self._split_h0(hx, B, device, torch.int32)
        for d in range(self.num_directions):
            self._ready_quant(d, device)
        outs = self._run_directions(
            lambda d, st: st.handle.forward_i32(x_q, h0[d], reverse=(d == 1), sync=False), device)
        output, h_n = self._combine(outs, T)
        if self.batch_first:
            output = output.transpose(0, 1).contiguous()
        return output, h_n

    def last_plans(self):
        return [st.handle.describe_plan() if st.handle else "" for st in self._dirs]

    def last_timings(self):
        return [st.handle.last_timing() for st in self._dirs if st.handle]

    def launch_count(self):
        return sum(st.handle.launch_count() for st in self._dirs if st.handle)

    def set_option(self, name, value):
        """Forward a kernel-selection option to every direction's handle (after first use)."""
        for st in self._dirs:
            if st.handle:
                st.handle.set_option(name, value)
