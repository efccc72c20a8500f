"""Host data model of the quantized GRU: operator configuration, ranges and quant params.

Mirrors the three objects the reference's Python module keeps per direction
(pytorch/lib/gru_interface_binding.cc:1298-1560: ``OperatorQuantConfig``,
``GRUQuantizationRanges``, ``GRUQuantParams``) and the two JSON formats it reads and writes:
the bit-width configuration (pytorch/config/gru_quant_bitwidth_config.json, loader
pytorch/quant_gru.py:1375-1561) and the exported quant-param file
(pytorch/quant_gru.py:3934-3944, 4252-4444).
"""
import ctypes as C
import json

import numpy as np

from . import _cabi
from ._cabi import NUM_OPS, OP_INDEX, OPS, PER_CHANNEL, PER_GATE, PER_TENSOR

# JSON operator name -> C-ABI operator name (pytorch/quant_gru.py:163-187)
JSON_TO_OP = {
    "input": "x", "output": "h", "weight_ih": "W", "weight_hh": "R", "bias_ih": "bw",
    "bias_hh": "br", "weight_ih_linear": "weight_ih_linear", "weight_hh_linear": "weight_hh_linear",
    "update_gate_input": "update_gate_input", "update_gate_output": "update_gate_output",
    "reset_gate_input": "reset_gate_input", "reset_gate_output": "reset_gate_output",
    "new_gate_input": "new_gate_input", "new_gate_output": "new_gate_output",
    "mul_reset_hidden": "mul_reset_hidden", "mul_old_contribution": "mul_old_contribution",
    "mul_new_contribution": "mul_new_contribution",
}
OP_TO_JSON = {v: k for k, v in JSON_TO_OP.items()}
LEGACY_KEYS = {"W": "weight_ih", "R": "weight_hh", "bw": "bias_ih", "br": "bias_hh",
               "x": "input", "h": "output"}
WEIGHT_OPS = ("W", "R", "bw", "br")
GRANULARITY = {"PER_TENSOR": PER_TENSOR, "PER_GATE": PER_GATE, "PER_CHANNEL": PER_CHANNEL}
GRANULARITY_NAME = {v: k for k, v in GRANULARITY.items()}


class OperatorQuantConfig:
    """Bit width, signedness and symmetry of the 17 operators plus weight granularities.

    Defaults are the reference's (include/quantize_bitwidth_config.h:57-86): everything
    8-bit signed except the two sigmoid outputs (unsigned); weights symmetric per-channel;
    activations asymmetric except ``new_gate_output``; affine M+shift rescale.
    """

    def __init__(self):
        self.bits = {n: 8 for n in OPS}
        self.unsigned = {n: n in ("update_gate_output", "reset_gate_output") for n in OPS}
        self.symmetric = {n: n in WEIGHT_OPS or n == "new_gate_output" for n in OPS}
        self.granularity = {n: PER_CHANNEL for n in WEIGHT_OPS}
        self.use_pot2 = False
        self.disable_quantization = False

    def set_all_bitwidth(self, bits=8, is_symmetric=True):
        """QuantGRU.set_all_bitwidth (pytorch/quant_gru.py:1563-1591): one width for every
        operator; weights stay symmetric, activations take ``is_symmetric``; signedness is
        left as it is."""
        if not 1 <= bits <= 32:
            raise ValueError(f"bitwidth must be in range [1, 32], got {bits}")
        for n in OPS:
            self.bits[n] = bits
            self.symmetric[n] = True if n in WEIGHT_OPS else bool(is_symmetric)
        return self

    @classmethod
    def from_json(cls, path_or_dict):
        """Read the reference's bit-width JSON (same keys, legacy aliases, same errors)."""
        data = path_or_dict
        if not isinstance(data, dict):
            with open(path_or_dict, "r", encoding="utf-8") as f:
                data = json.load(f)
        cfg = cls()
        gru = data.get("GRU_config", {})
        default = gru.get("default_config", {})
        cfg.disable_quantization = bool(default.get("disable_quantization", False))
        cfg.use_pot2 = bool(default.get("use_pot2_scale", False))
        ops = {LEGACY_KEYS.get(k, k): v for k, v in gru.get("operator_config", {}).items()}
        unknown = set(ops) - set(JSON_TO_OP)
        if unknown:
            raise ValueError(f"unknown operator fields in bit-width config: {sorted(unknown)}")
        for key, name in JSON_TO_OP.items():
            if key not in ops:
                continue  # missing operators keep the defaults: 8 bit, symmetric
            oc = ops[key]
            bits = oc.get("bitwidth", 8)
            if not 1 <= bits <= 32:
                raise ValueError(f"Invalid bitwidth {bits} for '{key}'. Must be in range [1, 32].")
            cfg.bits[name] = int(bits)
            cfg.symmetric[name] = bool(oc.get("is_symmetric", True))
            cfg.unsigned[name] = bool(oc.get("is_unsigned", cfg.unsigned[name]))
            if name in WEIGHT_OPS:
                g = oc.get("quantization_granularity", "PER_CHANNEL")
                if g not in GRANULARITY:
                    raise ValueError(f"Invalid quantization_granularity '{g}' for '{key}'. "
                                     "Must be one of: PER_TENSOR, PER_GATE, PER_CHANNEL")
                cfg.granularity[name] = GRANULARITY[g]
        # Operators the file omits keep the C++ defaults above: the reference's loader only
        # reports them (pytorch/quant_gru.py:1517-1519) and touches nothing.
        return cfg

    def to_json_dict(self):
        ops = {}
        for key, name in JSON_TO_OP.items():
            ops[key] = {"bitwidth": self.bits[name], "is_symmetric": self.symmetric[name],
                        "is_unsigned": self.unsigned[name]}
            if name in WEIGHT_OPS:
                ops[key]["quantization_granularity"] = GRANULARITY_NAME[self.granularity[name]]
        return {"GRU_config": {"default_config": {"disable_quantization": self.disable_quantization,
                                                  "use_pot2_scale": self.use_pot2},
                               "operator_config": ops}}

    def granularity_list(self):
        """QGRU_PER_* of W, R, bw, br."""
        return [self.granularity[n] for n in WEIGHT_OPS]

    def fill(self, params):
        """Write the configuration fields of a ``_cabi.Params``."""
        params.use_pot2 = int(self.use_pot2)
        for i, n in enumerate(OPS):
            params.op[i].bits = self.bits[n]
            params.op[i].is_unsigned = int(self.unsigned[n])
            params.op[i].symmetric = int(self.symmetric[n])
        for k, n in enumerate(WEIGHT_OPS):
            params.granularity[k] = self.granularity[n]


class Ranges:
    """GRUQuantizationRanges (include/gru_quantization_ranges.h:20-123): running min/max of
    every operator, per channel for W, R, bw, br."""

    def __init__(self, hidden):
        self.hidden = hidden
        self.reset()

    def reset(self):
        big = np.finfo(np.float32).max
        self.min_v = np.full(NUM_OPS, big, np.float32)
        self.max_v = np.full(NUM_OPS, -big, np.float32)
        self.ch_min = {n: np.full(3 * self.hidden, big, np.float32) for n in WEIGHT_OPS}
        self.ch_max = {n: np.full(3 * self.hidden, -big, np.float32) for n in WEIGHT_OPS}

    def struct(self):
        """A ``_cabi.Ranges`` whose pointers alias this object's arrays (keep ``self`` alive)."""
        r = _cabi.Ranges()
        r.hidden = self.hidden
        for i in range(NUM_OPS):
            r.min_v[i] = float(self.min_v[i])
            r.max_v[i] = float(self.max_v[i])
        fp = C.POINTER(C.c_float)
        for n in WEIGHT_OPS:
            setattr(r, "min_" + n, self.ch_min[n].ctypes.data_as(fp))
            setattr(r, "max_" + n, self.ch_max[n].ctypes.data_as(fp))
        return r

    def load(self, r):
        """Take the scalar ranges back from a ``_cabi.Ranges`` (channel arrays are aliased)."""
        for i in range(NUM_OPS):
            self.min_v[i] = r.min_v[i]
            self.max_v[i] = r.max_v[i]

    def merge(self, other):
        """Union of two range sets (used when calibration batches are split over ranks)."""
        self.min_v = np.minimum(self.min_v, other.min_v)
        self.max_v = np.maximum(self.max_v, other.max_v)
        for n in WEIGHT_OPS:
            self.ch_min[n] = np.minimum(self.ch_min[n], other.ch_min[n])
            self.ch_max[n] = np.maximum(self.ch_max[n], other.ch_max[n])

    def as_vector(self):
        return np.concatenate([self.min_v, self.max_v] + [self.ch_min[n] for n in WEIGHT_OPS] +
                              [self.ch_max[n] for n in WEIGHT_OPS])


class Histograms:
    """One direction's histogram collectors (GRUGPUHistogramCollectors,
    include/histogram_gpu.cuh): 2048-bin histograms with range growth for the 13 activation
    operators and, by granularity, per-tensor / per-gate / per-channel ones for W, R, bw, br.
    Counts live on the GPU inside the library."""

    def __init__(self, hidden, device=0, num_bins=2048):
        self.hidden, self.device, self.num_bins = hidden, device, num_bins
        self._lib = _cabi.lib()
        self._h = C.c_void_p()
        _cabi.check(self._lib.qgru_hist_create(C.byref(self._h), device, hidden, num_bins), "qgru_hist_create")

    def close(self):
        if getattr(self, "_h", None) is not None and self._h.value:
            self._lib.qgru_hist_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _ck(self, st, where):
        if st != 0:
            raise RuntimeError(f"{where}: {_cabi.status_string(st)}: "
                               f"{(self._lib.qgru_hist_last_error(self._h) or b'').decode()}")

    def reset(self):
        self._ck(self._lib.qgru_hist_reset(self._h), "qgru_hist_reset")

    def count(self):
        return int(self._lib.qgru_hist_count(self._h))

    def collect(self, index, data):
        """Fold a float32 CUDA tensor into collector ``index`` (GPUHistogramCollector::collect)."""
        import torch
        if not (data.is_cuda and data.dtype == torch.float32 and data.is_contiguous()):
            raise ValueError("data must be a contiguous float32 CUDA tensor")
        stream = C.c_void_p(torch.cuda.current_stream(data.device).cuda_stream)
        self._ck(self._lib.qgru_hist_collect(self._h, int(index), C.c_void_p(data.data_ptr()),
                                             int(data.numel()), stream), "qgru_hist_collect")

    def get(self, index):
        """(counts [num_bins] float32, min, max, total) of collector ``index``."""
        counts = np.zeros(self.num_bins, np.float32)
        mn, mx, tot = C.c_float(), C.c_float(), C.c_int64()
        self._ck(self._lib.qgru_hist_export(self._h, int(index), counts.ctypes.data_as(C.POINTER(C.c_float)),
                                            C.byref(mn), C.byref(mx), C.byref(tot)), "qgru_hist_export")
        return counts, float(mn.value), float(mx.value), int(tot.value)

    def put(self, index, counts, min_val, max_val, total):
        counts = np.ascontiguousarray(counts, np.float32)
        if counts.size != self.num_bins:
            raise ValueError("counts must hold num_bins values")
        self._ck(self._lib.qgru_hist_import(self._h, int(index), counts.ctypes.data_as(C.POINTER(C.c_float)),
                                            float(min_val), float(max_val), int(total)), "qgru_hist_import")

    def is_valid(self):
        return self.get_total(OP["x"]) > 0

    def get_total(self, index):
        tot = C.c_int64()
        self._ck(self._lib.qgru_hist_export(self._h, int(index), None, None, None, C.byref(tot)), "qgru_hist_export")
        return int(tot.value)


class GRUQuantParams:
    """One direction's quant params: the ``_cabi.Params`` POD plus the four per-channel scale
    arrays (GRUQuantParams, include/quantize_param_types.h:100-146)."""

    def __init__(self, hidden, config=None):
        self.hidden = hidden
        self.c = _cabi.Params()
        self.c.hidden = hidden
        (config or OperatorQuantConfig()).fill(self.c)
        self.scales = {n: np.ones(3 * hidden, np.float32) for n in WEIGHT_OPS}

    # ---- construction
    @classmethod
    def from_ranges(cls, ranges, config):
        """calculate_gru_quantitative_parameters (MinMax): ranges + config -> params + LUTs."""
        self = cls(ranges.hidden, config)
        L = _cabi.lib()
        rs = ranges.struct()
        fp = C.POINTER(C.c_float)
        st = L.qgru_calc_params_from_ranges(C.byref(rs), C.byref(self.c),
                                            *[self.scales[n].ctypes.data_as(fp) for n in WEIGHT_OPS])
        _cabi.check(st, "qgru_calc_params_from_ranges")
        return self

    @classmethod
    def from_histograms(cls, hist, config, use_percentile=False, percentile=99.99):
        """calculate_gru_quantitative_parameters_from_histograms: histograms + config -> params +
        LUTs, by Percentile (use_percentile) or by the SQNR search."""
        self = cls(hist.hidden, config)
        fp = C.POINTER(C.c_float)
        st = hist._lib.qgru_calc_params_from_hist(hist._h, int(bool(use_percentile)), float(percentile),
                                                  C.byref(self.c),
                                                  *[self.scales[n].ctypes.data_as(fp) for n in WEIGHT_OPS])
        hist._ck(st, "qgru_calc_params_from_hist")
        return self

    def regenerate_luts(self):
        _cabi.check(_cabi.lib().qgru_generate_luts(C.byref(self.c)), "qgru_generate_luts")

    def scale_list(self):
        return [self.scales[n] for n in WEIGHT_OPS]

    def config(self):
        cfg = OperatorQuantConfig()
        cfg.use_pot2 = bool(self.c.use_pot2)
        for i, n in enumerate(OPS):
            cfg.bits[n] = int(self.c.op[i].bits)
            cfg.unsigned[n] = bool(self.c.op[i].is_unsigned)
            cfg.symmetric[n] = bool(self.c.op[i].symmetric)
        for k, n in enumerate(WEIGHT_OPS):
            cfg.granularity[n] = int(self.c.granularity[k])
        return cfg

    # ---- serialisation (binary, for golden files and worker processes)
    def to_bytes(self):
        return bytes(self.c) + b"".join(self.scales[n].tobytes() for n in WEIGHT_OPS)

    @classmethod
    def from_bytes(cls, blob, hidden):
        self = cls(hidden)
        n = C.sizeof(_cabi.Params)
        C.memmove(C.byref(self.c), blob[:n], n)
        off = n
        for name in WEIGHT_OPS:
            self.scales[name] = np.frombuffer(blob, np.float32, 3 * hidden, off).copy()
            off += 12 * hidden
        return self

    # ---- the reference's exported quant-param JSON
    def to_export_dict(self):
        """The ``operators`` object of export_quant_params (pytorch/quant_gru.py:3934-3944):
        scalar operators export scale / zero_point / real_min / real_max; weight operators
        always export full 3H scale lists tagged PER_CHANNEL.  That is what the reference's
        exporter writes whatever the configured granularity: it looks the granularity up under
        ``weight_ih_granularity_`` (:3788), a name the binding's configuration object does not
        have (its attribute is ``W_granularity_``), and falls back to PER_CHANNEL (:3811-3814);
        tests/golden/ref_export_*.json are files that exporter produced."""
        out = {}
        for i, n in enumerate(OPS):
            o = self.c.op[i]
            uns = bool(o.is_unsigned) and o.bits < 32
            qmin = 0 if uns else -(1 << (o.bits - 1))
            qmax = (1 << o.bits) - 1 if uns else (1 << (o.bits - 1)) - 1
            entry = {"dtype": ("UINT" if uns else "INT") + str(int(o.bits)),
                     "symmetric": bool(o.symmetric)}
            if n in WEIGHT_OPS:
                sc = self.scales[n]
                entry.update(scale=[float(s) for s in sc], zero_point=[0] * len(sc),
                             enc_type="PER_CHANNEL",
                             real_min=[float(s) * qmin for s in sc],
                             real_max=[float(s) * qmax for s in sc])
            else:
                entry.update(scale=float(o.scale), zero_point=int(o.zero_point),
                             enc_type="PER_TENSOR",
                             real_min=float(o.scale) * (qmin - o.zero_point),
                             real_max=float(o.scale) * (qmax - o.zero_point))
            out[OP_TO_JSON[n]] = entry
        return out

    @staticmethod
    def _scale_list(key, entry):
        """The scale values of one exported operator as a list, in the reference's order of
        preference (_parse_runtime_scale_lists, pytorch/quant_gru.py:4008-4045): `scale`
        (scalar or list); else `multiplier` + `shift` (M * 2^-shift each); else the old
        power-of-two fields `n` / `exp2_inv` / `shift` (2^-n each)."""
        def as_list(v):
            return list(v) if isinstance(v, (list, tuple)) else [v]
        if "scale" in entry:
            sc = [float(v) for v in as_list(entry["scale"])]
            if not sc:
                raise ValueError(f"{key}: empty scale")
            if any(v <= 0 for v in sc):
                raise ValueError(f"{key}: every scale must be > 0")
            return sc
        if "multiplier" in entry and "shift" in entry:
            m, sh = as_list(entry["multiplier"]), as_list(entry["shift"])
            if len(m) != len(sh):
                raise ValueError(f"{key}: multiplier and shift differ in length")
            return [float(int(a)) * 2.0 ** (-int(b)) for a, b in zip(m, sh)]
        for old in ("n", "exp2_inv", "shift"):
            if old in entry:
                return [2.0 ** (-int(v)) for v in as_list(entry[old])]
        raise ValueError(f"{key}: no scale / multiplier+shift / power-of-two field")

    @classmethod
    def from_export_dict(cls, ops, hidden, use_pot2=False):
        """Read the ``operators`` object of a quant-param file (_parse_operators_dict,
        pytorch/quant_gru.py:4051-4127).  Weight operators carry 1 (PER_TENSOR), 3 (PER_GATE) or
        3H (PER_CHANNEL, the default) scales; every other operator one scale, given as a scalar
        or a one-element list."""
        self = cls(hidden)
        self.c.use_pot2 = int(use_pot2)
        for key, entry in ops.items():
            n = JSON_TO_OP[LEGACY_KEYS.get(key, key)]
            o = self.c.op[OP_INDEX[n]]
            dt = entry["dtype"].upper()
            o.is_unsigned = int(dt.startswith("UINT"))
            o.bits = int(dt.replace("UINT", "").replace("INT", ""))
            o.symmetric = int(bool(entry.get("symmetric", True)))
            sc = np.asarray(cls._scale_list(key, entry), np.float32)
            if n in WEIGHT_OPS:
                enc = entry.get("enc_type") or "PER_CHANNEL"
                if enc == "PER_TENSOR":
                    sc = np.full(3 * hidden, sc[0], np.float32)
                elif enc == "PER_GATE":
                    if sc.size != 3:
                        raise ValueError(f"{key}: PER_GATE needs 3 scales, got {sc.size}")
                    sc = np.repeat(sc, hidden)
                if sc.size != 3 * hidden:
                    raise ValueError(f"{key}: expected {3 * hidden} scales, got {sc.size}")
                self.scales[n] = np.ascontiguousarray(sc)
                self.c.granularity[WEIGHT_OPS.index(n)] = GRANULARITY.get(enc, PER_CHANNEL)
                o.scale = float(sc[0])
                o.zero_point = 0
            else:
                zp = entry.get("zero_point", 0)
                o.scale = float(sc[0])
                o.zero_point = int(zp[0] if isinstance(zp, (list, tuple)) else zp)
        self.regenerate_luts()
        return self
