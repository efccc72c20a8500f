"""Seeded synthetic workloads: the five benchmark configurations of the quantized GRU forward.

No dataset is involved anywhere: inputs, weights and calibration batches are drawn from seeded
numpy generators with the shapes and distributions the benchmark configurations name
(weights like ``QuantGRU.reset_parameters``, pytorch/quant_gru.py:1296-1300 of the reference:
uniform in +-1/sqrt(H)).  bench.py and the tests build their problems from this one module, so
that a test of "the benchmark's configuration 2" runs exactly what the benchmark times.
"""
import numpy as np

from . import _cabi
from . import params as params_mod

# name: (I, H, B per GPU-unit, T, bidirectional, bit-width configuration, x distribution,
#        calibration batches)
WORKLOADS = {
    "cfg1": (64, 128, 32, 50, False, "sym8_tensor", "normal", 8),
    "cfg2": (256, 512, 256, 200, True, "cfg2", "normal", 16),
    "cfg3": (128, 256, 4096, 100, False, "cfg3", "outliers", 16),
    "cfg4": (1024, 1024, 64, 1000, False, "sym8_tensor", "normal05", 4),
    "cfg5": (80, 256, 1, 16000, False, "cfg5", "ar1", 4),
}
# calibration method of each workload: (method, percentile)
CALIBRATION = {"cfg1": ("minmax", 0.0), "cfg2": ("minmax", 0.0), "cfg3": ("percentile", 99.9),
               "cfg4": ("sqnr", 0.0), "cfg5": ("minmax", 0.0)}


def gen_x(rng, T, B, I, dist="normal", sigma=1.0):
    """One input batch [T, B, I] fp32 of the named distribution."""
    if dist == "normal":
        return (rng.standard_normal((T, B, I)) * sigma).astype(np.float32)
    if dist == "normal05":   # N(0, 0.5)
        return (rng.standard_normal((T, B, I)) * 0.5).astype(np.float32)
    if dist == "outliers":   # N(0,1) with 1 % of the entries scaled by 8
        x = rng.standard_normal((T, B, I))
        x = np.where(rng.random((T, B, I)) < 0.01, x * 8.0, x)
        return x.astype(np.float32)
    if dist == "ar1":        # per-channel AR(1), coefficient 0.9, unit stationary variance
        x = np.zeros((T, B, I))
        prev = rng.standard_normal((B, I))
        for t in range(T):
            prev = 0.9 * prev + np.sqrt(1 - 0.81) * rng.standard_normal((B, I))
            x[t] = prev
        return x.astype(np.float32)
    if dist == "uniform":    # the reference's own test input range
        return rng.uniform(-0.7, 0.8, (T, B, I)).astype(np.float32)
    raise ValueError(dist)


def gen_weights(rng, I, H):
    """W [I,3H], R [H,3H], bw, br [3H] in the reference's (z, r, n) column layout."""
    k = 1.0 / np.sqrt(H)
    W = rng.uniform(-k, k, (I, 3 * H)).astype(np.float32)
    R = rng.uniform(-k, k, (H, 3 * H)).astype(np.float32)
    bw = rng.uniform(-k, k, 3 * H).astype(np.float32)
    br = rng.uniform(-k, k, 3 * H).astype(np.float32)
    return W, R, bw, br


def config_named(name):
    """Bit-width configurations of the benchmark workloads and the variations the tests add."""
    c = params_mod.OperatorQuantConfig()
    acts = [n for n in _cabi.OPS if n not in params_mod.WEIGHT_OPS]
    if name == "default":
        return c
    if name == "sym8_tensor":      # config 1 / 4: all 8 bit symmetric, per-tensor weights
        c.set_all_bitwidth(8, True)
        for n in params_mod.WEIGHT_OPS:
            c.granularity[n] = _cabi.PER_TENSOR
        return c
    if name == "cfg2":             # per-channel W, asymmetric activations, 16-bit gate outputs
        for n in acts:
            c.symmetric[n] = False
        for n in ("update_gate_output", "reset_gate_output", "new_gate_output"):
            c.bits[n] = 16
        return c
    if name == "cfg3":             # per-gate weights, everything else 8 bit symmetric
        c.set_all_bitwidth(8, True)
        c.granularity["W"] = c.granularity["R"] = _cabi.PER_GATE
        return c
    if name == "cfg5":             # 4-bit per-channel weights, asymmetric 8-bit activations
        for n in acts:
            c.symmetric[n] = False
        c.bits["W"] = c.bits["R"] = 4
        return c
    if name == "pot2":
        c.set_all_bitwidth(8, True)
        c.use_pot2 = True
        return c
    if name == "pot2_asym":
        c.use_pot2 = True
        return c
    if name == "ih16":             # 16-bit linear outputs (int16 storage of W*x + bw)
        c.bits["weight_ih_linear"] = c.bits["weight_hh_linear"] = 16
        return c
    if name == "wide16":           # every activation 16 bit
        c.set_all_bitwidth(16, False)
        for n in params_mod.WEIGHT_OPS:
            c.bits[n] = 8
        return c
    if name == "gate_in16":        # 16-bit gate inputs: segment search instead of tables
        for n in ("update_gate_input", "reset_gate_input", "new_gate_input"):
            c.bits[n] = 16
        return c
    if name == "unsigned_x":
        c.unsigned["x"] = True
        c.symmetric["x"] = False
        return c
    raise ValueError(name)


def workload_weights(name):
    """Seeded float weights of every direction of a workload."""
    I, H, _, _, bidir = WORKLOADS[name][:5]
    base = 1000 + int(name[3:]) * 10
    return [gen_weights(np.random.default_rng(base + d), I, H) for d in range(2 if bidir else 1)]


def workload_calibration_batch(name, k, rows=None):
    """Calibration batch k of a workload (the unit shape unless `rows` says otherwise)."""
    I, _, B, T, _, _, xdist, _ = WORKLOADS[name]
    return gen_x(np.random.default_rng(100 * int(name[3:]) + k), T, rows or B, I, xdist)


def workload_input(name, rank, rows):
    """The timed input of one rank: [T, rows, I] fp32."""
    I, _, _, T, _, _, xdist, _ = WORKLOADS[name]
    return gen_x(np.random.default_rng(int(name[3:]) + 7919 * rank), T, rows, I, xdist)


def calibrate_workload(handle, name, direction, weights_dev, to_device, n_calib=None, rows=None):
    """Run a workload's calibration on `handle` and return its GRUQuantParams.

    weights_dev: (W, R, bw, br) device tensors of this direction; to_device: numpy -> device
    tensor.  The reverse direction calibrates on the time-flipped batches, as the reference's
    module feeds it (pytorch/quant_gru.py:2143-2158)."""
    method, pct = CALIBRATION[name]
    cfg = config_named(WORKLOADS[name][5])
    H = WORKLOADS[name][1]
    n = n_calib or WORKLOADS[name][7]
    W, R, bw, br = weights_dev
    ranges = params_mod.Ranges(H)
    hist = params_mod.Histograms(H, device=handle.device) if method != "minmax" else None
    for k in range(n):
        xc = to_device(workload_calibration_batch(name, k, rows))
        if direction == 1:
            xc = xc.flip(0).contiguous()
        if hist is None:
            handle.calibrate_minmax(W, R, bw, br, xc, ranges)
        else:
            handle.calibrate_hist(W, R, bw, br, xc, hist, cfg.granularity_list())
    if hist is None:
        return params_mod.GRUQuantParams.from_ranges(ranges, cfg)
    qp = params_mod.GRUQuantParams.from_histograms(hist, cfg, method == "percentile", pct)
    hist.close()
    return qp
