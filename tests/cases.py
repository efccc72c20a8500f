"""Seeded test problems: float weights and inputs, MinMax calibration, quantized operands.

A case is built entirely on the CPU with one of the two checkers (the C oracle or the
compiled reference); GPU tests then feed the same quantized operands to the CUDA path.
"""
import importlib
from dataclasses import dataclass

import numpy as np

from __graft_entry__ import PKG_NAME, load_package

load_package()
params_mod = importlib.import_module(PKG_NAME + ".params")
_cabi = importlib.import_module(PKG_NAME + "._cabi")
OP = _cabi.OP_INDEX


@dataclass
class Case:
    T: int
    B: int
    I: int
    H: int
    W: np.ndarray
    R: np.ndarray
    bw: np.ndarray
    br: np.ndarray
    x: np.ndarray
    h0: np.ndarray
    params: object          # params.GRUQuantParams
    wq: list                # [W_q, R_q, bw_q, br_q] int32
    x_q: np.ndarray
    h0_q: np.ndarray


def gen_x(rng, T, B, I, dist="normal", sigma=1.0):
    if dist == "normal":
        return (rng.standard_normal((T, B, I)) * sigma).astype(np.float32)
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
    k = 1.0 / np.sqrt(H)
    W = rng.uniform(-k, k, (I, 3 * H)).astype(np.float32)
    R = rng.uniform(-k, k, (H, 3 * H)).astype(np.float32)
    bw = rng.uniform(-k, k, 3 * H).astype(np.float32)
    br = rng.uniform(-k, k, 3 * H).astype(np.float32)
    return W, R, bw, br


def calibrate_minmax(oracle, T, B, I, H, W, R, bw, br, batches):
    ranges = params_mod.Ranges(H)
    for xb in batches:
        oracle.forward_float(T, B, I, H, W, R, bw, br, xb, None, ranges=ranges)
    return ranges


def make_case(seed, T, B, I, H, checker, config=None, dist="normal", sigma=1.0, calib_batches=2,
              with_h0=False, oracle=None):
    """Build a case; `checker` derives params and quantizes, `oracle` (default: checker if it
    has forward_float, else a fresh Oracle) produces the calibration ranges."""
    from oracle.binding import Oracle
    rng = np.random.default_rng(seed)
    cfg = config or params_mod.OperatorQuantConfig()
    W, R, bw, br = gen_weights(rng, I, H)
    x = gen_x(rng, T, B, I, dist, sigma)
    h0 = (rng.standard_normal((B, H)) * 0.3).astype(np.float32) if with_h0 else None
    fl = oracle or (checker if hasattr(checker, "forward_float") else Oracle())
    crng = np.random.default_rng(seed + 100003)
    ranges = calibrate_minmax(fl, T, B, I, H, W, R, bw, br,
                              [gen_x(crng, T, B, I, dist, sigma) for _ in range(calib_batches)])
    p = params_mod.GRUQuantParams(H, cfg)
    sc = checker.calc_params_from_ranges(ranges, p.c)
    for name, arr in zip(params_mod.WEIGHT_OPS, sc):
        p.scales[name] = arr
    wq = checker.quantize_weights(I, H, W, R, bw, br, p.c, p.scale_list())
    x_q = checker.quantize(x, p.c, OP["x"])
    h0_q = checker.quantize(h0, p.c, OP["h"]) if with_h0 else None
    return Case(T, B, I, H, W, R, bw, br, x, h0, p, wq, x_q, h0_q)


def config_named(name):
    """Bit-width configurations used across the tests (the benchmark configurations and variations)."""
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
    if name == "wide16":           # every activation 16 bit: generic int32 path
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
