"""TEST INFRASTRUCTURE: seeded problems built on the CPU with one of the two checkers.

A case holds float weights and inputs, MinMax-calibrated quant params and the quantized operands
derived by a checker (the C oracle or the compiled reference); GPU tests feed the same operands
to the CUDA path.  Used by tests/, the smoke test and the CPU legs of bench.py only.
"""
import importlib
import os
import sys
from dataclasses import dataclass

import numpy as np

_ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if _ROOT not in sys.path:
    sys.path.insert(0, _ROOT)
from __graft_entry__ import PKG_NAME, load_package  # noqa: E402

load_package()
params_mod = importlib.import_module(PKG_NAME + ".params")
_cabi = importlib.import_module(PKG_NAME + "._cabi")
_workloads = importlib.import_module(PKG_NAME + ".workloads")
OP = _cabi.OP_INDEX
# the seeded generators and bit-width configurations are the benchmark's own
gen_x, gen_weights, config_named = _workloads.gen_x, _workloads.gen_weights, _workloads.config_named


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
