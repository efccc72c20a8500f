"""Histogram calibration (Percentile / SQNR): the oracle against the compiled reference, the
product's host function against the oracle.  CPU only.

The collector restated in the oracle follows the reference's GPU collector, which cannot run
here; it is compared with the reference's CPU HistogramCollector, whose bin arithmetic differs
in operand form only (division instead of multiplication by the inverse width): totals and
ranges must be equal, and no more than a few values in 100 000 may sit in a neighbouring bin."""
import ctypes as C
import importlib

import numpy as np
import pytest

from __graft_entry__ import PKG_NAME
import tests.cases  # noqa: F401  (loads the package)

_cabi = importlib.import_module(PKG_NAME + "._cabi")


class _Op:
    def __init__(self, bits, is_unsigned, symmetric):
        self.bits, self.is_unsigned, self.symmetric = bits, is_unsigned, symmetric


def _random_hist(rng, kind):
    bins = 2048
    if kind == "normal":
        data = rng.normal(0.1, 1.3, 40000).astype(np.float32)
    elif kind == "sigmoid":
        data = (1 / (1 + np.exp(-rng.normal(0, 3, 40000)))).astype(np.float32)
    elif kind == "outliers":
        data = rng.normal(0, 1, 40000).astype(np.float32)
        data[rng.integers(0, data.size, 400)] *= 8
    elif kind == "positive":
        data = np.abs(rng.normal(0, 0.4, 40000)).astype(np.float32)
    else:  # sparse weights-like: few samples
        data = rng.normal(0, 0.05, 256).astype(np.float32)
    mn, mx = float(data.min()), float(data.max())
    counts, _ = np.histogram(data, bins=bins, range=(mn, mx))
    return counts.astype(np.float32), mn, mx, data.size


OPS = [_Op(8, 0, 1), _Op(8, 0, 0), _Op(8, 1, 0), _Op(8, 1, 1), _Op(16, 0, 0), _Op(16, 1, 0), _Op(4, 0, 1),
       _Op(4, 0, 0), _Op(12, 0, 1)]


@pytest.mark.parametrize("use_percentile", [True, False])
@pytest.mark.parametrize("pot2", [False, True])
def test_oracle_histogram_params_equal_reference(oracle, reference, use_percentile, pot2):
    rng = np.random.default_rng(5 + 2 * use_percentile + pot2)
    checked = 0
    for kind in ("normal", "sigmoid", "outliers", "positive", "sparse"):
        counts, mn, mx, total = _random_hist(rng, kind)
        for op in OPS:
            for pct in ((99.9, 99.99, 100.0) if use_percentile else (99.99,)):
                a = oracle.calibrate_from_histogram(counts, mn, mx, total, op, pot2, use_percentile, pct)
                b = reference.calibrate_from_histogram(counts, mn, mx, total, op, pot2, use_percentile, pct)
                assert a == b, (kind, op.__dict__, pct, a, b)
                checked += a is not None
    assert checked > 40


@pytest.mark.parametrize("use_percentile", [True, False])
def test_product_histogram_params_equal_oracle(oracle, use_percentile):
    lib = _cabi.lib()
    rng = np.random.default_rng(17 + use_percentile)
    for kind in ("normal", "sigmoid", "outliers", "positive", "sparse"):
        counts, mn, mx, total = _random_hist(rng, kind)
        for op in OPS:
            for pot2 in (0, 1):
                want = oracle.calibrate_from_histogram(counts, mn, mx, total, op, pot2, use_percentile, 99.9)
                o = _cabi.Op(0.0, 0, op.bits, op.is_unsigned, op.symmetric, 0)
                rc = lib.qgru_calibrate_from_histogram(
                    counts.ctypes.data_as(C.POINTER(C.c_float)), counts.size, mn, mx, total, pot2,
                    int(use_percentile), 99.9, C.byref(o))
                got = None if rc else (float(np.float32(o.scale)), int(o.zero_point))
                assert got == want, (kind, op.__dict__, pot2, got, want)


def test_histogram_argument_errors():
    lib = _cabi.lib()
    counts = np.zeros(16, np.float32)
    o = _cabi.Op(0.0, 0, 8, 0, 1, 0)
    ptr = counts.ctypes.data_as(C.POINTER(C.c_float))
    assert lib.qgru_calibrate_from_histogram(None, 16, 0.0, 1.0, 10, 0, 1, 99.9, C.byref(o)) == _cabi.QGRU_ERR_BAD_ARG
    # an empty histogram is "not ready" (Histogram::is_valid is false in the reference)
    assert lib.qgru_calibrate_from_histogram(ptr, 16, 0.0, 1.0, 0, 0, 1, 99.9, C.byref(o)) == _cabi.QGRU_ERR_NOT_READY


def test_oracle_collector_against_reference_cpu_collector(oracle, reference):
    """Several batches with growing range: same range, same total, same counts up to values
    that sit exactly on a bin edge."""
    rng = np.random.default_rng(23)
    for trial in range(4):
        a, b = oracle.hist_new(2048), reference.hist_new(2048)
        scale = 1.0
        for batch in range(5):
            data = (rng.normal(0.2 * trial, scale, 30000)).astype(np.float32)
            a.collect(data)
            b.collect(data)
            scale *= 1.0 if batch % 2 else 1.6          # every other batch widens the range
        ca, mna, mxa, ta = a.get()
        cb, mnb, mxb, tb = b.get()
        assert (mna, mxa, ta) == (mnb, mxb, tb)
        assert ca.sum() == cb.sum() == ta
        assert np.abs(ca - cb).sum() <= 2e-4 * ta, np.abs(ca - cb).sum()


def test_oracle_collector_degenerate_inputs(oracle):
    """Constant tensors get the +-0.5 range, non-finite values are skipped."""
    h = oracle.hist_new(64)
    h.collect(np.full(100, 3.0, np.float32))
    counts, mn, mx, total = h.get()
    assert (mn, mx, total) == (2.5, 3.5, 100) and counts.sum() == 100
    h2 = oracle.hist_new(64)
    h2.collect(np.array([0.0, 1.0, np.inf, np.nan, -np.inf, 0.5], np.float32))
    counts, mn, mx, total = h2.get()
    assert (mn, mx) == (0.0, 1.0) and counts.sum() == 3 and total == 6


def test_golden_histogram_params(oracle):
    """Known answers from the compiled reference (tests/golden/hist/hist_calibration.npz, written by
    tests/golden/make_golden.py): the oracle and the product's host function reproduce them on
    machines without the reference tree."""
    import importlib.util
    import os
    here = os.path.dirname(os.path.abspath(__file__))
    spec = importlib.util.spec_from_file_location("make_golden", os.path.join(here, "golden", "make_golden.py"))
    mg = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mg)
    d = np.load(os.path.join(here, "golden", "hist", "hist_calibration.npz"))
    hists = mg.hist_inputs(int(d["seed"]))
    lib = _cabi.lib()
    assert len(d["rows"]) >= 200
    for h_idx, o_idx, pot2, method, pct, scale_bits, zp in d["rows"]:
        counts, mn, mx, total = hists[int(h_idx)]
        bits, uns, sym = mg.HIST_OPS[int(o_idx)]
        want = (float(np.uint32(scale_bits).view(np.float32)), int(zp))
        got = oracle.calibrate_from_histogram(counts, mn, mx, total, _Op(bits, uns, sym), int(pot2), int(method),
                                              pct or 99.99)
        assert got == want, (h_idx, o_idx, pot2, method, pct, got, want)
        o = _cabi.Op(0.0, 0, bits, uns, sym, 0)
        rc = lib.qgru_calibrate_from_histogram(counts.ctypes.data_as(C.POINTER(C.c_float)), counts.size, mn, mx,
                                               total, int(pot2), int(method), pct or 99.99, C.byref(o))
        assert rc == 0 and (float(np.float32(o.scale)), int(o.zero_point)) == want
