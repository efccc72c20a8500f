"""Generate the golden vectors in this directory from the UNMODIFIED reference sources.

Run where the reference tree is present (it is compiled into oracle/_ref by oracle/Makefile):

    python tests/golden/make_golden.py

Each .npz holds one seeded problem: float weights / input / h0, the MinMax ranges fed to
calculateGRUQuantitativeParameters, the quant params it returned (struct bytes + per-channel
scales, LUTs included), the quantized operands from quantitativeWeightCPU / quantize, and the
outputs of the reference's CPU integer forward: h_q (int32, every timestep) and h (float,
quantGRUForwardCPU).  The reference's own tests contain no known-answer vectors, so these are
the fixtures that pin the oracle and the CUDA path on machines without the reference tree."""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from oracle.binding import Oracle, Reference  # noqa: E402
from tests.cases import calibrate_minmax, config_named, gen_weights, gen_x, params_mod, OP  # noqa: E402

CASES = [  # name, seed, T, B, I, H, config, x distribution, with h0
    ("c1_sym8_tensor", 1, 7, 5, 16, 24, "sym8_tensor", "normal", False),
    ("c2_perchannel_asym_gate16", 2, 6, 4, 20, 40, "cfg2", "normal", True),
    ("c3_pergate_outliers", 3, 5, 9, 12, 16, "cfg3", "outliers", False),
    ("c5_w4bit_ar1_batch1", 5, 12, 1, 10, 24, "cfg5", "ar1", False),
    ("pot2_sym", 6, 4, 3, 8, 8, "pot2", "normal", True),
    ("pot2_asym", 7, 3, 2, 9, 16, "pot2_asym", "uniform", False),
    ("all16_generic", 8, 4, 3, 12, 16, "wide16", "normal", True),
    ("gate_in16_segment_search", 9, 5, 2, 8, 24, "gate_in16", "normal", False),
    ("ih16", 10, 3, 6, 24, 8, "ih16", "normal", False),
    ("unsigned_x", 11, 2, 7, 5, 40, "unsigned_x", "uniform", False),
    ("single_step_single_row", 12, 1, 1, 1, 1, "default", "normal", False),
]


def main():
    ref, orc = Reference(), Oracle()
    for name, seed, T, B, I, H, cfg_name, dist, with_h0 in CASES:
        rng = np.random.default_rng(seed)
        W, R, bw, br = gen_weights(rng, I, H)
        x = gen_x(rng, T, B, I, dist)
        h0 = (rng.standard_normal((B, H)) * 0.3).astype(np.float32) if with_h0 else None
        ranges = calibrate_minmax(orc, T, B, I, H, W, R, bw, br, [gen_x(rng, T, B, I, dist) for _ in range(2)])
        p = params_mod.GRUQuantParams(H, config_named(cfg_name))
        sc = ref.calc_params_from_ranges(ranges, p.c)
        for n, a in zip(params_mod.WEIGHT_OPS, sc):
            p.scales[n] = a
        wq = ref.quantize_weights(I, H, W, R, bw, br, p.c, p.scale_list())
        x_q = ref.quantize(x, p.c, OP["x"])
        h0_q = ref.quantize(h0, p.c, OP["h"]) if with_h0 else None
        h_q = ref.forward_i32(T, B, I, H, wq, x_q, h0_q, p.c, p.scale_list())
        h = ref.forward_f32(T, B, I, H, wq, x, h0, p.c, p.scale_list())
        out = dict(shape=np.array([T, B, I, H]), config=np.array(cfg_name), W=W, R=R, bw=bw, br=br, x=x,
                   ranges=ranges.as_vector(), params=np.frombuffer(p.to_bytes(), np.uint8),
                   W_q=wq[0], R_q=wq[1], bw_q=wq[2], br_q=wq[3], x_q=x_q, h_q=h_q, h=h)
        if with_h0:
            out.update(h0=h0, h0_q=h0_q)
        np.savez_compressed(os.path.join(HERE, name + ".npz"), **out)
        print(name, "h_q", h_q.shape, "unique", len(np.unique(h_q)))


HIST_OPS = [(8, 0, 1), (8, 0, 0), (8, 1, 0), (8, 1, 1), (16, 0, 0), (4, 0, 1), (12, 0, 1)]  # bits, unsigned, symmetric


def hist_inputs(seed):
    """Seeded 2048-bin histograms of five value distributions (the ones the GRU's operators show)."""
    rng = np.random.default_rng(seed)
    out = []
    for kind in ("normal", "sigmoid", "outliers", "positive", "sparse"):
        if kind == "normal":
            data = rng.normal(0.1, 1.3, 40000)
        elif kind == "sigmoid":
            data = 1 / (1 + np.exp(-rng.normal(0, 3, 40000)))
        elif kind == "outliers":
            data = rng.normal(0, 1, 40000)
            data[rng.integers(0, data.size, 400)] *= 8
        elif kind == "positive":
            data = np.abs(rng.normal(0, 0.4, 40000))
        else:
            data = rng.normal(0, 0.05, 256)
        data = data.astype(np.float32)
        mn, mx = float(data.min()), float(data.max())
        counts, _ = np.histogram(data, bins=2048, range=(mn, mx))
        out.append((counts.astype(np.float32), mn, mx, int(data.size)))
    return out


def main_hist():
    """Percentile / SQNR parameters of the reference's host code for seeded histograms:
    golden/hist/hist_calibration.npz (inputs are regenerated from the seed by the test)."""
    ref = Reference()

    class Op:
        pass
    rows = []
    for h_idx, (counts, mn, mx, total) in enumerate(hist_inputs(77)):
        for o_idx, (bits, uns, sym) in enumerate(HIST_OPS):
            op = Op()
            op.bits, op.is_unsigned, op.symmetric = bits, uns, sym
            for pot2 in (0, 1):
                for method, pct in ((1, 99.9), (1, 99.99), (0, 0.0)):
                    r = ref.calibrate_from_histogram(counts, mn, mx, total, op, pot2, method, pct or 99.99)
                    rows.append([h_idx, o_idx, pot2, method, pct, np.float32(r[0]).view(np.uint32), r[1]])
    os.makedirs(os.path.join(HERE, "hist"), exist_ok=True)
    np.savez_compressed(os.path.join(HERE, "hist", "hist_calibration.npz"),
                        rows=np.array(rows, dtype=np.float64), seed=np.array(77))
    print("hist_calibration", len(rows), "rows")


if __name__ == "__main__":
    main()
    main_hist()
