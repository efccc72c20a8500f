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


if __name__ == "__main__":
    main()
