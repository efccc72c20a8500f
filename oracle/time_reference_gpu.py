"""TEST INFRASTRUCTURE: time the reference's own GPU integer forward (quantGRUForwardInt32,
compiled unmodified into oracle/_ref) on the benchmark workloads, for context beside bench.py's
numbers.  Inputs are resident on the device; the time is CUDA-event time per call, which
includes what the reference does inside every call (buffer allocation, rescale upload,
device-wide synchronisations).  One direction per call, as the reference runs it.

    python oracle/time_reference_gpu.py cfg2 [cfg1 ...]
"""
import json
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main(names):
    from bench import WORKLOADS
    from oracle.binding import Oracle, Reference, ReferenceGpu
    from tests.cases import config_named, make_case
    ref = Reference()
    gpu = ReferenceGpu(ref)
    if gpu.device_count() < 1:
        raise SystemExit("no CUDA device")
    for name in names:
        I, H, B, T, bidir, cfg_name, xdist, _ = WORKLOADS[name]
        cal = make_case(1000, min(T, 20), 4, I, H, ref, config_named(cfg_name), dist=xdist, calib_batches=1,
                        oracle=Oracle())
        x = np.random.default_rng(77).standard_normal((T, B, I)).astype(np.float32)
        x_q = ref.quantize(x, cal.params.c, 0)
        ms = gpu.time_forward_i32(T, B, I, H, cal.wq, x_q, cal.params.c, cal.params.scale_list(),
                                  warmup=1, iters=3)
        print(json.dumps({"workload": name, "impl": "reference GPU path, one direction", "T": T, "B": B,
                          "I": I, "H": H, "ms_per_forward": ms, "tokens_per_s": T * B / ms * 1e3,
                          "us_per_timestep": ms * 1e3 / T}))


if __name__ == "__main__":
    main(sys.argv[1:] or ["cfg2"])
