"""TEST INFRASTRUCTURE: time the reference's own GPU integer forward (quantGRUForwardInt32,
compiled unmodified into oracle/_ref) on the benchmark workloads, for context beside bench.py's
numbers; with --fstorage, its float-storage forward (quantGRUForwardFP) and this library's
(qgru_forward_fstorage) side by side.  Inputs are resident on the device; the time is CUDA-event time per call, which
includes what the reference does inside every call (buffer allocation, rescale upload,
device-wide synchronisations).  One direction per call, as the reference runs it.

    python oracle/time_reference_gpu.py [--fstorage] cfg2 [cfg1 ...]
"""
import json
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main(names):
    fstorage = "--fstorage" in names
    names = [n for n in names if not n.startswith("--")] or ["cfg2"]
    from oracle.binding import Oracle, Reference, ReferenceGpu
    from oracle.cases import config_named, make_case, _workloads
    WORKLOADS = _workloads.WORKLOADS
    ref = Reference()
    gpu = ReferenceGpu(ref)
    if gpu.device_count() < 1:
        raise SystemExit("no CUDA device")
    for name in names:
        I, H, B, T, bidir, cfg_name, xdist, _ = WORKLOADS[name]
        cal = make_case(1000, min(T, 20), 4, I, H, ref, config_named(cfg_name), dist=xdist, calib_batches=1,
                        oracle=Oracle())
        x = _workloads.gen_x(np.random.default_rng(77), T, B, I, xdist)
        if fstorage:
            time_fstorage(name, gpu, cal, x, T, B, I, H)
            continue
        x_q = ref.quantize(x, cal.params.c, 0)
        ms = gpu.time_forward_i32(T, B, I, H, cal.wq, x_q, cal.params.c, cal.params.scale_list(),
                                  warmup=1, iters=3)
        print(json.dumps({"workload": name, "impl": "reference GPU path, one direction", "T": T, "B": B,
                          "I": I, "H": H, "ms_per_forward": ms, "tokens_per_s": T * B / ms * 1e3,
                          "us_per_timestep": ms * 1e3 / T}))


def time_fstorage(name, gpu, cal, x, T, B, I, H):
    import torch
    import importlib
    from __graft_entry__ import PKG_NAME, load_package
    load_package()
    gru_ops = importlib.import_module(PKG_NAME + ".gru_ops")
    sc = cal.params.scale_list()
    ms_ref = gpu.time_forward_fstorage(T, B, I, H, cal.W, cal.R, cal.bw, cal.br, x, cal.params.c, sc)
    dev = torch.device("cuda:0")
    with gru_ops.Handle(I, H, device=0) as hd:
        hd.set_params(cal.params)
        hd.set_weights_f32(*[torch.from_numpy(a).to(dev) for a in (cal.W, cal.R, cal.bw, cal.br)])
        xd = torch.from_numpy(x).to(dev)
        for _ in range(2):
            hd.forward_fstorage(xd)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(3):
            hd.forward_fstorage(xd, sync=False)
        e1.record()
        torch.cuda.synchronize()
        ms_ours = e0.elapsed_time(e1) / 3
    print(json.dumps({"workload": name, "path": "float-storage forward, one direction", "T": T, "B": B,
                      "reference_gpu_ms": ms_ref, "this_library_ms": ms_ours,
                      "reference_us_per_timestep": ms_ref * 1e3 / T, "ours_us_per_timestep": ms_ours * 1e3 / T}))


if __name__ == "__main__":
    main(sys.argv[1:])
