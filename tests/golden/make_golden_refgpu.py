"""Generate tests/golden/refgpu/*.npz: outputs of the reference's own GPU code for the problems
of the golden files beside this script.  Needs a CUDA device and the checker library built
from the unmodified reference sources (oracle/_ref/libqgru_ref.so); the reference tree itself is
not needed.

    python tests/golden/make_golden_refgpu.py [output directory]

Per problem: the float-storage quantized forward (quantGRUForwardFP, inference: h and the
quantized x), and the training-mode integer forward (quantGRUForwardInt32: h_q, v_q and the five
clamp masks) on an input four times wider than the calibrated one, so that clamps occur.
collector.npz: one GPUHistogramCollector fed five batches of growing and shrinking spread (counts,
range and total after every batch).  These are the fixtures that pin the oracle's restatement of
those three paths on machines without a GPU."""
import glob
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from oracle.binding import Reference, ReferenceGpu  # noqa: E402
from tests.cases import OP, params_mod  # noqa: E402


def collector_batches():
    rng = np.random.default_rng(3)
    return [rng.normal(0.3, s, 20000).astype(np.float32) for s in (1.0, 1.0, 1.7, 0.5, 3.0)]


def main(out_dir):
    os.makedirs(out_dir, exist_ok=True)
    ref = Reference()
    gpu = ReferenceGpu(ref)
    assert gpu.device_count() >= 1, "needs a CUDA device"
    for path in sorted(glob.glob(os.path.join(HERE, "*.npz"))):
        d = np.load(path)
        T, B, I, H = [int(v) for v in d["shape"]]
        p = params_mod.GRUQuantParams.from_bytes(d["params"].tobytes(), H)
        sc = p.scale_list()
        wq = [d["W_q"], d["R_q"], d["bw_q"], d["br_q"]]
        h0 = d["h0"] if "h0" in d else None
        h_fs, xq_fs, _ = gpu.forward_fstorage(T, B, I, H, d["W"], d["R"], d["bw"], d["br"], d["x"], h0, p.c, sc)
        x_wide_q = ref.quantize(d["x"] * np.float32(4.0), p.c, OP["x"])
        h_q, v_q, masks = gpu.forward_i32(T, B, I, H, wq, x_wide_q, None, p.c, sc, training=True, masks=True)
        name = os.path.basename(path)
        np.savez_compressed(os.path.join(out_dir, name), h_fs=h_fs, xq_fs=xq_fs, x_wide_q=x_wide_q, h_q=h_q,
                            v_q=v_q, **{f"mask{k}": np.packbits(m) for k, m in enumerate(masks)})
        print(name, "fs h", h_fs.shape, "clamped share", [round(1 - float(m.mean()), 3) for m in masks])
    col = gpu.hist_new(2048)
    out = {}
    for k, data in enumerate(collector_batches()):
        col.collect(data)
        counts, mn, mx, tot = col.get()
        out[f"counts{k}"] = counts
        out[f"meta{k}"] = np.array([mn, mx], np.float32)
        out[f"total{k}"] = np.array(tot)
    np.savez_compressed(os.path.join(out_dir, "collector.npz"), **out)
    print("collector.npz")


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else os.path.join(HERE, "refgpu"))
