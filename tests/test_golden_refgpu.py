"""CPU tests of the oracle against outputs of the reference's own GPU code, recorded on a B200 by
tests/golden/make_golden_refgpu.py: the float-storage quantized forward, the training-mode
integer forward with its clamp masks, and the GPU histogram collector."""
import glob
import os

import numpy as np
import pytest

from tests.cases import OP, params_mod

HERE = os.path.dirname(__file__)
NAMES = sorted(os.path.basename(p) for p in glob.glob(os.path.join(HERE, "golden", "refgpu", "*.npz"))
               if not p.endswith("collector.npz"))


def _load(name):
    d = np.load(os.path.join(HERE, "golden", name))
    g = np.load(os.path.join(HERE, "golden", "refgpu", name))
    T, B, I, H = [int(v) for v in d["shape"]]
    p = params_mod.GRUQuantParams.from_bytes(d["params"].tobytes(), H)
    return d, g, (T, B, I, H), p, [d["W_q"], d["R_q"], d["bw_q"], d["br_q"]]


def test_fixtures_exist():
    assert len(NAMES) >= 10


@pytest.mark.parametrize("name", NAMES, ids=[n[:-4] for n in NAMES])
def test_float_storage_forward_matches_reference_gpu_vectors(oracle, name):
    """quantGRUForwardFP: the quantized input equal; h within one step of the h scale on at most
    1 % of the elements (the host's expf / tanhf against CUDA's: a gate output can round across
    a .5 boundary differently)."""
    d, g, (T, B, I, H), p, wq = _load(name)
    h0 = d["h0"] if "h0" in d else None
    h, xq = oracle.forward_fstorage(T, B, I, H, wq, d["x"], h0, p.c, p.scale_list())
    assert np.array_equal(xq, g["xq_fs"])
    hs = float(np.float32(p.c.op[OP["h"]].scale))
    diff = np.abs(np.rint(h.astype(np.float64) / hs) - np.rint(g["h_fs"].astype(np.float64) / hs))
    assert diff.max() <= 1 and (diff > 0).mean() <= 0.01, (diff.max(), (diff > 0).mean())


@pytest.mark.parametrize("name", NAMES, ids=[n[:-4] for n in NAMES])
def test_training_forward_and_masks_match_reference_gpu_vectors(oracle, name):
    """quantGRUForwardInt32(is_training): h_q, v_q and the five clamp masks, bit for bit."""
    d, g, (T, B, I, H), p, wq = _load(name)
    h, v, masks = oracle.forward_i32_train(T, B, I, H, wq, g["x_wide_q"], None, p.c, p.scale_list())
    assert np.array_equal(h, g["h_q"]) and np.array_equal(v, g["v_q"])
    for k, m in enumerate(masks):
        want = np.unpackbits(g[f"mask{k}"])[:m.size].reshape(m.shape)
        assert np.array_equal(m, want), k


def test_collector_matches_reference_gpu_vectors(oracle):
    """GPUHistogramCollector over five batches (range growth and redistribution included)."""
    from tests.golden.make_golden_refgpu import collector_batches
    g = np.load(os.path.join(HERE, "golden", "refgpu", "collector.npz"))
    col = oracle.hist_new(2048)
    for k, data in enumerate(collector_batches()):
        col.collect(data)
        counts, mn, mx, tot = col.get()
        assert (np.float32(mn), np.float32(mx)) == tuple(g[f"meta{k}"]) and tot == int(g[f"total{k}"])
        assert np.array_equal(counts, g[f"counts{k}"]), k
