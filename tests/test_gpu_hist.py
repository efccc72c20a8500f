"""GPU tests of histogram calibration: the collector kernels against the oracle's collector
(bit-exact on identical arrays), the whole calibration forward, and Percentile / SQNR
parameters end to end through the QuantGRU module."""
import importlib

import numpy as np
import pytest

from __graft_entry__ import PKG_NAME
from tests.cases import OP, config_named, gen_weights, gen_x, params_mod

gru_ops = importlib.import_module(PKG_NAME + ".gru_ops")
quant_gru = importlib.import_module(PKG_NAME + ".quant_gru")
_cabi = importlib.import_module(PKG_NAME + "._cabi")
pytestmark = pytest.mark.gpu


def _t(a, dev):
    import torch
    return torch.from_numpy(np.ascontiguousarray(a)).to(dev)


def _same(hist_get, orc_get):
    c1, mn1, mx1, t1 = hist_get
    c2, mn2, mx2, t2 = orc_get
    assert (mn1, mx1, t1) == (mn2, mx2, t2), ((mn1, mx1, t1), (mn2, mx2, t2))
    assert np.array_equal(c1, c2), np.abs(c1 - c2).sum()


def test_collector_equals_oracle_over_growing_batches(oracle, cuda_device):
    rng = np.random.default_rng(3)
    hs = params_mod.Histograms(8, device=0)
    for idx, scales in enumerate(([1.0, 1.0, 1.7, 0.5, 3.0], [0.01, 5.0, 5.0], [2.0, 1.0, 1.0, 1.0])):
        want = oracle.hist_new(2048)
        for s in scales:
            data = (rng.normal(0.3, s, 50000)).astype(np.float32)
            data[rng.integers(0, data.size, 3)] = np.inf
            data[rng.integers(0, data.size, 3)] = np.nan
            hs.collect(idx, _t(data, cuda_device))
            want.collect(data)
            _same(hs.get(idx), want.get())
    hs.close()


def test_collector_degenerate_inputs(oracle, cuda_device):
    hs = params_mod.Histograms(8, device=0, num_bins=64)
    for idx, data in enumerate((np.full(1000, 3.0, np.float32), np.zeros(10, np.float32),
                                np.array([np.nan, np.inf], np.float32),
                                np.array([1e-12, 2e-12, 0.0], np.float32))):
        want = oracle.hist_new(64)
        for _ in range(2):
            hs.collect(idx, _t(data, cuda_device))
            want.collect(data)
        _same(hs.get(idx), want.get())
    hs.close()


@pytest.mark.parametrize("gran", ["PER_CHANNEL", "PER_GATE", "PER_TENSOR"])
def test_calibration_forward_histograms(oracle, cuda_device, gran):
    """Two batches through qgru_calibrate_hist: every histogram that is a function of tensors the
    library returns is compared exactly with the oracle's collector fed from those tensors."""
    T, B, I, H = 7, 6, 20, 40
    rng = np.random.default_rng(9)
    W, R, bw, br = gen_weights(rng, I, H)
    g = {"PER_CHANNEL": _cabi.PER_CHANNEL, "PER_GATE": _cabi.PER_GATE, "PER_TENSOR": _cabi.PER_TENSOR}[gran]
    hs = params_mod.Histograms(H, device=0)
    names = ["x", "h", "update_gate_output", "reset_gate_output", "new_gate_output", "mul_reset_hidden",
             "mul_new_contribution", "mul_old_contribution"]
    want = {n: oracle.hist_new(2048) for n in names}
    w_tensor = [oracle.hist_new(2048) for _ in range(4)]
    w_gate = [[oracle.hist_new(2048) for _ in range(3)] for _ in range(4)]
    with gru_ops.Handle(I, H, device=0) as hd:
        dev = [_t(a, cuda_device) for a in (W, R, bw, br)]
        for batch in range(2):
            x = gen_x(rng, T, B, I, sigma=1.0 + batch)
            hd.calibrate_hist(*dev, _t(x, cuda_device), hs, [g] * 4)
            h, v = hd.forward_float(*dev, _t(x, cuda_device), want_v=True)
            h, v = h.cpu().numpy(), v.cpu().numpy()
            z, r, n, rg = (v[:, :, k * H:(k + 1) * H] for k in range(4))
            want["x"].collect(x)
            want["h"].collect(h[1:])
            want["update_gate_output"].collect(z)
            want["reset_gate_output"].collect(r)
            want["new_gate_output"].collect(n)
            want["mul_reset_hidden"].collect(r * rg)
            want["mul_new_contribution"].collect((np.float32(1.0) - z) * n)
            want["mul_old_contribution"].collect(z * h[:-1])
            for k, m in enumerate((W, R, bw.reshape(1, -1), br.reshape(1, -1))):
                w_tensor[k].collect(m)
                for gi in range(3):
                    w_gate[k][gi].collect(m[:, gi * H:(gi + 1) * H])
    for n in names:
        _same(hs.get(OP[n]), want[n].get())
    # the remaining activation histograms: every value counted, sensible ranges
    for n in ("weight_ih_linear", "weight_hh_linear"):
        c, mn, mx, tot = hs.get(OP[n])
        assert tot == 2 * T * B * 3 * H and c.sum() == tot and mn < 0 < mx
    for n in ("update_gate_input", "reset_gate_input", "new_gate_input"):
        c, mn, mx, tot = hs.get(OP[n])
        assert tot == 2 * T * B * H and c.sum() == tot and mn < mx
    for k, (name, m) in enumerate((("W", W), ("R", R), ("bw", bw.reshape(1, -1)), ("br", br.reshape(1, -1)))):
        if gran == "PER_TENSOR":
            _same(hs.get(OP[name]), w_tensor[k].get())
        elif gran == "PER_GATE":
            for gi in range(3):
                _same(hs.get(_cabi.HIST_GATE0 + 3 * k + gi), w_gate[k][gi].get())
        else:
            for c_idx in (0, 1, H + 3, 3 * H - 1):       # collected once, whatever the batch count
                one = oracle.hist_new(2048)
                one.collect(m[:, c_idx])
                _same(hs.get(_cabi.HIST_CHANNEL0 + k * 3 * H + c_idx), one.get())
    hs.close()


@pytest.mark.parametrize("method", ["percentile", "sqnr"])
@pytest.mark.parametrize("cfg_name", ["default", "cfg3", "pot2_asym"])
def test_params_from_gpu_histograms_equal_oracle(oracle, cuda_device, method, cfg_name):
    """qgru_calc_params_from_hist against the oracle applied to the exported histograms."""
    T, B, I, H = 6, 5, 16, 24
    rng = np.random.default_rng(11)
    W, R, bw, br = gen_weights(rng, I, H)
    cfg = config_named(cfg_name)
    hs = params_mod.Histograms(H, device=0)
    with gru_ops.Handle(I, H, device=0) as hd:
        dev = [_t(a, cuda_device) for a in (W, R, bw, br)]
        for _ in range(2):
            hd.calibrate_hist(*dev, _t(gen_x(rng, T, B, I, dist="outliers"), cuda_device), hs, cfg.granularity_list())
    pct = method == "percentile"
    got = params_mod.GRUQuantParams.from_histograms(hs, cfg, use_percentile=pct, percentile=99.9)
    for name, idx in OP.items():
        if name in ("W", "R", "bw", "br"):
            continue
        op = got.c.op[idx]
        want = oracle.calibrate_from_histogram(*hs.get(idx), op, cfg.use_pot2, pct, 99.9)
        assert want == (float(np.float32(op.scale)), int(op.zero_point)), (name, want)
    for k, name in enumerate(("W", "R", "bw", "br")):
        op = got.c.op[OP[name]]
        gran = cfg.granularity[name]
        for c_idx in (0, H, 3 * H - 1):
            if gran == _cabi.PER_TENSOR:
                idx = OP[name]
            elif gran == _cabi.PER_GATE:
                idx = _cabi.HIST_GATE0 + 3 * k + c_idx // H
            else:
                idx = _cabi.HIST_CHANNEL0 + k * 3 * H + c_idx
            want = oracle.calibrate_from_histogram(*hs.get(idx), op, cfg.use_pot2, pct, 99.9)
            assert want is not None and want[0] == float(got.scales[name][c_idx]), (name, c_idx)
    hs.close()


@pytest.mark.parametrize("method", ["percentile", "sqnr"])
def test_quantgru_histogram_calibration_end_to_end(cuda_device, method):
    """The module with calibration_method = percentile / sqnr: calibrate, finalize, quantized
    forward close to the float forward (the reference's own acceptance form: cosine similarity)."""
    import torch
    torch.manual_seed(1)
    m = quant_gru.QuantGRU(24, 48, bidirectional=True, quant_storage_dtype="int32").cuda().eval()
    m.calibration_method = method
    m.percentile_value = 99.99
    m.calibrating = True
    for _ in range(3):
        m(torch.randn(12, 9, 24, device="cuda"))
    m.calibrating = False
    m.finalize_calibration()
    x = torch.randn(12, 9, 24, device="cuda")
    want, _ = m(x)
    m.use_quantization = True
    got, _ = m(x)
    cos = torch.nn.functional.cosine_similarity(got.flatten(), want.flatten(), dim=0).item()
    assert cos > 0.99, cos
    with pytest.raises(ValueError):
        m.calibration_method = "entropy"
        m.finalize_calibration()
