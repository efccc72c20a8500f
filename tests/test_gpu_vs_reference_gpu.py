"""GPU tests against the reference's own GPU code (the unmodified sources compiled into the
checker library, driven through the ref_gpu_* functions of oracle/ref_shim.cc): the integer
forward, its training buffer and clamp masks bit for bit, the histogram collectors bit for bit
on identical arrays, and the float forward, MinMax ranges and calibration histograms to the
precision the reference's float forward has on this GPU.  That forward switches cuBLAS to
tensor-op math (src/gru_forward_gpu.cu:359), i.e. TF32 products with a 10-bit mantissa, so its
outputs sit about 3e-4 from an fp32 GRU; the 1e-5 bound of the float mode is held against the
fp32 restatement and torch.nn.GRU in test_gpu_module.py, and here the bound is TF32_RTOL.
Skipped where the checker library has not been built."""
import importlib

import numpy as np
import pytest

from __graft_entry__ import PKG_NAME
from tests.cases import OP, config_named, gen_weights, gen_x, make_case, params_mod

gru_ops = importlib.import_module(PKG_NAME + ".gru_ops")
_cabi = importlib.import_module(PKG_NAME + "._cabi")
pytestmark = pytest.mark.gpu

TF32_RTOL = 2e-3     # relative to the largest magnitude of the compared tensor


@pytest.fixture(scope="module")
def refgpu(reference, cuda_device):
    from oracle.binding import ReferenceGpu
    g = ReferenceGpu(reference)
    if g.device_count() < 1:
        pytest.skip("the reference library sees no CUDA device")
    return g


def _t(a, dev):
    import torch
    return torch.from_numpy(np.ascontiguousarray(a)).to(dev)


def _rel_err(got, want):
    return np.abs(got - want).max() / max(np.abs(want).max(), 1e-30)


@pytest.mark.parametrize("cfg_name", ["default", "cfg2", "cfg3", "cfg5", "pot2_asym"])
@pytest.mark.parametrize("shape", [(5, 6, 20, 40), (4, 20, 48, 512), (6, 3, 80, 256)])
def test_integer_forward_equals_reference_gpu(reference, refgpu, cuda_device, cfg_name, shape):
    """h_q of every timestep: product == the reference's GPU integer path == its CPU path."""
    T, B, I, H = shape
    case = make_case(seed=31, T=T, B=B, I=I, H=H, checker=reference, config=config_named(cfg_name),
                     with_h0=(cfg_name == "cfg2"))
    sc = case.params.scale_list()
    want = refgpu.forward_i32(T, B, I, H, case.wq, case.x_q, case.h0_q, case.params.c, sc)
    cpu = reference.forward_i32(T, B, I, H, case.wq, case.x_q, case.h0_q, case.params.c, sc)
    assert np.array_equal(want, cpu), "the reference's GPU and CPU integer paths differ"
    with gru_ops.Handle(I, H, device=0) as hd:
        hd.set_params(case.params)
        hd.set_weights_i32(*[_t(a, cuda_device) for a in case.wq])
        got = hd.forward_i32(_t(case.x_q, cuda_device),
                             _t(case.h0_q, cuda_device) if case.h0_q is not None else None)
        got = got.cpu().numpy()
    assert np.array_equal(got, want)


@pytest.mark.parametrize("cfg_name,sigma", [("cfg2", 1.0), ("default", 4.0), ("pot2_asym", 4.0)])
def test_training_outputs_equal_reference_gpu(oracle, reference, refgpu, cuda_device, cfg_name, sigma):
    """Training mode: h_q, v_q and the five clamp masks: product == the reference's GPU path ==
    the oracle.  sigma = 4 feeds inputs four times wider than the calibration saw, so that a
    good share of the values is clamped and the masks hold both zeros and ones."""
    T, B, I, H = 5, 4, 24, 72
    case = make_case(seed=32, T=T, B=B, I=I, H=H, checker=reference, config=config_named(cfg_name))
    rng = np.random.default_rng(77)
    x_q = reference.quantize(gen_x(rng, T, B, I, sigma=sigma), case.params.c, OP["x"])
    sc = case.params.scale_list()
    want_h, want_v, want_m = refgpu.forward_i32(T, B, I, H, case.wq, x_q, None, case.params.c, sc,
                                                training=True, masks=True)
    orc_h, orc_v, orc_m = oracle.forward_i32_train(T, B, I, H, case.wq, x_q, None, case.params.c, sc)
    assert np.array_equal(orc_h, want_h) and np.array_equal(orc_v, want_v)
    for k in range(5):
        assert np.array_equal(orc_m[k], want_m[k]), k
    with gru_ops.Handle(I, H, device=0) as hd:
        hd.set_params(case.params)
        hd.set_weights_i32(*[_t(a, cuda_device) for a in case.wq])
        got_h, got_v, got_m = hd.forward_i32_train(_t(x_q, cuda_device), want_masks=True)
    assert np.array_equal(got_h.cpu().numpy(), want_h)
    assert np.array_equal(got_v.cpu().numpy(), want_v)
    for k in range(5):
        assert np.array_equal(got_m[k].cpu().numpy(), want_m[k]), k
    if sigma > 1.0:
        assert any(0 < m.mean() < 1 for m in want_m), "no clamp was exercised"


@pytest.mark.parametrize("shape", [(6, 5, 20, 40), (12, 33, 64, 128), (3, 2, 300, 520)])
def test_float_mode_matches_reference_gpu(refgpu, cuda_device, shape):
    """fp32 GRU against hasteGRUForward (TF32 products) on the same device."""
    T, B, I, H = shape
    rng = np.random.default_rng(5)
    W, R, bw, br = gen_weights(rng, I, H)
    x = gen_x(rng, T, B, I)
    h0 = (rng.standard_normal((B, H)) * 0.3).astype(np.float32)
    want_h, want_v = refgpu.forward_float(T, B, I, H, W, R, bw, br, x, h0, want_v=True)
    with gru_ops.Handle(I, H, device=0) as hd:
        h, v = hd.forward_float(*[_t(a, cuda_device) for a in (W, R, bw, br, x)], _t(h0, cuda_device),
                                want_v=True)
    assert _rel_err(h.cpu().numpy(), want_h) <= TF32_RTOL
    assert _rel_err(v.cpu().numpy(), want_v) <= TF32_RTOL


def test_minmax_ranges_match_reference_gpu(refgpu, cuda_device):
    """forwardWithCalibrationGPU(MINMAX) over three batches: computed ranges to TF32 precision,
    the ranges of x and of the weights exactly."""
    T, B, I, H = 9, 7, 20, 48
    rng = np.random.default_rng(9)
    W, R, bw, br = gen_weights(rng, I, H)
    batches = [gen_x(rng, T, B, I, "outliers") for _ in range(3)]
    want, got = params_mod.Ranges(H), params_mod.Ranges(H)
    with gru_ops.Handle(I, H, device=0) as hd:
        dW = [_t(a, cuda_device) for a in (W, R, bw, br)]
        for xb in batches:
            refgpu.calibrate_minmax(T, B, I, H, W, R, bw, br, xb, want)
            hd.calibrate_minmax(*dW, _t(xb, cuda_device), got)
    idx = [0, 1] + list(range(6, 17))
    span = np.maximum(np.abs(want.max_v[idx]), np.abs(want.min_v[idx]))
    assert np.all(np.abs(got.min_v[idx] - want.min_v[idx]) <= TF32_RTOL * span + 1e-6)
    assert np.all(np.abs(got.max_v[idx] - want.max_v[idx]) <= TF32_RTOL * span + 1e-6)
    for n in params_mod.WEIGHT_OPS:
        assert np.array_equal(got.ch_min[n], want.ch_min[n]) and np.array_equal(got.ch_max[n], want.ch_max[n])
    assert got.min_v[OP["x"]] == want.min_v[OP["x"]] and got.max_v[OP["x"]] == want.max_v[OP["x"]]


def _same(a, b):
    c1, mn1, mx1, t1 = a
    c2, mn2, mx2, t2 = b
    assert (mn1, mx1, t1) == (mn2, mx2, t2), ((mn1, mx1, t1), (mn2, mx2, t2))
    assert np.array_equal(c1, c2), np.abs(c1 - c2).sum()


def test_collector_equals_reference_gpu_collector(oracle, refgpu, cuda_device):
    """One collector over batches with growing and shrinking spread: product == the reference's
    GPUHistogramCollector == the oracle's restatement of it, counts and range, bit for bit."""
    rng = np.random.default_rng(3)
    hs = params_mod.Histograms(8, device=0)
    for idx, scales in enumerate(([1.0, 1.0, 1.7, 0.5, 3.0], [0.01, 5.0, 5.0], [2.0, 1.0, 1.0, 1.0])):
        want = refgpu.hist_new(2048)
        orc = oracle.hist_new(2048)
        for s in scales:
            data = (rng.normal(0.3, s, 50000)).astype(np.float32)
            hs.collect(idx, _t(data, cuda_device))
            want.collect(data)
            orc.collect(data)
            _same(orc.get(), want.get())
            _same(hs.get(idx), want.get())
    hs.close()


@pytest.mark.parametrize("gran", ["PER_CHANNEL", "PER_GATE", "PER_TENSOR"])
def test_calibration_histograms_match_reference_gpu(refgpu, cuda_device, gran):
    """Two batches through the calibration forward of both libraries.  Histograms of tensors that
    are read (x, the weights) are equal bit for bit; histograms of computed tensors agree in
    total, in range to TF32 precision, and in shape.  The bound on the shape follows from that
    precision: a value that is off by at most e = TF32_RTOL * span, binned on a grid whose ends are
    off by at most e as well, lands at most k = ceil(2 e / bin width) + 1 bins from where the
    reference put it, so the two cumulative counts differ at any bin edge by at most the mass of
    k neighbouring bins, i.e. by at most k times the fullest bin of the reference's histogram.
    81 920 samples per tensor, so that the fullest bin is a small part of the total for the
    bell-shaped tensors (the saturating gate outputs pile up in their end bins and get the
    correspondingly wider bound)."""
    T, B, I, H = 20, 64, 32, 64
    rng = np.random.default_rng(9)
    W, R, bw, br = gen_weights(rng, I, H)
    g = {"PER_CHANNEL": _cabi.PER_CHANNEL, "PER_GATE": _cabi.PER_GATE, "PER_TENSOR": _cabi.PER_TENSOR}[gran]
    cfg = params_mod.OperatorQuantConfig()
    for n in params_mod.WEIGHT_OPS:
        cfg.granularity[n] = g
    p = params_mod.GRUQuantParams(H, cfg)
    hs = params_mod.Histograms(H, device=0)
    ref_set = refgpu.histset_new(H, 2048)
    with gru_ops.Handle(I, H, device=0) as hd:
        dev = [_t(a, cuda_device) for a in (W, R, bw, br)]
        for batch in range(2):
            x = gen_x(rng, T, B, I, sigma=1.0 + batch)
            hd.calibrate_hist(*dev, _t(x, cuda_device), hs, [g] * 4)
            ref_set.calibrate(T, B, I, H, W, R, bw, br, x, p.c, use_percentile=True)
    ref_set.sync()
    _same(hs.get(OP["x"]), ref_set.get(OP["x"]))
    for name in ("h", "weight_ih_linear", "weight_hh_linear", "update_gate_input", "update_gate_output",
                 "reset_gate_input", "reset_gate_output", "new_gate_input", "new_gate_output",
                 "mul_reset_hidden", "mul_new_contribution", "mul_old_contribution"):
        c1, mn1, mx1, t1 = hs.get(OP[name])
        c2, mn2, mx2, t2 = ref_set.get(OP[name])
        assert t1 == t2, name
        span = max(abs(mx2 - mn2), 1e-30)
        assert abs(mn1 - mn2) <= TF32_RTOL * span + 1e-7 and abs(mx1 - mx2) <= TF32_RTOL * span + 1e-7, name
        moved = np.abs(np.cumsum(c1.astype(np.float64)) - np.cumsum(c2.astype(np.float64))).max()
        k_bins = int(np.ceil(2 * TF32_RTOL * len(c2))) + 1
        assert moved <= k_bins * float(c2.max()), (name, moved, k_bins, float(c2.max()), t1)
    C3 = 3 * H
    for k, name in enumerate(("W", "R", "bw", "br")):
        if gran == "PER_TENSOR":
            _same(hs.get(OP[name]), ref_set.get(OP[name]))
        elif gran == "PER_GATE":
            for gi in range(3):
                _same(hs.get(_cabi.HIST_GATE0 + 3 * k + gi), ref_set.get(_cabi.HIST_GATE0 + 3 * k + gi))
        else:
            for c_idx in (0, 1, H + 3, C3 - 1):
                _same(hs.get(_cabi.HIST_CHANNEL0 + k * C3 + c_idx),
                      ref_set.get(_cabi.HIST_CHANNEL0 + k * C3 + c_idx))
    hs.close()


def _quanta(h, case):
    """Dequantized h back to integer steps of the h scale."""
    hs = np.float32(case.params.c.op[OP["h"]].scale)
    return np.rint(h.astype(np.float64) / float(hs)).astype(np.int64)


@pytest.mark.parametrize("cfg_name", ["default", "sym8_tensor", "cfg2", "cfg3", "cfg5", "pot2_asym"])
@pytest.mark.parametrize("shape", [(6, 5, 20, 40), (5, 9, 64, 256)])
def test_float_storage_forward_equals_reference_gpu(oracle, reference, refgpu, cuda_device, cfg_name, shape):
    """quantGRUForwardFP (inference) on the same device: quantized x and every timestep of h are
    equal bit for bit (the products are exact integer sums on both sides and the float
    operations after them are the same in the same order).  The CPU oracle evaluates expf / tanhf
    with the host's libm, so a gate output may round across a .5 boundary differently: at most
    one step of the h scale on at most 1 % of the elements."""
    T, B, I, H = shape
    case = make_case(seed=41, T=T, B=B, I=I, H=H, checker=reference, config=config_named(cfg_name),
                     with_h0=True)
    sc = case.params.scale_list()
    want_h, want_xq, want_wq = refgpu.forward_fstorage(T, B, I, H, case.W, case.R, case.bw, case.br, case.x,
                                                       case.h0, case.params.c, sc)
    for a, b in zip(want_wq, case.wq):   # quantizeGRUWeights == the integer path's weight quantize
        assert np.array_equal(a.astype(np.int32).reshape(b.shape), b)
    with gru_ops.Handle(I, H, device=0) as hd:
        hd.set_params(case.params)
        hd.set_weights_f32(*[_t(a, cuda_device) for a in (case.W, case.R, case.bw, case.br)])
        got_h, got_xq = hd.forward_fstorage(_t(case.x, cuda_device), _t(case.h0, cuda_device), want_x_q=True)
        got_h, got_xq = got_h.cpu().numpy(), got_xq.cpu().numpy()
        assert "rec=gemv_float_cell" in hd.describe_plan()          # small batch: one CTA per row
        assert "gates=tabulated" in hd.describe_plan()
        for opt, form in (("mma", "rec=tcgen05_i8_float_cell"),     # tensor-core cluster recurrence
                          ("dp4a", "rec=dp4a_float_cell"),          # one launch, dp4a products
                          ("generic", "rec=per_step_float_cell")):  # two launches per step
            hd.set_option("rec", opt)
            other = hd.forward_fstorage(_t(case.x, cuda_device), _t(case.h0, cuda_device)).cpu().numpy()
            assert form in hd.describe_plan()
            assert np.array_equal(other, got_h), form
        hd.set_option("rec", "mma")
        hd.set_option("cell", "generic")                            # gates evaluated, not tabulated
        direct = hd.forward_fstorage(_t(case.x, cuda_device), _t(case.h0, cuda_device)).cpu().numpy()
        assert "gates=evaluated" in hd.describe_plan()
        assert np.array_equal(direct, got_h)
        hd.set_option("cell", "auto")
        hd.set_option("rec", "auto")
        flipped = np.ascontiguousarray(case.x[::-1])
        rev = hd.forward_fstorage(_t(flipped, cuda_device), _t(case.h0, cuda_device), reverse=True).cpu().numpy()
    assert np.array_equal(got_xq, want_xq)
    assert np.array_equal(got_h, want_h), np.abs(_quanta(got_h, case) - _quanta(want_h, case)).max()
    # reverse flag: slot T holds the initial state, slots T-1..0 the outputs
    assert np.array_equal(rev[::-1], want_h)
    orc_h, orc_xq = oracle.forward_fstorage(T, B, I, H, case.wq, case.x, case.h0, case.params.c, sc)
    assert np.array_equal(orc_xq, want_xq)
    d = np.abs(_quanta(orc_h, case) - _quanta(want_h, case))
    assert d.max() <= 1 and (d > 0).mean() <= 0.01, (d.max(), (d > 0).mean())


@pytest.mark.parametrize("cfg_name,sigma", [("default", 1.0), ("cfg2", 3.0), ("cfg3", 3.0), ("pot2_asym", 3.0)])
def test_float_storage_training_forward_equals_reference_gpu(reference, refgpu, cuda_device, cfg_name, sigma):
    """quantGRUForwardFP(is_training): h, the dequantized gate buffer v and the eleven clamp masks
    equal the reference's bit for bit; sigma = 3 feeds inputs three times wider than calibrated so
    that the masks hold zeros.  h also equals the inference-mode kernels' output."""
    T, B, I, H = 6, 5, 20, 72
    case = make_case(seed=43, T=T, B=B, I=I, H=H, checker=reference, config=config_named(cfg_name), with_h0=True)
    x = (case.x * np.float32(sigma)).astype(np.float32)
    h0 = (case.h0 * np.float32(sigma)).astype(np.float32)
    sc = case.params.scale_list()
    want_h, want_v, want_m = refgpu.forward_fstorage_train(T, B, I, H, case.W, case.R, case.bw, case.br, x, h0,
                                                           case.params.c, sc)
    with gru_ops.Handle(I, H, device=0) as hd:
        hd.set_params(case.params)
        dw = [_t(a, cuda_device) for a in (case.W, case.R, case.bw, case.br)]
        hd.set_weights_f32(*dw)
        h, v, x_q, masks = hd.forward_fstorage_train(*dw, _t(x, cuda_device), _t(h0, cuda_device))
        h_inf = hd.forward_fstorage(_t(x, cuda_device), _t(h0, cuda_device))
    assert np.array_equal(h.cpu().numpy(), want_h)
    assert np.array_equal(h_inf.cpu().numpy(), want_h)
    assert np.array_equal(v.cpu().numpy(), want_v)
    for n, m in masks.items():
        assert np.array_equal(m.cpu().numpy(), want_m[n]), n
    if sigma > 1.0:
        assert sum(0 < want_m[n].mean() < 1 for n in want_m) >= 3, "too few clamps were exercised"


@pytest.mark.parametrize("cfg_name,sigma", [("default", 1.0), ("cfg2", 3.0), ("pot2_asym", 3.0)])
def test_integer_training_forward_float_interface_equals_reference_gpu(reference, refgpu, cuda_device, cfg_name, sigma):
    """quantGRUForwardInt(is_training): dequantized h and v and the eleven clamp masks of the
    integer path, bit for bit."""
    T, B, I, H = 6, 5, 20, 72
    case = make_case(seed=44, T=T, B=B, I=I, H=H, checker=reference, config=config_named(cfg_name), with_h0=True)
    x = (case.x * np.float32(sigma)).astype(np.float32)
    h0 = (case.h0 * np.float32(sigma)).astype(np.float32)
    sc = case.params.scale_list()
    want_h, want_v, want_m = refgpu.forward_fstorage_train(T, B, I, H, case.W, case.R, case.bw, case.br, x, h0,
                                                           case.params.c, sc, int_storage=True)
    with gru_ops.Handle(I, H, device=0) as hd:
        hd.set_params(case.params)
        dw = [_t(a, cuda_device) for a in (case.W, case.R, case.bw, case.br)]
        hd.set_weights_f32(*dw)
        h, v, x_q, masks = hd.forward_fstorage_train(*dw, _t(x, cuda_device), _t(h0, cuda_device), int_storage=True)
        h_inf = hd.forward_f32(_t(x, cuda_device), _t(h0, cuda_device))
    assert np.array_equal(h.cpu().numpy(), want_h)
    assert np.array_equal(h_inf.cpu().numpy(), want_h)
    assert np.array_equal(v.cpu().numpy(), want_v)
    assert np.array_equal(x_q.cpu().numpy(), reference.quantize(x, case.params.c, OP["x"]))
    for n, m in masks.items():
        assert np.array_equal(m.cpu().numpy(), want_m[n]), n
