"""GPU tests of the layers above the integer kernels: float mode, MinMax calibration and the
nn.GRU-compatible QuantGRU module (bidirectional, batch_first, int-in/int-out, JSON files)."""
import importlib

import numpy as np
import pytest

from __graft_entry__ import PKG_NAME
from tests.cases import OP, config_named, gen_weights, gen_x, make_case, params_mod

gru_ops = importlib.import_module(PKG_NAME + ".gru_ops")
quant_gru = importlib.import_module(PKG_NAME + ".quant_gru")
pytestmark = pytest.mark.gpu

FLOAT_RTOL = 1e-5   # north star: float mode within 1e-5 relative error of the fp path


def _t(a, dev):
    import torch
    return torch.from_numpy(np.ascontiguousarray(a)).to(dev)


def _rel_err(got, want):
    return np.abs(got - want).max() / max(np.abs(want).max(), 1e-30)


@pytest.mark.parametrize("shape", [(6, 5, 20, 40), (12, 33, 64, 128), (3, 2, 300, 520)])
def test_float_mode_matches_fp32_reference(oracle, cuda_device, shape):
    T, B, I, H = shape
    rng = np.random.default_rng(5)
    W, R, bw, br = gen_weights(rng, I, H)
    x = gen_x(rng, T, B, I)
    h0 = (rng.standard_normal((B, H)) * 0.3).astype(np.float32)
    want_h, want_v = oracle.forward_float(T, B, I, H, W, R, bw, br, x, h0, want_v=True)
    with gru_ops.Handle(I, H, device=0) as hd:
        h, v = hd.forward_float(*[_t(a, cuda_device) for a in (W, R, bw, br, x)], _t(h0, cuda_device), want_v=True)
    assert _rel_err(h.cpu().numpy(), want_h) <= FLOAT_RTOL
    assert _rel_err(v.cpu().numpy(), want_v) <= FLOAT_RTOL


def test_float_mode_matches_torch_gru(cuda_device):
    """As the reference's own test_non_quantized: same weights in torch.nn.GRU (CPU, fp32)."""
    import torch
    torch.manual_seed(0)
    for bidir, bf in ((False, False), (True, True)):
        ref = torch.nn.GRU(24, 40, batch_first=bf, bidirectional=bidir)
        mine = quant_gru.QuantGRU(24, 40, batch_first=bf, bidirectional=bidir)
        mine.load_state_dict(ref.state_dict())
        x = torch.rand(7, 9, 24) * 1.5 - 0.7
        hx = torch.randn(2 if bidir else 1, 7 if bf else 9, 40) * 0.2
        want_o, want_h = ref(x, hx)
        got_o, got_h = mine.cuda()(x.cuda(), hx.cuda())
        assert _rel_err(got_o.detach().cpu().numpy(), want_o.detach().numpy()) <= FLOAT_RTOL
        assert _rel_err(got_h.detach().cpu().numpy(), want_h.detach().numpy()) <= FLOAT_RTOL


@pytest.mark.parametrize("bidir,bf", [(False, False), (True, True)])
def test_float_mode_trains_like_torch_gru(cuda_device, bidir, bf):
    """Gradients of a loss over output and h_n through QuantGRU (float mode, train()) against
    torch.nn.GRU on the CPU in fp32 with the same weights: parameters, input and hx."""
    import torch
    torch.manual_seed(1)
    I, H = 24, 40
    ref = torch.nn.GRU(I, H, batch_first=bf, bidirectional=bidir)
    mine = quant_gru.QuantGRU(I, H, batch_first=bf, bidirectional=bidir)
    mine.load_state_dict(ref.state_dict())
    mine = mine.cuda().train()
    x = torch.rand(7, 9, I) * 1.5 - 0.7
    hx = torch.randn(2 if bidir else 1, 7 if bf else 9, H) * 0.2
    g_o = torch.randn(7, 9, H * (2 if bidir else 1))
    g_h = torch.randn_like(hx)
    xr, hr = x.clone().requires_grad_(), hx.clone().requires_grad_()
    o, hn = ref(xr, hr)
    ((o * g_o).sum() + (hn * g_h).sum()).backward()
    xm, hm = x.cuda().requires_grad_(), hx.cuda().requires_grad_()
    o2, hn2 = mine(xm, hm)
    ((o2 * g_o.cuda()).sum() + (hn2 * g_h.cuda()).sum()).backward()
    assert _rel_err(o2.detach().cpu().numpy(), o.detach().numpy()) <= FLOAT_RTOL
    assert _rel_err(xm.grad.cpu().numpy(), xr.grad.numpy()) <= 5e-5
    assert _rel_err(hm.grad.cpu().numpy(), hr.grad.numpy()) <= 5e-5
    for (name, p_ref), (_, p_mine) in zip(ref.named_parameters(), mine.named_parameters()):
        assert _rel_err(p_mine.grad.cpu().numpy(), p_ref.grad.numpy()) <= 5e-5, name


def test_minmax_calibration_matches_oracle(oracle, cuda_device):
    """Ranges folded on the GPU vs the CPU fp32 restatement: 1e-5 relative; the params derived
    from them: equal zero points, scales within 1e-5."""
    T, B, I, H = 9, 7, 20, 48
    rng = np.random.default_rng(9)
    W, R, bw, br = gen_weights(rng, I, H)
    batches = [gen_x(rng, T, B, I, "outliers") for _ in range(3)]
    want = params_mod.Ranges(H)
    got = params_mod.Ranges(H)
    with gru_ops.Handle(I, H, device=0) as hd:
        dW = [_t(a, cuda_device) for a in (W, R, bw, br)]
        for xb in batches:
            oracle.forward_float(T, B, I, H, W, R, bw, br, xb, None, ranges=want)
            hd.calibrate_minmax(*dW, _t(xb, cuda_device), got)
    np.testing.assert_allclose(got.min_v[[0, 1] + list(range(6, 17))], want.min_v[[0, 1] + list(range(6, 17))], rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(got.max_v[[0, 1] + list(range(6, 17))], want.max_v[[0, 1] + list(range(6, 17))], rtol=1e-5, atol=1e-6)
    for n in params_mod.WEIGHT_OPS:   # weights are read, not computed: exact
        assert np.array_equal(got.ch_min[n], want.ch_min[n]) and np.array_equal(got.ch_max[n], want.ch_max[n])
    assert got.min_v[OP["x"]] == want.min_v[OP["x"]] and got.max_v[OP["x"]] == want.max_v[OP["x"]]
    for cfg in ("default", "cfg2"):
        pg = params_mod.GRUQuantParams.from_ranges(got, config_named(cfg))
        pw = params_mod.GRUQuantParams.from_ranges(want, config_named(cfg))
        for i in range(17):
            assert abs(pg.c.op[i].zero_point - pw.c.op[i].zero_point) <= 1
            assert abs(pg.c.op[i].scale - pw.c.op[i].scale) <= 1e-5 * pw.c.op[i].scale
        # given the same ranges the derivation is deterministic (checked bit-exact on the CPU)


def test_nan_and_inf_are_skipped_by_calibration(cuda_device):
    T, B, I, H = 3, 2, 8, 8
    rng = np.random.default_rng(1)
    W, R, bw, br = gen_weights(rng, I, H)
    x = gen_x(rng, T, B, I)
    x[0, 0, 0] = np.inf
    r = params_mod.Ranges(H)
    with gru_ops.Handle(I, H, device=0) as hd:
        hd.calibrate_minmax(*[_t(a, cuda_device) for a in (W, R, bw, br, x)], r)
    assert np.isfinite(r.max_v[OP["x"]]) and r.max_v[OP["x"]] == np.max(x[np.isfinite(x)])


def _oracle_module_forward(oracle, mod, x, hx, T, B, float_storage=False):
    """Compose the oracle the way the reference module composes its kernels."""
    I, H = mod.input_size, mod.hidden_size
    outs, hns = [], []
    for d in range(mod.num_directions):
        sfx = "_reverse" if d else ""
        qp = mod.quant_params_reverse if d else mod.quant_params
        W, R, bw, br = [t.cpu().numpy() for t in quant_gru.convert_weights_to_haste_format(
            getattr(mod, "weight_ih_l0" + sfx), getattr(mod, "weight_hh_l0" + sfx),
            getattr(mod, "bias_ih_l0" + sfx), getattr(mod, "bias_hh_l0" + sfx), H, "cpu")]
        wq = oracle.quantize_weights(I, H, W, R, bw, br, qp.c, qp.scale_list())
        xd = x[::-1].copy() if d else x
        h0 = hx[d] if hx is not None else None
        if float_storage:
            h, _ = oracle.forward_fstorage(T, B, I, H, wq, xd, h0, qp.c, qp.scale_list())
        else:
            h = oracle.forward_f32(T, B, I, H, wq, xd, h0, qp.c, qp.scale_list())
        outs.append(h[1:][::-1] if d else h[1:])
        hns.append(h[-1:])
    return np.concatenate(outs, -1), np.concatenate(hns, 0)


@pytest.mark.parametrize("bidir,bf", [(False, False), (True, False), (True, True)])
def test_quantgru_module_end_to_end(oracle, cuda_device, bidir, bf):
    """calibrating=True -> finalize -> quantized forward, against the oracle fed with the
    module's own quant params; then forward_quantized (int32 in / int32 out)."""
    import torch
    torch.manual_seed(3)
    T, B, I, H = 8, 6, 20, 40
    mod = quant_gru.QuantGRU(I, H, batch_first=bf, bidirectional=bidir, quant_storage_dtype="int32").cuda().eval()
    mod.load_bitwidth_config(config_named("cfg2").to_json_dict())
    rng = np.random.default_rng(4)
    mod.calibrating = True
    for _ in range(3):
        xc = gen_x(rng, T, B, I)
        mod(_t(xc.transpose(1, 0, 2) if bf else xc, cuda_device))
    mod.calibrating = False
    mod.use_quantization = True
    x = gen_x(rng, T, B, I)
    hx = (rng.standard_normal((2 if bidir else 1, B, H)) * 0.2).astype(np.float32)
    out, hn = mod(_t(x.transpose(1, 0, 2) if bf else x, cuda_device), _t(hx, cuda_device))
    assert mod.is_calibrated()
    want_o, want_h = _oracle_module_forward(oracle, mod, x, hx, T, B)
    got_o = out.cpu().numpy().transpose(1, 0, 2) if bf else out.cpu().numpy()
    assert np.array_equal(got_o.view(np.uint32), want_o.view(np.uint32))
    assert np.array_equal(hn.cpu().numpy().view(np.uint32), want_h.view(np.uint32))
    # second call reuses the packed weights; a parameter update re-quantizes them
    out2, _ = mod(_t(x.transpose(1, 0, 2) if bf else x, cuda_device), _t(hx, cuda_device))
    assert torch.equal(out, out2)
    with torch.no_grad():
        mod.weight_hh_l0.mul_(0.5)
    out3, _ = mod(_t(x.transpose(1, 0, 2) if bf else x, cuda_device), _t(hx, cuda_device))
    want_o3, _ = _oracle_module_forward(oracle, mod, x, hx, T, B)
    got_o3 = out3.cpu().numpy().transpose(1, 0, 2) if bf else out3.cpu().numpy()
    assert np.array_equal(got_o3.view(np.uint32), want_o3.view(np.uint32))

    # int in / int out
    x_q = oracle.quantize(x, mod.quant_params.c, OP["x"])
    oq, hq = mod.forward_quantized(_t(x_q.transpose(1, 0, 2) if bf else x_q, cuda_device))
    parts = []
    for d in range(mod.num_directions):
        qp = mod.quant_params_reverse if d else mod.quant_params
        h = oracle.dequantize(  # compare through exact dequantization of both sides
            (oq.cpu().numpy().transpose(1, 0, 2) if bf else oq.cpu().numpy())[..., d * H:(d + 1) * H], qp.c, OP["h"])
        parts.append(h)
    want_o, _ = _oracle_module_forward(oracle, mod, x, None, T, B)
    assert np.array_equal(np.concatenate(parts, -1).view(np.uint32), want_o.view(np.uint32))
    assert oq.dtype == torch.int32 and hq.shape == (mod.num_directions, B, H)


def test_quantgru_param_file_round_trip(oracle, cuda_device, tmp_path):
    import torch
    torch.manual_seed(5)
    T, B, I, H = 5, 4, 12, 24
    a = quant_gru.QuantGRU(I, H, bidirectional=True, quant_storage_dtype="int32").cuda().eval()
    a.calibrating = True
    a(torch.randn(T, B, I, device=cuda_device))
    a.calibrating = False
    a.use_quantization = True
    x = torch.randn(T, B, I, device=cuda_device)
    want, _ = a(x)
    path = str(tmp_path / "qp.json")
    a.export_quant_params(path)
    b = quant_gru.QuantGRU(I, H, bidirectional=True, quant_storage_dtype="int32").cuda().eval()
    b.load_state_dict(a.state_dict())
    b.load_quant_params(path)
    got, _ = b(x)
    assert torch.equal(got, want)


@pytest.mark.parametrize("bidir,bf", [(False, False), (True, True)])
def test_quantgru_module_float_storage(oracle, cuda_device, bidir, bf):
    """The module's default quantized mode (quant_storage_dtype="float32": float requantization,
    real sigmoid / tanh) against the oracle's restatement of that path: at most one step of the
    h scale on at most 1 % of the elements (host libm against CUDA's expf / tanhf); the same
    path is bit-exact against the reference's GPU code in test_gpu_vs_reference_gpu.py."""
    import torch
    torch.manual_seed(5)
    T, B, I, H = 8, 6, 20, 40
    mod = quant_gru.QuantGRU(I, H, batch_first=bf, bidirectional=bidir).cuda().eval()
    assert mod.quant_storage_dtype == "float32"
    rng = np.random.default_rng(6)
    mod.calibrating = True
    for _ in range(3):
        xc = gen_x(rng, T, B, I)
        mod(_t(xc.transpose(1, 0, 2) if bf else xc, cuda_device))
    mod.calibrating = False
    mod.use_quantization = True
    x = gen_x(rng, T, B, I)
    hx = (rng.standard_normal((2 if bidir else 1, B, H)) * 0.2).astype(np.float32)
    out, hn = mod(_t(x.transpose(1, 0, 2) if bf else x, cuda_device), _t(hx, cuda_device))
    want_o, want_h = _oracle_module_forward(oracle, mod, x, hx, T, B, float_storage=True)
    got_o = out.cpu().numpy().transpose(1, 0, 2) if bf else out.cpu().numpy()
    for d in range(mod.num_directions):
        qp = mod.quant_params_reverse if d else mod.quant_params
        hs = float(np.float32(qp.c.op[OP["h"]].scale))
        diff = np.abs(np.rint(got_o[..., d * H:(d + 1) * H].astype(np.float64) / hs) -
                      np.rint(want_o[..., d * H:(d + 1) * H].astype(np.float64) / hs))
        assert diff.max() <= 1 and (diff > 0).mean() <= 0.01
    assert hn.shape == (mod.num_directions, B, H)
    assert np.abs(hn.cpu().numpy() - want_h).max() <= 1.01 * hs


@pytest.mark.parametrize("storage", ["float32", "int32"])
def test_quantgru_qat_gradients(oracle, cuda_device, storage):
    """Quantization-aware training through the module: the training forward returns what the
    eval-mode float-storage forward returns, and the gradients are those of the masked backward
    (numpy oracle) applied to the dequantized quantized tensors, gate buffer and clamp masks of
    that forward, mapped back to PyTorch's parameter layout."""
    import torch
    from oracle.backward_np import gru_backward
    torch.manual_seed(7)
    T, B, I, H = 6, 5, 16, 24
    mod = quant_gru.QuantGRU(I, H, quant_storage_dtype=storage).cuda()
    ints = storage == "int32"
    rng = np.random.default_rng(8)
    mod.eval()
    mod.calibrating = True
    for _ in range(2):
        mod(_t(gen_x(rng, T, B, I), cuda_device))
    mod.calibrating = False
    mod.use_quantization = True
    x = gen_x(rng, T, B, I, sigma=2.5)            # wider than calibrated: some clamps
    hx = (rng.standard_normal((1, B, H)) * 0.2).astype(np.float32)
    with torch.no_grad():
        want_o, want_hn = mod(_t(x, cuda_device), _t(hx, cuda_device))
    mod.train()
    xm, hm = _t(x, cuda_device).requires_grad_(), _t(hx, cuda_device).requires_grad_()
    out, hn = mod(xm, hm)
    assert torch.equal(out.detach(), want_o) and torch.equal(hn.detach(), want_hn)
    g_o = torch.randn(T, B, H, device=cuda_device)
    g_h = torch.randn(1, B, H, device=cuda_device)
    ((out * g_o).sum() + (hn * g_h).sum()).backward()

    # the same through the library's pieces and the numpy oracle
    W, R, bw, br = quant_gru.convert_weights_to_haste_format(mod.weight_ih_l0, mod.weight_hh_l0, mod.bias_ih_l0,
                                                             mod.bias_hh_l0, H, cuda_device)
    with gru_ops.Handle(I, H, device=0) as hd:
        hd.set_params(mod.quant_params)
        hd.set_weights_f32(W, R, bw, br)
        h, v, x_q, masks = hd.forward_fstorage_train(W, R, bw, br, _t(x, cuda_device), _t(hx[0], cuda_device),
                                                     int_storage=ints)
        Wd, Rd, _, _ = hd.get_weights_dequantized()
        xd = hd.dequantize_f32(x_q.to(torch.float32), "x")
    dh_new = np.zeros((T + 1, B, H), np.float32)
    dh_new[1:] = g_o.cpu().numpy()
    dh_new[T] += g_h.cpu().numpy()[0]
    dx, dW, dR, dbw, dbr, dh0 = gru_backward(Wd.cpu().numpy(), Rd.cpu().numpy(), xd.cpu().numpy(), dh_new,
                                             h.cpu().numpy(), v.cpu().numpy(),
                                             masks={n: m.cpu().numpy() for n, m in masks.items()})
    re = quant_gru.reorder_weights_pytorch_to_haste
    pairs = [(xm.grad, dx), (hm.grad[0], dh0), (mod.weight_ih_l0.grad, re(torch.from_numpy(dW).t()).numpy()),
             (mod.weight_hh_l0.grad, re(torch.from_numpy(dR).t()).numpy()),
             (mod.bias_ih_l0.grad, re(torch.from_numpy(dbw)).numpy()),
             (mod.bias_hh_l0.grad, re(torch.from_numpy(dbr)).numpy())]
    for k, (got, want) in enumerate(pairs):
        assert _rel_err(got.cpu().numpy(), np.asarray(want)) <= 5e-5, k
    assert any(0 < float(m.float().mean()) < 1 for m in masks.values()), "no clamp was exercised"

    if ints:
        return
    # the reference-named pair of entry points gives the same gradients
    fwd = gru_ops.forward_quant_float_storage(True, T, B, I, H, W, R, bw, br, _t(x, cuda_device),
                                              _t(hx[0], cuda_device), mod.quant_params)
    assert len(fwd) == 18 and torch.equal(fwd[0], h) and torch.equal(fwd[1], v)
    got = gru_ops.backward_quant_float_storage(T, B, I, H, *fwd[2:7], _t(dh_new, cuda_device), fwd[0], fwd[1],
                                               mod.quant_params, *fwd[7:])
    for g, w in zip(got, (dx, dW, dR, dbw, dbr, dh0)):
        assert _rel_err(g.cpu().numpy().reshape(w.shape), w) <= 5e-5


def test_reference_named_quantized_forwards_return_the_reference_tuple(oracle, cuda_device):
    """forward_quant_int_storage / forward_quant_float_storage: 18 results like the binding's;
    inference and training mode give the same h; training fills v and the masks."""
    import torch
    T, B, I, H = 5, 4, 12, 24
    case = make_case(seed=61, T=T, B=B, I=I, H=H, checker=oracle, config=config_named("cfg2"), with_h0=True)
    dev = [_t(a, cuda_device) for a in (case.W, case.R, case.bw, case.br, case.x, case.h0)]
    for fn, xq_dtype in ((gru_ops.forward_quant_int_storage, torch.int32),
                         (gru_ops.forward_quant_float_storage, torch.float32)):
        inf = fn(False, T, B, I, H, *dev, case.params)
        trn = fn(True, T, B, I, H, *dev, case.params)
        assert len(inf) == len(trn) == 18
        assert torch.equal(inf[0], trn[0]) and inf[1].numel() == 0 and trn[1].shape == (T, B, 4 * H)
        assert inf[6].dtype == trn[6].dtype == xq_dtype and torch.equal(inf[6], trn[6])
        assert all(m.numel() == 0 for m in inf[7:]) and all(m.dtype == torch.uint8 and m.numel() > 0 for m in trn[7:])
    want = oracle.forward_f32(T, B, I, H, case.wq, case.x, case.h0, case.params.c, case.params.scale_list())
    got = gru_ops.forward_quant_int_storage(False, T, B, I, H, *dev, case.params)[0]
    assert np.array_equal(got.cpu().numpy().view(np.uint32), want.view(np.uint32))


def test_quantgru_errors(cuda_device):
    import torch
    m = quant_gru.QuantGRU(8, 16, quant_storage_dtype="int32").cuda().eval()
    m.use_quantization = True
    with pytest.raises(RuntimeError):          # not calibrated
        m(torch.randn(3, 2, 8, device=cuda_device))
    with pytest.raises(RuntimeError):
        m.forward_quantized(torch.zeros(3, 2, 8, dtype=torch.int32, device=cuda_device))
    with pytest.raises(NotImplementedError):
        quant_gru.QuantGRU(8, 16, num_layers=2)
    with pytest.raises(ValueError):
        quant_gru.QuantGRU(8, 16, quant_storage_dtype="int8")
    m.calibrating = True
    m(torch.randn(3, 2, 8, device=cuda_device))
    m.calibrating = False
    m.finalize_calibration()
    with pytest.raises(TypeError):             # float input to the int-in/int-out entry
        m.forward_quantized(torch.randn(3, 2, 8, device=cuda_device))
    f = quant_gru.QuantGRU(8, 16, quant_storage_dtype="int32").cuda()   # QAT runs on float32 storage only
    f.calibrating = True
    f(torch.randn(3, 2, 8, device=cuda_device))
    f.calibrating = False
    f.use_quantization = True
    xt = torch.randn(3, 2, 8, device=cuda_device)
    f.eval()
    want = f(xt)
    f.train()
    with torch.no_grad():                      # train() mode without gradients: the inference kernels
        got = f(xt)
    assert torch.equal(got[0], want[0]) and torch.equal(got[1], want[1])


@pytest.mark.parametrize("method", ["sqnr", "percentile"])
def test_quantgru_histogram_flow_needs_no_explicit_finalize(cuda_device, method):
    """calibrating=True; forward(); calibrating=False; forward() - the reference's documented flow
    (pytorch/quant_gru.py:2106-2125) - derives the params on the first quantized forward for the
    histogram methods too, and a second calibration pass replaces them."""
    import torch
    torch.manual_seed(3)
    m = quant_gru.QuantGRU(12, 24, bidirectional=True, quant_storage_dtype="int32").cuda().eval()
    m.calibration_method = method
    m.percentile_value = 99.9
    x = torch.randn(6, 5, 12, device=cuda_device)
    m.calibrating = True
    m(x)
    m.calibrating = False
    m.use_quantization = True
    out1, _ = m(x)                              # no finalize_calibration() call
    assert m.is_calibrated() and torch.isfinite(out1).all()
    ref = quant_gru.QuantGRU(12, 24, bidirectional=True, quant_storage_dtype="int32").cuda().eval()
    ref.load_state_dict(m.state_dict())
    ref.calibration_method, ref.percentile_value = method, 99.9
    ref.calibrating = True
    ref(x)
    ref.calibrating = False
    ref.finalize_calibration()
    ref.use_quantization = True
    out_ref, _ = ref(x)
    assert torch.equal(out1, out_ref)
    scale1 = float(m.quant_params.c.op[OP["x"]].scale)
    m.calibrating = True                        # second pass with wider data: params must follow
    m(x * 4.0)
    m.calibrating = False
    m(x)
    assert float(m.quant_params.c.op[OP["x"]].scale) > scale1
