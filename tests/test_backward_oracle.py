"""CPU test of the backward oracle (oracle/backward_np.py) against torch autograd through
torch.nn.GRU with the same weights: the float backward is the gradient of the float forward."""
import importlib

import numpy as np
import torch

from __graft_entry__ import PKG_NAME
from oracle.backward_np import gru_backward

quant_gru = importlib.import_module(PKG_NAME + ".quant_gru")


def test_backward_oracle_equals_torch_autograd(oracle):
    torch.manual_seed(0)
    T, B, I, H = 6, 4, 10, 12
    gru = torch.nn.GRU(I, H).double()
    x = torch.randn(T, B, I, dtype=torch.float64, requires_grad=True)
    h0 = (torch.randn(1, B, H, dtype=torch.float64) * 0.3).requires_grad_()
    G = torch.randn(T, B, H, dtype=torch.float64)
    out, _ = gru(x, h0)
    (out * G).sum().backward()

    W, R, bw, br = [t.detach().numpy().astype(np.float32) for t in quant_gru.convert_weights_to_haste_format(
        gru.weight_ih_l0.float(), gru.weight_hh_l0.float(), gru.bias_ih_l0.float(), gru.bias_hh_l0.float(), H, "cpu")]
    xf = x.detach().numpy().astype(np.float32)
    h, v = oracle.forward_float(T, B, I, H, W, R, bw, br, xf, h0.detach().numpy()[0].astype(np.float32), want_v=True)
    dh_new = np.concatenate([np.zeros((1, B, H)), G.numpy()], 0).astype(np.float32)
    dx, dW, dR, dbw, dbr, dh = gru_backward(W, R, xf, dh_new, h, v)

    re = quant_gru.reorder_weights_pytorch_to_haste

    def close(got, want, what):
        want = want.detach().numpy()
        err = np.abs(got - want).max() / max(np.abs(want).max(), 1e-30)
        assert err <= 2e-5, (what, err)     # the forward here ran in fp32, torch's in fp64

    close(dx, x.grad, "dx")
    close(dh, h0.grad[0], "dh0")
    close(dW, re(gru.weight_ih_l0.grad).t(), "dW")
    close(dR, re(gru.weight_hh_l0.grad).t(), "dR")
    close(dbw, re(gru.bias_ih_l0.grad), "dbw")
    close(dbr, re(gru.bias_hh_l0.grad), "dbr")


def test_backward_oracle_masks_drop_gradients():
    """Every mask set to one changes nothing; a zero in the h mask of the last step removes that
    cell's contribution."""
    rng = np.random.default_rng(1)
    T, B, I, H = 3, 2, 4, 5
    W = rng.standard_normal((I, 3 * H)).astype(np.float32)
    R = rng.standard_normal((H, 3 * H)).astype(np.float32)
    x = rng.standard_normal((T, B, I)).astype(np.float32)
    h = rng.uniform(-1, 1, (T + 1, B, H)).astype(np.float32)
    v = rng.uniform(0.1, 0.9, (T, B, 4 * H)).astype(np.float32)
    dh_new = rng.standard_normal((T + 1, B, H)).astype(np.float32)
    base = gru_backward(W, R, x, dh_new, h, v)
    ones = {"x": np.ones((T * B, I), np.uint8), "h0": np.ones((B, H), np.uint8), "W": np.ones((I, 3 * H), np.uint8),
            "R": np.ones((H, 3 * H), np.uint8), "bw": np.ones(3 * H, np.uint8), "br": np.ones(3 * H, np.uint8),
            "ih_linear": np.ones((T * B, 3 * H), np.uint8), "hh_linear": np.ones((T * B, 3 * H), np.uint8),
            "gate_input": np.ones((T * B, 3 * H), np.uint8), "gate_output": np.ones((T * B, 3 * H), np.uint8),
            "h": np.ones((T * B, H), np.uint8)}
    same = gru_backward(W, R, x, dh_new, h, v, masks=ones)
    for a, b in zip(base, same):
        assert np.array_equal(a, b)
    ones["h"][:] = 0
    zero = gru_backward(W, R, x, dh_new, h, v, masks=ones)
    assert all(np.all(a == 0) for a in zero)
