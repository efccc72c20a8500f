"""The compiled reference-side binding (quant-gru-pytorch_b200/shim/gru_interface_b200.cc): the
three integer forward entry points with the reference's own signatures
(include/gru_interface.h:266, 305, 389), taking a real GRUQuantParams, held against the
reference's CPU integer path on the same operands.  The params are derived by the reference's
own calculateGRUQuantitativeParameters (through oracle/_ref), so the field-by-field
marshalling GRUQuantParams -> qgru_params is what is under test."""
import os

import numpy as np
import pytest

from tests.cases import config_named, make_case

pytestmark = pytest.mark.gpu

_SO = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle", "_ref", "libqgru_shimtest.so")


@pytest.fixture(scope="module")
def shim(cuda_device):
    if not os.path.exists(_SO):
        pytest.skip("oracle/_ref/libqgru_shimtest.so not built (needs the reference's headers)")
    from oracle.binding import ShimTest
    return ShimTest()


@pytest.mark.parametrize("cfg,shape", [("cfg2", (7, 20, 48, 512)), ("sym8_tensor", (5, 3, 20, 40)),
                                       ("cfg3", (6, 70, 24, 256)), ("cfg5", (9, 1, 80, 256)),
                                       ("pot2", (4, 9, 16, 130)), ("wide16", (3, 4, 12, 24))])
def test_shim_int32_matches_reference_cpu(shim, reference, oracle, cfg, shape):
    T, B, I, H = shape
    case = make_case(seed=300 + T, T=T, B=B, I=I, H=H, checker=reference, config=config_named(cfg), with_h0=True,
                     oracle=oracle)
    sc = case.params.scale_list()
    want = reference.forward_i32(T, B, I, H, case.wq, case.x_q, case.h0_q, case.params.c, sc)
    got = shim.forward_i32(T, B, I, H, case.wq, case.x_q, case.h0_q, case.params.c, sc)
    assert np.array_equal(got, want)
    got2 = shim.forward_i32(T, B, I, H, case.wq, case.x_q, None, case.params.c, sc)   # h0 = nullptr -> zero point
    assert np.array_equal(got2, reference.forward_i32(T, B, I, H, case.wq, case.x_q, None, case.params.c, sc))


def test_shim_training_buffers_match_reference_cpu(shim, reference, oracle):
    T, B, I, H = 5, 6, 16, 40
    case = make_case(seed=311, T=T, B=B, I=I, H=H, checker=reference, config=config_named("cfg2"), oracle=oracle)
    sc = case.params.scale_list()
    h, v, masks = shim.forward_i32(T, B, I, H, case.wq, case.x_q, None, case.params.c, sc, training=True)
    want_h, want_v = reference.forward_i32_v(T, B, I, H, case.wq, case.x_q, None, case.params.c, sc)
    assert np.array_equal(h, want_h) and np.array_equal(v, want_v)
    assert all(m.min() >= 0 and m.max() <= 1 for m in masks) and masks[4].mean() > 0.5


def test_shim_float_and_intio_entry_points(shim, reference, oracle):
    T, B, I, H = 6, 10, 32, 128
    case = make_case(seed=312, T=T, B=B, I=I, H=H, checker=reference, config=config_named("cfg2"), with_h0=True,
                     oracle=oracle)
    sc = case.params.scale_list()
    h, wq, x_q = shim.forward_f32(T, B, I, H, case.W, case.R, case.bw, case.br, case.x, case.h0, case.params.c, sc)
    for a, b in zip(wq, case.wq):
        assert np.array_equal(a, b)            # quantitativeWeight: W_q_out ... br_q_out
    assert np.array_equal(x_q, case.x_q)
    want = reference.forward_f32(T, B, I, H, case.wq, case.x, case.h0, case.params.c, sc)
    assert np.array_equal(h.view(np.uint32), want.view(np.uint32))
    hq = shim.forward_intio(T, B, I, H, case.W, case.R, case.bw, case.br, case.x_q, case.h0_q, case.params.c, sc)
    assert np.array_equal(hq, reference.forward_i32(T, B, I, H, case.wq, case.x_q, case.h0_q, case.params.c, sc))


def test_shim_turns_status_codes_into_the_reference_exceptions(shim, reference, oracle):
    T, B, I, H = 3, 2, 8, 16
    case = make_case(seed=313, T=T, B=B, I=I, H=H, checker=reference, oracle=oracle)
    sc = case.params.scale_list()
    bad = type(case.params.c)()
    import ctypes
    ctypes.memmove(ctypes.byref(bad), ctypes.byref(case.params.c), ctypes.sizeof(bad))
    bad.op[2].symmetric = 0                     # asymmetric W: ensureSymmetricWeightBiasConfig throws invalid_argument
    with pytest.raises(ValueError):
        shim.forward_i32(T, B, I, H, case.wq, case.x_q, None, bad, sc)
