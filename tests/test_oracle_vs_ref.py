"""The oracle is pinned here: the C restatement (oracle/qgru_oracle.c) must agree bit for bit
with the unmodified reference sources compiled into oracle/_ref/ on every function it
restates.  Skipped where the reference tree was never compiled (then tests/golden/ pins it)."""
import numpy as np
import pytest

from tests.cases import OP, config_named, make_case

CONFIGS = ["default", "sym8_tensor", "cfg2", "cfg3", "cfg5", "pot2", "pot2_asym", "ih16", "wide16",
           "gate_in16", "unsigned_x"]


def test_rshift_round_and_encode(oracle, reference):
    rng = np.random.default_rng(0)
    for _ in range(5000):
        x = int(rng.integers(-2 ** 45, 2 ** 45))
        n = int(rng.integers(-6, 50))
        assert oracle.rshift_round(x, n) == reference.rshift_round(x, n)
    # the survey's known answers (banker's rounding on the magnitude, negative n = left shift)
    for (x, n, want) in [(5, 1, 2), (7, 1, 4), (-5, 1, -2), (3, -2, 12), (6, 2, 2), (10, 2, 2), (-6, 2, -2)]:
        assert oracle.rshift_round(x, n) == want == reference.rshift_round(x, n)
    for _ in range(5000):
        s = float(np.float32(10 ** rng.uniform(-9, 4)))
        assert oracle.encode_mshift(s) == reference.encode_mshift(s)
    assert oracle.encode_mshift(42.0) == (43008, 10) == reference.encode_mshift(42.0)
    assert oracle.encode_mshift(2.0 ** -7) == (32768, 22) == reference.encode_mshift(2.0 ** -7)
    assert oracle.encode_mshift(0.0) is None and reference.encode_mshift(0.0) is None
    assert oracle.encode_mshift(-1.0) is None and reference.encode_mshift(-1.0) is None


@pytest.mark.parametrize("name", CONFIGS)
def test_params_quantize_forward(oracle, reference, name):
    for seed, (T, B, I, H) in enumerate([(7, 5, 12, 24), (3, 1, 9, 8), (5, 3, 33, 40)]):
        cr = make_case(seed, T, B, I, H, reference, config_named(name), with_h0=(seed == 1), oracle=oracle)
        co = make_case(seed, T, B, I, H, oracle, config_named(name), with_h0=(seed == 1), oracle=oracle)
        assert bytes(cr.params.c) == bytes(co.params.c), "scales / zero points / LUTs differ"
        for a, b in zip(cr.params.scale_list(), co.params.scale_list()):
            assert np.array_equal(a, b)
        for a, b in zip(cr.wq, co.wq):
            assert np.array_equal(a, b)
        assert np.array_equal(cr.x_q, co.x_q)
        args = (cr.T, cr.B, cr.I, cr.H, cr.wq)
        sc = cr.params.scale_list()
        hr = reference.forward_i32(*args, cr.x_q, cr.h0_q, cr.params.c, sc)
        ho = oracle.forward_i32(*args, cr.x_q, cr.h0_q, cr.params.c, sc)
        assert np.array_equal(hr, ho)
        fr = reference.forward_f32(*args, cr.x, cr.h0, cr.params.c, sc)
        fo = oracle.forward_f32(*args, cr.x, cr.h0, cr.params.c, sc)
        assert np.array_equal(fr, fo)
        assert np.array_equal(reference.dequantize(hr, cr.params.c, OP["h"]), fr)


def test_multithreaded_slices_are_identical(oracle, reference):
    c = make_case(3, 6, 11, 10, 16, oracle, config_named("cfg2"), with_h0=True)
    sc = c.params.scale_list()
    one = oracle.forward_i32(c.T, c.B, c.I, c.H, c.wq, c.x_q, c.h0_q, c.params.c, sc)
    for chk in (oracle, reference):
        for th in (2, 4, 11, 16):
            got = chk.forward_i32(c.T, c.B, c.I, c.H, c.wq, c.x_q, c.h0_q, c.params.c, sc, threads=th)
            assert np.array_equal(got, one)


def test_lut_eval_whole_domain(oracle, reference):
    c = make_case(5, 4, 4, 8, 16, reference, config_named("cfg2"), oracle=oracle)
    p = c.params.c
    for lut, i_in, i_out in ((0, OP["update_gate_input"], OP["update_gate_output"]),
                             (1, OP["reset_gate_input"], OP["reset_gate_output"]),
                             (2, OP["new_gate_input"], OP["new_gate_output"])):
        for q in range(-300, 300):
            assert oracle.lut_eval(p.lut[lut], q, p.op[i_in], p.op[i_out]) == \
                reference.lut_eval(p.lut[lut], q, p.op[i_in], p.op[i_out])


def test_training_buffer_matches_reference(oracle, reference):
    """v_q (gate outputs and the new gate's R*h row) of the training-mode CPU forward."""
    for seed, cfg in enumerate(("default", "cfg2", "pot2_asym", "wide16")):
        case = make_case(70 + seed, 5, 3, 12, 20, reference, config_named(cfg), with_h0=bool(seed & 1))
        args = (case.T, case.B, case.I, case.H, case.wq, case.x_q, case.h0_q, case.params.c, case.params.scale_list())
        h_r, v_r = reference.forward_i32_v(*args)
        h_o, v_o = oracle.forward_i32_v(*args)
        assert np.array_equal(h_r, h_o) and np.array_equal(v_r, v_o)
        assert np.array_equal(h_o, oracle.forward_i32(*args))


def test_training_masks_of_the_oracle(oracle, reference):
    """The reference's CPU path writes no clamp masks, so on the CPU the oracle's masks are held
    against what they must imply: same h_q and v_q as the plain training forward, and wherever a
    mask is 0 the clamped value sits on a bound of its range (the GPU tests compare the masks
    themselves with the reference's GPU path)."""
    from tests.cases import gen_x
    case = make_case(91, 6, 4, 12, 20, reference, config_named("default"))
    p = case.params.c
    x_q = reference.quantize(gen_x(np.random.default_rng(4), 6, 4, 12, sigma=5.0), p, OP["x"])
    args = (case.T, case.B, case.I, case.H, case.wq, x_q, None, p, case.params.scale_list())
    h, v, m = oracle.forward_i32_train(*args)
    h_r, v_r = reference.forward_i32_v(*args)
    assert np.array_equal(h, h_r) and np.array_equal(v, v_r)
    H = case.H

    def bounds(name):
        o = p.op[OP[name]]
        lo = 0 if o.is_unsigned else -(1 << (o.bits - 1))
        return lo, lo + (1 << o.bits) - 1

    lo, hi = bounds("h")
    clamped = m[4].reshape(case.T, case.B, H) == 0
    assert np.all((h[1:][clamped] == lo) | (h[1:][clamped] == hi))
    gate_out = m[3].reshape(case.T, case.B, 3 * H)
    for g, name in enumerate(("update_gate_output", "reset_gate_output", "new_gate_output")):
        lo, hi = bounds(name)
        vals = v[:, :, g * H:(g + 1) * H][gate_out[:, :, g * H:(g + 1) * H] == 0]
        assert np.all((vals == lo) | (vals == hi))
    assert all(set(np.unique(a)) <= {0, 1} for a in m)
    assert m[0].mean() < 1.0, "inputs five times wider than calibrated must clamp W*x somewhere"
