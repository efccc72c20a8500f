"""CPU-only checks of the product library: it loads, exports every symbol include/qgru.h
declares, and its host-side helpers (scale encoding, LUT generation, MinMax parameter
derivation) agree bit for bit with the oracle and, where built, the reference."""
import ctypes as C
import importlib
import os
import re

import numpy as np
import pytest

from __graft_entry__ import PKG_NAME
from tests.cases import OP, config_named, make_case, params_mod

_cabi = importlib.import_module(PKG_NAME + "._cabi")
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    hdr = open(os.path.join(ROOT, "include", "qgru.h")).read()
    declared = set(re.findall(r"QGRU_API\s+[\w\s\*]+?\b(qgru_\w+)\s*\(", hdr))
    assert len(declared) >= 25
    assert declared == set(_cabi.SYMBOLS), declared ^ set(_cabi.SYMBOLS)
    lib = _cabi.lib()
    for name in declared:
        assert getattr(lib, name) is not None
    assert lib.qgru_version().decode().startswith("qgru-b200")
    assert lib.qgru_status_string(3).decode() == "device-side wait timed out"


def test_struct_sizes_match_header():
    assert C.sizeof(_cabi.Op) == 12
    assert C.sizeof(_cabi.LutSegment) == 16
    assert C.sizeof(_cabi.Lut) == 16 * 16 + 16
    assert C.sizeof(_cabi.Params) == 8 + 17 * 12 + 16 + 3 * 272


def test_create_without_gpu_fails_loudly():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    h = C.c_void_p()
    assert _cabi.lib().qgru_create(C.byref(h), 0, 8, 8) == _cabi.QGRU_ERR_CUDA
    assert not h.value


def test_host_primitives_match_oracle(oracle):
    lib = _cabi.lib()
    rng = np.random.default_rng(1)
    for _ in range(5000):
        x = int(rng.integers(-2 ** 45, 2 ** 45))
        n = int(rng.integers(-6, 50))
        assert lib.qgru_rshift_round(x, n) == oracle.rshift_round(x, n)
    for _ in range(5000):
        s = float(np.float32(10 ** rng.uniform(-9, 4)))
        m, sh = C.c_uint16(), C.c_int8()
        st = lib.qgru_encode_mshift(C.c_float(s), C.byref(m), C.byref(sh))
        want = oracle.encode_mshift(s)
        assert (st == 0 and (m.value, sh.value) == want) or (st == _cabi.QGRU_ERR_RANGE and want is None)
    m, sh = C.c_uint16(), C.c_int8()
    assert lib.qgru_encode_mshift(C.c_float(0.0), C.byref(m), C.byref(sh)) == _cabi.QGRU_ERR_RANGE


def test_apply_rescale_fast_form_matches_oracle(oracle):
    """The shift-free form (x * (M << k), rounding on the high word) against the oracle's
    rshift_round(x * M, n): ties, signs, POT2 (M = 1) and shifts outside the form's range."""
    lib = _cabi.lib()
    rng = np.random.default_rng(7)
    checked = 0
    for _ in range(20000):
        u = rng.random()
        mult = 1 if u < 0.2 else (32768 + 16384 * int(rng.integers(0, 2))) if u < 0.4 else int(rng.integers(32768, 65536))
        n = int(rng.integers(1, 52))
        if rng.random() < 0.3:
            # an exact tie: x * mult = (2k + 1) * 2^(n-1)
            k = int(rng.integers(-2 ** 12, 2 ** 12))
            num = (2 * k + 1) << (n - 1)
            if num % mult:
                continue
            x = num // mult
        else:
            x = int(rng.integers(-2 ** 31, 2 ** 31))
        want = oracle.rshift_round(x * mult, n)
        if not (-2 ** 31 <= x < 2 ** 31) or not (-2 ** 31 <= want < 2 ** 31):
            continue
        assert lib.qgru_apply_rescale(x, mult, n) == want, (x, mult, n)
        checked += 1
    assert checked > 10000


@pytest.mark.parametrize("name", ["default", "sym8_tensor", "cfg2", "cfg3", "cfg5", "pot2", "pot2_asym",
                                  "wide16", "gate_in16"])
def test_params_from_ranges_and_luts_match(oracle, name):
    from oracle.binding import reference_or_none
    checkers = [oracle] + ([reference_or_none()] if reference_or_none() else [])
    for seed, (T, B, I, H) in enumerate([(6, 4, 10, 16), (4, 2, 7, 40)]):
        case = make_case(seed, T, B, I, H, oracle, config_named(name))
        rng = np.random.default_rng(seed)
        ranges = params_mod.Ranges(H)
        oracle.forward_float(T, B, I, H, case.W, case.R, case.bw, case.br,
                             rng.standard_normal((T, B, I)).astype(np.float32), None, ranges=ranges)
        mine = params_mod.GRUQuantParams.from_ranges(ranges, config_named(name))
        for chk in checkers:
            theirs = params_mod.GRUQuantParams(H, config_named(name))
            sc = chk.calc_params_from_ranges(ranges, theirs.c)
            assert bytes(mine.c) == bytes(theirs.c), f"{chk.kind}: params/LUTs differ"
            for a, b in zip(mine.scale_list(), sc):
                assert np.array_equal(a, b)
        # LUT evaluation over the clamped domain and beyond
        lib = _cabi.lib()
        p = mine.c
        for lut, i_in, i_out in ((0, OP["update_gate_input"], OP["update_gate_output"]),
                                 (2, OP["new_gate_input"], OP["new_gate_output"])):
            for q in list(range(-260, 260, 3)) + [-40000, 40000]:
                assert lib.qgru_lut_eval(C.byref(p.lut[lut]), q, C.byref(p.op[i_in]), C.byref(p.op[i_out])) == \
                    oracle.lut_eval(p.lut[lut], q, p.op[i_in], p.op[i_out])


def test_asymmetric_weights_are_rejected(oracle):
    cfg = config_named("default")
    cfg.symmetric["W"] = False
    ranges = params_mod.Ranges(8)
    ranges.min_v[:] = -1
    ranges.max_v[:] = 1
    for n in params_mod.WEIGHT_OPS:
        ranges.ch_min[n][:] = -1
        ranges.ch_max[n][:] = 1
    with pytest.raises(Exception):
        params_mod.GRUQuantParams.from_ranges(ranges, cfg)


def test_bitwidth_json_round_trip(tmp_path):
    import json
    cfg = config_named("cfg5")
    path = tmp_path / "bw.json"
    path.write_text(json.dumps(cfg.to_json_dict()))
    back = params_mod.OperatorQuantConfig.from_json(str(path))
    assert back.bits == cfg.bits and back.symmetric == cfg.symmetric and back.unsigned == cfg.unsigned
    assert back.granularity == cfg.granularity and back.use_pot2 == cfg.use_pot2
    # legacy aliases and error behaviour of the reference's loader
    d = cfg.to_json_dict()
    d["GRU_config"]["operator_config"]["W"] = d["GRU_config"]["operator_config"].pop("weight_ih")
    assert params_mod.OperatorQuantConfig.from_json(d).bits["W"] == 4
    d["GRU_config"]["operator_config"]["bogus"] = {"bitwidth": 8}
    with pytest.raises(ValueError):
        params_mod.OperatorQuantConfig.from_json(d)
    d["GRU_config"]["operator_config"].pop("bogus")
    d["GRU_config"]["operator_config"]["input"]["bitwidth"] = 40
    with pytest.raises(ValueError):
        params_mod.OperatorQuantConfig.from_json(d)


def test_reference_shipped_bitwidth_json_loads():
    from oracle.binding import REF_ROOT
    path = os.path.join(REF_ROOT, "pytorch", "config", "gru_quant_bitwidth_config.json")
    if not os.path.exists(path):
        pytest.skip("reference tree not present")
    cfg = params_mod.OperatorQuantConfig.from_json(path)
    assert cfg.bits["x"] == 8 and cfg.unsigned["update_gate_output"] and cfg.symmetric["x"]


def test_quant_param_export_round_trip(oracle):
    case = make_case(2, 5, 3, 9, 12, oracle, config_named("cfg2"))
    d = case.params.to_export_dict()
    assert d["weight_ih"]["enc_type"] == "PER_CHANNEL" and len(d["weight_ih"]["scale"]) == 36
    assert d["update_gate_output"]["dtype"] == "UINT16"
    back = params_mod.GRUQuantParams.from_export_dict(d, 12, use_pot2=False)
    back.c.granularity[:] = case.params.c.granularity[:]
    assert bytes(back.c) == bytes(case.params.c)
    for a, b in zip(back.scale_list(), case.params.scale_list()):
        assert np.array_equal(a, b)
    blob = case.params.to_bytes()
    again = params_mod.GRUQuantParams.from_bytes(blob, 12)
    assert bytes(again.c) == bytes(case.params.c)


@pytest.mark.parametrize("name,hidden", [("cfg2_h8", 8), ("cfg3_h4", 4)])
def test_quant_param_file_written_by_the_reference_exporter(name, hidden):
    """tests/golden/ref_export_*.json were formatted by the reference's own exporter
    (_build_operators_dict, run by tests/golden/make_export_fixture.py) from the parameters
    stored beside them: this library's reader gives those parameters back, and its writer
    produces the same document, key order and number formatting included."""
    import json
    here = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
    with open(os.path.join(here, f"ref_export_{name}.json"), encoding="utf-8") as f:
        text = f.read()
    doc = json.loads(text)
    with open(os.path.join(here, f"ref_export_{name}.params.bin"), "rb") as f:
        want = params_mod.GRUQuantParams.from_bytes(f.read(), hidden)
    got = params_mod.GRUQuantParams.from_export_dict(doc["operators"], hidden,
                                                     bool(doc["model_info"]["use_pot2_scale"]))
    for i in range(len(want.c.op)):
        a, b = got.c.op[i], want.c.op[i]
        assert (a.scale, a.zero_point, a.bits, a.is_unsigned, a.symmetric) == \
               (b.scale, b.zero_point, b.bits, b.is_unsigned, b.symmetric), i
    for a, b in zip(got.scale_list(), want.scale_list()):
        assert np.array_equal(a, b)
    assert bytes(got.c.lut[0]) == bytes(want.c.lut[0])      # LUTs are regenerated from the loaded scales
    ours = want.to_export_dict()
    ref_ops = doc["operators"]
    assert set(ours) == set(ref_ops)
    for k in ref_ops:
        assert ours[k] == ref_ops[k], k
        assert list(ours[k]) == list(ref_ops[k]), k          # field order inside an operator


def test_quant_param_import_accepts_the_reference_parsers_other_encodings():
    """_parse_runtime_scale_lists (pytorch/quant_gru.py:4008-4045): one-element lists for scalar
    operators, multiplier + shift, the old power-of-two fields; enc_type PER_TENSOR / PER_GATE."""
    import json
    H = 4
    base = {"dtype": "INT8", "symmetric": True}
    with open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "ref_export_cfg3_h4.json"),
              encoding="utf-8") as f:
        ops = json.load(f)["operators"]        # a complete file; some operators re-encoded below
    ops.update({"input": dict(base, scale=[0.5], zero_point=[3]),
           "output": dict(base, multiplier=40000, shift=20, zero_point=-2),
           "weight_ih_linear": dict(base, n=5, zero_point=0),
           "weight_ih": dict(base, scale=0.25, enc_type="PER_TENSOR"),
           "weight_hh": dict(base, scale=[0.5, 0.25, 0.125], enc_type="PER_GATE"),
           "bias_ih": dict(base, multiplier=[32768] * 12, shift=[20] * 12)})
    p = params_mod.GRUQuantParams.from_export_dict(ops, H)
    assert p.c.op[OP["x"]].scale == 0.5 and p.c.op[OP["x"]].zero_point == 3
    assert p.c.op[OP["h"]].scale == np.float32(40000 * 2.0 ** -20) and p.c.op[OP["h"]].zero_point == -2
    assert p.c.op[OP["weight_ih_linear"]].scale == 2.0 ** -5
    assert np.all(p.scales["W"] == 0.25) and list(p.scales["R"]) == [0.5] * 4 + [0.25] * 4 + [0.125] * 4
    assert np.all(p.scales["bw"] == np.float32(2.0 ** -5))
    for bad in (dict(base, scale=[0.5, 0.25], enc_type="PER_GATE"), dict(base, scale=-1.0), dict(base)):
        with pytest.raises(ValueError):
            params_mod.GRUQuantParams.from_export_dict({"weight_ih": bad}, H)


def test_tie_free_ranges_round_half_up_like_half_even():
    """qgru_rescale_can_tie: exhaustive on small ranges (it says "tie possible" exactly when some x
    in the range makes round-half-up differ from the reference's rounding ... or hits an even
    quotient tie, where both agree), and where it says "no tie" the cheap rounding equals
    qgru_apply_rescale on every x of the range."""
    lib = _cabi.lib()
    rng = np.random.default_rng(5)
    checked_free = 0
    for _ in range(400):
        mult = int(rng.integers(32768, 65536)) if rng.random() < 0.7 else int(1 << rng.integers(0, 16)) * int(rng.integers(1, 4))
        mult = min(mult, 65535)
        shift = int(rng.integers(17, 40))
        lo = int(rng.integers(-3000, 0)) * int(rng.integers(1, 300))
        hi = lo + int(rng.integers(1, 4000))
        can = bool(lib.qgru_rescale_can_tie(mult, shift, lo, hi))
        xs = np.arange(lo, hi + 1, dtype=np.int64)
        rem = (xs * mult) % (1 << shift)
        has_tie = bool(np.any(rem == (1 << (shift - 1))))
        assert can == has_tie, (mult, shift, lo, hi)
        if not can:
            for x in xs[:: max(1, len(xs) // 200)]:
                assert lib.qgru_apply_rescale_half_up(int(x), mult, shift) == lib.qgru_apply_rescale(int(x), mult, shift)
            checked_free += 1
    assert checked_free > 50
    # a tie that round-half-up gets wrong is reported: 3 * 2^15 / 2^16 = 1.5 -> 2 (even), 1 * 2^15 / 2^16 = 0.5 -> 0
    assert lib.qgru_rescale_can_tie(32768, 16, 1, 1) == 1
    assert lib.qgru_apply_rescale(1, 32768, 16) == 0 and lib.qgru_rshift_round(1 * 32768, 16) == 0


def test_decode_effective_scale_matches_encoding(oracle):
    """qgru_decode_effective_scale == multiplier * 2^-shift of encodeMShift (POT2: 2^-round(-log2 s))."""
    import importlib
    from __graft_entry__ import PKG_NAME
    gru_ops = importlib.import_module(PKG_NAME + ".gru_ops")
    rng = np.random.default_rng(0)
    for s in list(10.0 ** rng.uniform(-6, 1, 200)) + [1.0, 0.5, 0.0078125]:
        m, sh = oracle.encode_mshift(float(np.float32(s)))
        assert gru_ops.decode_effective_scale(s, False) == float(np.float32(m) * np.float32(2.0) ** np.float32(-sh))
        assert gru_ops.decode_effective_scale(s, True) == 2.0 ** -round(-np.log2(float(np.float32(s))))
    with pytest.raises(ValueError):
        gru_ops.decode_effective_scale(0.0, False)
