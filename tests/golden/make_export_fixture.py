"""Generate tests/golden/ref_export_*.json with the reference's OWN exporter code.

The reference's Python module (pytorch/quant_gru.py) needs its compiled CUDA binding at import
time, which cannot be built or loaded without a GPU.  Its quant-param exporter
(_build_operators_dict, pytorch/quant_gru.py:3896-3990), however, is plain Python that only
reads attributes off two objects.  This script imports the unmodified module with a stand-in
for the binding (attribute bags with the binding's attribute names), fills the bags from a
seeded GRUQuantParams of this repository, runs the reference's exporter and writes its output
next to the parameters it was given, so that the CPU suite can hold this library's JSON reader
and writer against a file the reference itself formatted.

    QGRU_REF_ROOT=<reference checkout> python tests/golden/make_export_fixture.py
"""
import json
import os
import sys
import types

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from oracle.binding import REF_ROOT, Oracle  # noqa: E402
from oracle.cases import config_named, make_case, params_mod, _cabi  # noqa: E402


class _Bag:
    """Stand-in for the binding's OperatorQuantConfig / GRUQuantParams objects."""


def _stub_binding():
    m = types.ModuleType("gru_interface_binding")

    def _no_binding(*a, **k):   # the module's import-time self-check skips itself when this raises
        raise RuntimeError("stand-in for the compiled binding")
    m.OperatorQuantConfig = _no_binding
    m.GRUQuantParams = _no_binding
    sys.modules["gru_interface_binding"] = m


def reference_module():
    _stub_binding()
    sys.path.insert(0, os.path.join(REF_ROOT, "pytorch"))
    import warnings
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        import quant_gru as ref   # the reference's module, unmodified
    return ref


def bags_from(params, ref):
    """Binding-style attribute bags of one GRUQuantParams (attribute names: _OPERATOR_MAP)."""
    cfg, qp = _Bag(), _Bag()
    for json_name, info in ref._OPERATOR_MAP.items():
        n = params_mod.JSON_TO_OP[json_name]
        o = params.c.op[_cabi.OP_INDEX[n]]
        setattr(cfg, info["bw_attr"], int(o.bits))
        setattr(cfg, info["sym_attr"], bool(o.symmetric))
        setattr(cfg, info["unsigned_attr"], bool(o.is_unsigned))
        if info["is_per_channel"]:
            setattr(qp, info["scale_attr"], [float(v) for v in params.scales[n]])
        else:
            setattr(qp, info["scale_attr"], float(np.float32(o.scale)))
            setattr(qp, info["zp_attr"], int(o.zero_point))
    for k, n in enumerate(params_mod.WEIGHT_OPS):   # the binding's own granularity attribute names
        setattr(cfg, f"{n}_granularity_", int(params.c.granularity[k]))
    return cfg, qp


def main():
    ref = reference_module()
    orc = Oracle()
    for name, cfg_name, (I, H) in (("cfg2_h8", "cfg2", (6, 8)), ("cfg3_h4", "cfg3", (5, 4))):
        case = make_case(seed=900 + H, T=6, B=3, I=I, H=H, checker=orc, config=config_named(cfg_name))
        cfg, qp = bags_from(case.params, ref)
        doc = {"model_info": {"input_size": I, "hidden_size": H, "bias": True, "batch_first": False,
                              "bidirectional": False, "use_pot2_scale": False},
               "operators": ref._build_operators_dict(cfg, qp)}
        with open(os.path.join(HERE, f"ref_export_{name}.json"), "w", encoding="utf-8") as f:
            json.dump(doc, f, indent=2, ensure_ascii=False)
        with open(os.path.join(HERE, f"ref_export_{name}.params.bin"), "wb") as f:
            f.write(case.params.to_bytes())
        print("wrote", name, list(doc["operators"])[:3], "...")


if __name__ == "__main__":
    main()
