"""Seeded test problems (oracle/cases.py) under the name the tests import them by."""
from oracle.cases import (OP, Case, _cabi, calibrate_minmax, config_named, gen_weights, gen_x,  # noqa: F401
                          make_case, params_mod)
