"""The tensor-pipe rate probe (qgru_probe_mma_i8) runs and returns plausible figures."""
import importlib

import pytest

from __graft_entry__ import PKG_NAME, load_package

load_package()
gru_ops = importlib.import_module(PKG_NAME + ".gru_ops")

pytestmark = pytest.mark.gpu


def test_probe_mma_rates(cuda_device):
    # the full-width shape sustains far more than the 16-column one, per instruction and in total
    c_wide, t_wide = gru_ops.probe_mma_i8(128, 256, mmas=8192, ctas=148)
    c_thin, t_thin = gru_ops.probe_mma_i8(128, 16, a_in_tmem=True, mmas=8192, ctas=148)
    assert 1.0 < c_thin < c_wide < 10000.0
    assert t_wide > 500.0 and t_wide > t_thin > 1.0


def test_probe_rejects_bad_shapes():
    with pytest.raises(ValueError):
        gru_ops.probe_mma_i8(128, 24)
    with pytest.raises(ValueError):
        gru_ops.probe_mma_i8(128, 256, accumulators=3)
