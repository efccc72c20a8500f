"""The allocation-free entry point (qgru_forward_i32_static) against the ordinary one.

It exists for callers that may not allocate device memory when they call a forward - a serving
loop with a fixed memory budget, a process whose allocator belongs to another framework, a
real-time thread - and keeps its whole workspace in a fixed array inside the library.  That
array is shared by every call on the GPU and keeps the previous call's contents, so the check is
made on two calls in a row (different problems, then the first again).  This file is named to be
collected last: if it fails, `pytest -x` has already run every other test."""
import importlib

import numpy as np
import pytest

from __graft_entry__ import PKG_NAME
from tests.cases import config_named, make_case

gru_ops = importlib.import_module(PKG_NAME + ".gru_ops")
pytestmark = pytest.mark.gpu


def _t(a, dev):
    import torch
    return torch.from_numpy(np.ascontiguousarray(a)).to(dev)


def test_static_workspace_forward_matches_allocating_forward(oracle, cuda_device):
    import torch
    cases = [make_case(101, 7, 6, 24, 48, oracle, config_named("default"), with_h0=True),
             make_case(102, 5, 33, 40, 300, oracle, config_named("cfg2")),      # per-step barrier, 16-bit gates
             make_case(103, 9, 3, 20, 40, oracle, config_named("ih16"))]
    for reverse in (False, True):
        for case in cases + cases[:1]:                      # the last one repeats the first problem
            with gru_ops.Handle(case.I, case.H, device=0) as hd:
                hd.set_params(case.params)
                hd.set_weights_i32(*[_t(w, cuda_device) for w in case.wq])
                x_q = _t(case.x_q, cuda_device)
                h0 = _t(case.h0_q, cuda_device) if case.h0_q is not None else None
                want = hd.forward_i32(x_q, h0, reverse=reverse)
                out1, out2 = torch.empty_like(want), torch.empty_like(want)
                # the first call on a device is the set-up call (the array's address is looked up and the
                # driver loads the code of the kernels it launches): made before free memory is measured
                hd.forward_i32_static(x_q, h0, reverse=reverse, out=out1)
                out1.zero_()
                torch.cuda.synchronize()
                free_before = torch.cuda.mem_get_info()[0]
                first = hd.forward_i32_static(x_q, h0, reverse=reverse, out=out1)
                second = hd.forward_i32_static(x_q, h0, reverse=reverse, out=out2)
                assert torch.cuda.mem_get_info()[0] == free_before      # nothing was allocated
                assert "workspace=static" in hd.describe_plan()
                assert torch.equal(first, want), "first call differs (integer path: tolerance is zero)"
                assert torch.equal(second, want), "second call in a row differs"
            if not reverse:
                ref = oracle.forward_i32(case.T, case.B, case.I, case.H, case.wq, case.x_q, case.h0_q,
                                         case.params.c, case.params.scale_list())
                assert np.array_equal(want.cpu().numpy(), ref)


def test_static_workspace_rejects_oversized_problems(oracle, cuda_device):
    case = make_case(104, 2, 2, 16, 32, oracle, config_named("default"))
    import torch
    with gru_ops.Handle(case.I, case.H, device=0) as hd:
        hd.set_params(case.params)
        hd.set_weights_i32(*[_t(w, cuda_device) for w in case.wq])
        big = torch.zeros((4000, 64, case.I), dtype=torch.int32, device=cuda_device)   # ~62 MB of workspace
        with pytest.raises(ValueError, match="static workspace too small"):
            hd.forward_i32_static(big)
        small = hd.forward_i32_static(_t(case.x_q, cuda_device))                      # still usable
        assert torch.equal(small, hd.forward_i32(_t(case.x_q, cuda_device)))
