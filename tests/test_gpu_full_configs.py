"""Parity at the five benchmark configurations themselves, full size.

Each test builds the workload exactly as bench.py does (bench.Job: seeded weights, the
configuration's own calibration method and batch count on the GPU, the plan the library
picks for the full shape), runs the forward bench.py times and compares every timestep of
the checked rows bit for bit with the reference's CPU integer path
(cpu::ForwardPassQuantCPU::Run, src/gru_forward_cpu_quant.cc:290-340, compiled unmodified
into oracle/_ref; the C restatement where that library is absent) run on exactly those rows.
Rows never interact, so a row subset of the full-batch GPU result is a complete check of
those rows.  The plan string is asserted, so that the test fails if the benchmark's shape
silently moves to another kernel.
"""
import os

import pytest

pytestmark = pytest.mark.gpu

# workload -> (rows compared per direction (0 = all), substrings the plan must contain)
FULL = {
    "cfg1": (0, ["path=int8", "gemm=tcgen05_i8", "rec=gemv"]),
    "cfg2": (0, ["path=int8", "gemm=tcgen05_i8", "rec=tcgen05_i8", "exchange=cluster_dsmem", "cell=fused_shiftfree"]),
    "cfg3": (96, ["path=int8", "gemm=tcgen05_i8", "rec=tcgen05_i8", "exchange=cluster_dsmem"]),
    "cfg4": (0, ["path=int8", "gemm=tcgen05_i8", "rec=tcgen05_i8", "exchange=cluster_dsmem", "P=8"]),
    "cfg5": (0, ["path=int8", "gemm=tcgen05_i8", "rec=gemv"]),
}


@pytest.mark.parametrize("name", sorted(FULL))
def test_full_size_config_bit_exact(cuda_device, name):
    import torch
    import bench
    rows_checked, plan_parts = FULL[name]
    B = bench.WORKLOADS[name][2]
    job = bench.Job(None, name, torch, cuda_device, 0, 0, 1, B)
    try:
        threads = os.cpu_count() or 1
        res = job.check(rows_checked or B, threads)
        plan = job.plan()
        for part in plan_parts:
            assert part in plan, f"{name}: plan '{plan}' lacks '{part}'"
        want = (rows_checked or B) * len(job.handles)
        assert res["rows"] >= min(want, B * len(job.handles)) and res["steps"] == bench.WORKLOADS[name][3]
        assert res["mismatches"] == 0, f"{name}: {res['mismatches']} values differ from the {res['kind']} CPU path ({plan})"
        # a second run on the same handles gives the same bits (no state left behind by the first)
        res2 = job.check(min(32, B), threads)
        assert res2["mismatches"] == 0
    finally:
        job.close()
