"""Parity of the CUDA path with the oracle, through the C ABI, bit for bit.

Every case is built on the CPU (seeded floats -> MinMax calibration -> quantized operands),
run once by the oracle and once by libqgru_b200.so on cuda:0, and compared with array_equal:
every timestep of h_q, hence `output` and `h_n`."""
import importlib

import numpy as np
import pytest

from __graft_entry__ import PKG_NAME
from tests.cases import config_named, make_case

gru_ops = importlib.import_module(PKG_NAME + ".gru_ops")
pytestmark = pytest.mark.gpu

SHAPES = [  # (T, B, I, H)
    (6, 5, 20, 40),      # nothing a multiple of anything
    (1, 1, 1, 1),        # degenerate
    (3, 2, 7, 8),
    (9, 33, 64, 128),    # config-1 shape, shortened
    (5, 70, 48, 96),
    (4, 3, 80, 256),     # H = 256: R exactly fills one CTA's shared memory
    (3, 17, 33, 300),    # ragged H above 256: two CTAs per group, per-step barrier
    (4, 40, 64, 512),    # config-2 hidden size: eight CTAs per group
]
CONFIGS = ["default", "sym8_tensor", "cfg2", "cfg3", "cfg5", "pot2", "pot2_asym", "ih16", "gate_in16",
           "unsigned_x"]


def _t(a, dev):
    import torch
    return torch.from_numpy(np.ascontiguousarray(a)).to(dev)


def _run(case, dev, reverse=False, opts=(), f32=False, host=False):
    import torch
    with gru_ops.Handle(case.I, case.H, device=dev.index or 0) as hd:
        for k, v in opts:
            hd.set_option(k, v)
        hd.set_params(case.params)
        hd.set_weights_i32(*[_t(a, dev) for a in case.wq])
        if f32:
            if host:
                out = hd.forward_f32_host(torch.from_numpy(case.x), torch.from_numpy(case.h0) if case.h0 is not None else None, reverse=reverse)
            else:
                out = hd.forward_f32(_t(case.x, dev), _t(case.h0, dev) if case.h0 is not None else None, reverse=reverse)
        elif host:
            out = hd.forward_i32_host(torch.from_numpy(case.x_q), torch.from_numpy(case.h0_q) if case.h0_q is not None else None, reverse=reverse)
        else:
            out = hd.forward_i32(_t(case.x_q, dev), _t(case.h0_q, dev) if case.h0_q is not None else None, reverse=reverse)
        plan = hd.describe_plan()
        launches = hd.launch_count()
    return out.cpu().numpy(), plan, launches


def _want(oracle, case):
    return oracle.forward_i32(case.T, case.B, case.I, case.H, case.wq, case.x_q, case.h0_q, case.params.c,
                              case.params.scale_list())


@pytest.mark.parametrize("rec", ["dp4a", "gemv", "mma_cluster", "mma_cluster_smem", "mma_global"])
@pytest.mark.parametrize("shape", SHAPES)
def test_shapes_default_config(oracle, cuda_device, shape, rec):
    """The dp4a recurrence and the tcgen05 recurrence with both ways of exchanging the state
    (distributed shared memory in a cluster, global counter) on every shape; tcgen05 GEMM."""
    T, B, I, H = shape
    if rec == "gemv" and H > 256:
        pytest.skip("the one-CTA-per-row form keeps all of R in one SM: H <= 256")
    case = make_case(11, T, B, I, H, oracle, config_named("default"))
    opts = {"dp4a": (("rec", "dp4a"),), "gemv": (("rec", "gemv"),), "mma_cluster": (("rec", "mma"), ("exchange", "cluster")),
            "mma_cluster_smem": (("rec", "mma"), ("exchange", "cluster"), ("r_resident", "smem")),
            "mma_global": (("rec", "mma"), ("exchange", "global"))}[rec]
    got, plan, launches = _run(case, cuda_device, opts=opts)
    assert "path=int8" in plan and launches > 0
    assert ("rec=tcgen05_i8" in plan) == (rec not in ("dp4a", "gemv")) and "gemm=tcgen05_i8" in plan
    assert ("rec=gemv" in plan) == (rec == "gemv")
    if rec not in ("dp4a", "gemv"):
        assert ("exchange=cluster_dsmem" in plan) == rec.startswith("mma_cluster")
    if rec.startswith("mma_cluster"):   # the R slice sits in tensor memory unless told otherwise
        assert ("r_in=tmem" in plan) == (rec == "mma_cluster")
    assert np.array_equal(got, _want(oracle, case)), plan
    if rec == "gemv":   # R held in registers (the tabulated cell's default) and in shared memory: the same bits
        assert "r_in=registers" in plan, plan
        got, plan, _ = _run(case, cuda_device, opts=opts + (("gemv_r", "smem"),))
        assert "r_in=smem" in plan and np.array_equal(got, _want(oracle, case)), plan
        rev, plan, _ = _run(case, cuda_device, reverse=True, opts=opts)
        import copy
        flipped = copy.copy(case)
        flipped.x_q = np.ascontiguousarray(case.x_q[::-1])
        assert "r_in=registers" in plan and np.array_equal(rev, _want(oracle, flipped)[::-1]), plan


def test_simt_gemm_and_wide_hidden(oracle, cuda_device):
    """The SIMT GEMM stays available (option); 512 < H <= 1024 runs on the cluster recurrence with
    the R slice split between tensor memory and shared memory; H > 1024 on the dp4a recurrence."""
    case = make_case(12, 5, 9, 72, 136, oracle, config_named("cfg2"))
    got, plan, _ = _run(case, cuda_device, opts=(("gemm", "simt"),))
    assert "gemm=simt_dp4a" in plan and np.array_equal(got, _want(oracle, case))
    for H in (640, 1024):
        wide = make_case(13, 3, 21, 40, H, oracle, config_named("default"))
        got, plan, _ = _run(wide, cuda_device)
        assert "rec=tcgen05_i8" in plan and "r_in=tmem+smem" in plan, plan
        assert np.array_equal(got, _want(oracle, wide)), plan
        got, plan, _ = _run(wide, cuda_device, opts=(("rec", "dp4a"),))
        assert "rec=dp4a" in plan and np.array_equal(got, _want(oracle, wide)), plan
        with pytest.raises(Exception):
            _run(wide, cuda_device, opts=(("rec", "mma"), ("exchange", "global")))
    huge = make_case(15, 2, 3, 24, 1100, oracle, config_named("default"))
    got, plan, _ = _run(huge, cuda_device)
    assert "rec=dp4a" in plan and np.array_equal(got, _want(oracle, huge)), plan
    with pytest.raises(Exception):
        _run(huge, cuda_device, opts=(("rec", "mma"),))


def test_two_tiles_per_cta_option(oracle, cuda_device):
    """128 < H <= 256 with both 128-unit tiles in one CTA (no exchange): kept as an option."""
    case = make_case(16, 5, 37, 24, 200, oracle, config_named("cfg2"))
    got, plan, _ = _run(case, cuda_device, opts=(("rec", "mma"), ("tiles_per_cta", "2")))
    assert "MT=2" in plan and "P=1" in plan and np.array_equal(got, _want(oracle, case)), plan
    got, plan, _ = _run(case, cuda_device, opts=(("rec", "mma"), ("unit_tile", "128")))
    assert "MT=1" in plan and "P=2" in plan and np.array_equal(got, _want(oracle, case)), plan


@pytest.mark.parametrize("shape", [(9, 40, 64, 512), (7, 33, 40, 300), (6, 70, 24, 128), (5, 100, 32, 640),
                                   (12, 5, 16, 256), (4, 200, 48, 384)])
@pytest.mark.parametrize("cfg", ["default", "cfg2", "gate_in16"])
def test_two_subgroups_per_cta(oracle, cuda_device, shape, cfg):
    """Two independent batch sub-groups per CTA (their MMAs and cells overlap): same bits as one,
    with ragged last sub-groups, one or several CTAs per cluster, R in tensor or shared memory,
    the fused, the generic and the segment-search cell, both directions."""
    T, B, I, H = shape
    case = make_case(17, T, B, I, H, oracle, config_named(cfg), with_h0=True)
    want = _want(oracle, case)
    for extra in ((), (("r_resident", "smem"),), (("cell", "generic"),)):
        if extra == (("r_resident", "smem"),) and H > 384:
            continue                      # the slice of R and four state tiles do not fit shared memory together
        got, plan, _ = _run(case, cuda_device, opts=(("rec", "mma"), ("exchange", "cluster"), ("subgroups", "2"), ("unit_tile", "128")) + extra)
        assert "NG=2" in plan and "exchange=cluster_dsmem" in plan, plan
        assert np.array_equal(got, want), plan
    got, plan, _ = _run(case, cuda_device, opts=(("rec", "mma"), ("exchange", "cluster"), ("subgroups", "1")))
    assert "NG=1" in plan and np.array_equal(got, want), plan
    rev, plan, _ = _run(case, cuda_device, reverse=True, opts=(("rec", "mma"), ("subgroups", "2"), ("unit_tile", "128")))
    import copy
    flipped = copy.copy(case)
    flipped.x_q = np.ascontiguousarray(case.x_q[::-1])
    assert np.array_equal(rev, _want(oracle, flipped)[::-1]), plan


@pytest.mark.parametrize("shape,sm_limit", [((9, 40, 64, 512), 0), ((7, 33, 40, 300), 0), ((6, 70, 24, 128), 0),
                                            ((12, 5, 16, 256), 0), ((4, 200, 48, 384), 0), ((5, 200, 48, 384), 24),
                                            ((5, 200, 32, 192), 9), ((3, 1, 8, 64), 0), ((30, 64, 32, 512), 0)])
@pytest.mark.parametrize("cfg", ["default", "cfg2", "sym8_tensor"])
def test_64_units_per_cta(oracle, cuda_device, shape, sm_limit, cfg):
    """The low-latency form of the cluster recurrence (64 hidden units per CTA, update and reset rows
    sharing one MMA tile, lane pairs splitting a unit's cells): same bits as the oracle for ragged
    H and B, clusters of 1 to 8 CTAs, 16, 32 and 48 rows per sub-group, both directions."""
    T, B, I, H = shape
    case = make_case(19, T, B, I, H, oracle, config_named(cfg), with_h0=True)
    want = _want(oracle, case)
    _, plan, _ = _run(case, cuda_device, opts=(("rec", "mma"), ("unit_tile", "128")))
    if "cell=fused_shiftfree" not in plan:
        pytest.skip("this configuration does not get the branch-free tabulated cell: " + plan)
    opts = (("rec", "mma"), ("unit_tile", "64")) + ((("sm_limit", str(sm_limit)),) if sm_limit else ())
    got, plan, _ = _run(case, cuda_device, opts=opts)
    assert "UT=64" in plan and "NG=2" in plan and "cell=fused_shiftfree" in plan, plan
    if sm_limit == 24:
        assert "NB=32" in plan, plan
    if sm_limit == 9:
        assert "NB=48" in plan, plan
    assert np.array_equal(got, want), plan
    got, plan, _ = _run(case, cuda_device, opts=opts, f32=True)
    assert "UT=64" in plan
    assert np.array_equal(got.view(np.uint32), oracle.dequantize(want, case.params.c, 1).view(np.uint32)), plan
    rev, plan, _ = _run(case, cuda_device, reverse=True, opts=opts)
    import copy
    flipped = copy.copy(case)
    flipped.x_q = np.ascontiguousarray(case.x_q[::-1])
    assert np.array_equal(rev, _want(oracle, flipped)[::-1]), plan


def test_sync_floor_probe_runs(oracle, cuda_device):
    """The synchronisation-floor probe (cluster recurrence without MMAs and cells) launches, ends
    and leaves the handle usable: the next forward is bit-exact again."""
    import torch
    case = make_case(18, 20, 40, 64, 512, oracle, config_named("cfg2"))
    dev = cuda_device
    with gru_ops.Handle(case.I, case.H, device=dev.index or 0) as hd:
        hd.set_params(case.params)
        hd.set_weights_i32(*[_t(a, dev) for a in case.wq])
        x = _t(case.x_q, dev)
        want = _want(oracle, case)
        assert np.array_equal(hd.forward_i32(x).cpu().numpy(), want)
        hd.set_option("probe_floor", 1)
        hd.forward_i32(x)
        assert "FLOOR PROBE" in hd.describe_plan()
        t_floor = hd.last_timing()
        hd.set_option("probe_floor", 0)
        assert np.array_equal(hd.forward_i32(x).cpu().numpy(), want)
        t_real = hd.last_timing()
        assert 0 < t_floor["recurrence_ms"] < t_real["recurrence_ms"] * 1.5
    torch.cuda.synchronize()


def test_bounded_wait_runs_out_and_the_handle_stays_usable(oracle, cuda_device):
    """The failure path of the per-step group barrier (dp4a recurrence, three CTAs per group): one CTA
    leaves out an arrival (a host-set test option), the others' bounded wait runs out after
    `spin_limit` polls, every CTA leaves, the call reports QGRU_ERR_TIMEOUT - and the next forward on
    the same handle is bit-exact again.  Nothing faults, traps or waits without a bound."""
    _cabi = importlib.import_module(PKG_NAME + "._cabi")
    case = make_case(21, 6, 9, 24, 300, oracle, config_named("default"))
    want = _want(oracle, case)
    dev = cuda_device
    with gru_ops.Handle(case.I, case.H, device=dev.index or 0) as hd:
        hd.set_option("rec", "dp4a")
        hd.set_params(case.params)
        hd.set_weights_i32(*[_t(a, dev) for a in case.wq])
        x = _t(case.x_q, dev)
        assert np.array_equal(hd.forward_i32(x).cpu().numpy(), want)
        assert "rec=dp4a" in hd.describe_plan() and "P=3" in hd.describe_plan()   # several CTAs per group
        hd.set_option("spin_limit", 2000)
        hd.set_option("test_withhold_arrive", 1)
        with pytest.raises(_cabi.QgruError) as err:
            hd.forward_i32(x)
        assert err.value.status == _cabi.QGRU_ERR_TIMEOUT
        hd.set_option("test_withhold_arrive", 0)
        hd.set_option("spin_limit", 1 << 24)
        assert np.array_equal(hd.forward_i32(x).cpu().numpy(), want)


@pytest.mark.parametrize("opts", [(), (("rec", "gemv"),), (("rec", "dp4a"),), (("rec", "mma"), ("exchange", "global")),
                                  (("rec", "mma"), ("unit_tile", "64")), (("rec", "mma"), ("cell", "generic"))])
@pytest.mark.parametrize("cfg", ["cfg2", "unsigned_x"])
def test_8bit_output_equals_the_float_output(oracle, cuda_device, opts, cfg):
    """qgru_forward_f32_q8: the quantized states in their 8-bit container; dequantized with the h
    operator's (scale, zero point) they are the fp32 output of qgru_forward_f32 bit for bit, and
    they are the oracle's integers."""
    import torch
    T, B, I, H = 7, 19, 24, 200
    case = make_case(23, T, B, I, H, oracle, config_named(cfg), with_h0=True)
    want = _want(oracle, case)
    dev = cuda_device
    with gru_ops.Handle(I, H, device=dev.index or 0) as hd:
        for k, v in opts:
            hd.set_option(k, v)
        hd.set_params(case.params)
        hd.set_weights_i32(*[_t(a, dev) for a in case.wq])
        for reverse in (False, True):
            try:
                q8 = hd.forward_f32_q8(_t(case.x, dev), _t(case.h0, dev), reverse=reverse)
            except Exception as e:
                if "unit_tile=64" in str(e):
                    pytest.skip("no branch-free tabulated cell for this configuration")
                raise
            f32 = hd.forward_f32(_t(case.x, dev), _t(case.h0, dev), reverse=reverse)
            scale, zp, uns = hd.h_quant_meta()
            assert q8.dtype == (torch.uint8 if uns else torch.int8)
            deq = (q8.to(torch.int32) - zp).to(torch.float32) * np.float32(scale)
            assert torch.equal(deq, f32), hd.describe_plan()
            if not reverse:
                assert np.array_equal(q8.cpu().numpy().astype(np.int32), want), hd.describe_plan()


def test_large_batch_many_groups(oracle, cuda_device):
    """More batch rows than one wave of groups holds at H = 512: consecutive launches."""
    case = make_case(14, 3, 700, 32, 384, oracle, config_named("default"), calib_batches=1)
    got, plan, _ = _run(case, cuda_device, opts=(("sm_limit", "12"),))
    assert "rec=tcgen05_i8" in plan and np.array_equal(got, _want(oracle, case)), plan


@pytest.mark.parametrize("name", CONFIGS)
def test_bitwidth_configs(oracle, cuda_device, name):
    for seed, (T, B, I, H) in enumerate([(7, 6, 24, 48), (4, 9, 40, 72)]):
        case = make_case(20 + seed, T, B, I, H, oracle, config_named(name), with_h0=(seed == 1))
        for opts in ((("rec", "mma"),), (("rec", "mma"), ("tie_rule", "always")), (("rec", "gemv"),),
                     (("rec", "mma"), ("cell", "fused")),
                     (("rec", "mma"), ("cell", "generic")), (("rec", "dp4a"),),
                     (("rec", "mma"), ("exchange", "global")),
                     (("rec", "mma"), ("exchange", "global"), ("cell", "generic"))):
            got, plan, _ = _run(case, cuda_device, opts=opts)
            assert "path=int8" in plan
            assert np.array_equal(got, _want(oracle, case)), (name, plan)


@pytest.mark.parametrize("name", ["wide16", "default", "cfg2"])
def test_generic_path(oracle, cuda_device, name):
    """16-bit activations cannot use 8-bit storage: the int32 / 64-bit-accumulate kernels run.
    They are also forced on 8-bit configs as a second, independent GPU implementation."""
    case = make_case(31, 5, 4, 12, 24, oracle, config_named(name), with_h0=True)
    got, plan, _ = _run(case, cuda_device, opts=(("rec", "generic"),))
    assert "path=generic" in plan
    assert np.array_equal(got, _want(oracle, case))
    if name == "wide16":
        got2, plan2, _ = _run(case, cuda_device)
        assert "path=generic" in plan2 and np.array_equal(got2, got)


@pytest.mark.parametrize("name", ["default", "cfg2", "wide16"])
def test_reverse_direction_equals_flip(oracle, cuda_device, name):
    """QGRU_FLAG_REVERSE == the reference's flip -> forward -> flip for the reverse direction."""
    case = make_case(41, 6, 5, 16, 40, oracle, config_named(name), with_h0=True)
    got, _, _ = _run(case, cuda_device, reverse=True)
    flipped = oracle.forward_i32(case.T, case.B, case.I, case.H, case.wq, case.x_q[::-1].copy(), case.h0_q,
                                 case.params.c, case.params.scale_list())
    assert np.array_equal(got[:case.T], flipped[1:][::-1])       # output
    assert np.array_equal(got[0], flipped[case.T])               # h_n
    assert np.array_equal(got[case.T], flipped[0])               # the initial state slot


@pytest.mark.parametrize("name", ["default", "cfg2", "pot2", "wide16"])
def test_float_interface_bitwise(oracle, cuda_device, name):
    """Float in / float out (quantGRUForwardInt): quantize, forward and dequantize must give the
    very same floats as the CPU path; includes h0 and values that saturate the x range."""
    case = make_case(51, 6, 7, 20, 40, oracle, config_named(name), with_h0=True, sigma=1.5)
    want = oracle.forward_f32(case.T, case.B, case.I, case.H, case.wq, case.x, case.h0, case.params.c,
                              case.params.scale_list())
    got, _, _ = _run(case, cuda_device, f32=True)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


def test_host_buffer_entry_points(oracle, cuda_device):
    case = make_case(61, 5, 6, 24, 48, oracle, config_named("cfg2"), with_h0=True)
    got, _, _ = _run(case, cuda_device, host=True)
    assert np.array_equal(got, _want(oracle, case))
    want_f = oracle.forward_f32(case.T, case.B, case.I, case.H, case.wq, case.x, case.h0, case.params.c,
                                case.params.scale_list())
    got_f, _, _ = _run(case, cuda_device, f32=True, host=True)
    assert np.array_equal(got_f.view(np.uint32), want_f.view(np.uint32))


def test_weight_quantize_on_device_matches(oracle, cuda_device):
    """set_weights_f32 (per-channel quantize on the GPU) == quantitativeWeightCPU."""
    for name in ("default", "cfg3", "cfg5", "pot2"):
        case = make_case(71, 3, 2, 40, 24, oracle, config_named(name))
        with gru_ops.Handle(case.I, case.H, device=0) as hd:
            hd.set_params(case.params)
            hd.set_weights_f32(*[_t(a, cuda_device) for a in (case.W, case.R, case.bw, case.br)])
            got = [t.cpu().numpy() for t in hd.get_weights_i32()]
            h = hd.forward_i32(_t(case.x_q, cuda_device)).cpu().numpy()
        for a, b in zip(got, case.wq):
            assert np.array_equal(a, b), name
        assert np.array_equal(h, _want(oracle, case))


def test_repeated_calls_and_handle_reuse(oracle, cuda_device):
    """Two calls in a row, then a different (T, B) and new params on the same handle."""
    import torch
    a = make_case(81, 5, 4, 16, 32, oracle, config_named("default"))
    b = make_case(82, 9, 7, 16, 32, oracle, config_named("cfg2"))
    with gru_ops.Handle(16, 32, device=0) as hd:
        for case in (a, a, b, a):
            hd.set_params(case.params)
            hd.set_weights_i32(*[_t(w, cuda_device) for w in case.wq])
            got = hd.forward_i32(_t(case.x_q, cuda_device)).cpu().numpy()
            assert np.array_equal(got, _want(oracle, case))
    torch.cuda.synchronize()


def test_argument_errors(oracle, cuda_device):
    import torch
    case = make_case(91, 3, 2, 8, 16, oracle, config_named("default"))
    with gru_ops.Handle(8, 16, device=0) as hd:
        with pytest.raises(Exception):   # forward before params / weights
            hd.forward_i32(_t(case.x_q, cuda_device))
        hd.set_params(case.params)
        with pytest.raises(ValueError):  # wrong weight shape
            hd.set_weights_i32(*[_t(w, cuda_device) for w in (case.wq[1], case.wq[1], case.wq[2], case.wq[3])])
        hd.set_weights_i32(*[_t(w, cuda_device) for w in case.wq])
        with pytest.raises(ValueError):  # wrong dtype
            hd.forward_i32(_t(case.x, cuda_device))
        bad = case.x_q.copy()
        bad[0, 0, 0] = 1000            # outside the 8-bit range x declares
        with pytest.raises(ValueError):
            hd.forward_i32(_t(bad, cuda_device))
        got = hd.forward_i32(_t(case.x_q, cuda_device)).cpu().numpy()   # handle still usable
        assert np.array_equal(got, _want(oracle, case))
    with pytest.raises(Exception):
        bad_cfg = config_named("default")
        bad_cfg.symmetric["R"] = False
        p = importlib.import_module(PKG_NAME + ".params").GRUQuantParams(16, bad_cfg)
        with gru_ops.Handle(8, 16, device=0) as hd:
            hd.set_params(p)


def test_forward_is_capturable_into_a_cuda_graph(oracle, cuda_device):
    """After one warm-up call (workspace allocation, tensor maps) a forward only enqueues work on
    the caller's stream, so it can be captured into a CUDA graph and replayed on new inputs -
    the way a streaming caller removes the per-call launch overhead."""
    import torch
    case = make_case(41, 6, 5, 24, 48, oracle, config_named("cfg2"))
    want = _want(oracle, case)
    with gru_ops.Handle(case.I, case.H, device=0) as hd:
        hd.set_params(case.params)
        hd.set_weights_i32(*[_t(a, cuda_device) for a in case.wq])
        x_static = torch.zeros((case.T, case.B, case.I), dtype=torch.int32, device=cuda_device)
        out_static = torch.zeros((case.T + 1, case.B, case.H), dtype=torch.int32, device=cuda_device)
        side = torch.cuda.Stream(device=cuda_device)
        side.wait_stream(torch.cuda.current_stream(cuda_device))
        with torch.cuda.stream(side):
            hd.forward_i32(x_static, None, out=out_static, sync=False)      # warm-up: allocations happen here
        torch.cuda.current_stream(cuda_device).wait_stream(side)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            hd.forward_i32(x_static, None, out=out_static, sync=False)
        for _ in range(2):
            x_static.copy_(_t(case.x_q, cuda_device))
            graph.replay()
            torch.cuda.synchronize()
            assert np.array_equal(out_static.cpu().numpy(), want)
            out_static.zero_()
            x_static.zero_()


@pytest.mark.parametrize("name", ["default", "cfg2", "wide16"])
def test_training_buffer(oracle, cuda_device, name):
    """qgru_forward_i32_train: h_q as in inference plus v_q equal to the oracle's training buffer;
    in reverse mode slot t of v_q belongs to x_q[t]."""
    case = make_case(51, 6, 5, 24, 40, oracle, config_named(name), with_h0=True)
    args = (case.T, case.B, case.I, case.H, case.wq, case.x_q, case.h0_q, case.params.c, case.params.scale_list())
    want_h, want_v = oracle.forward_i32_v(*args)
    with gru_ops.Handle(case.I, case.H, device=0) as hd:
        hd.set_params(case.params)
        hd.set_weights_i32(*[_t(a, cuda_device) for a in case.wq])
        h, v = hd.forward_i32_train(_t(case.x_q, cuda_device), _t(case.h0_q, cuda_device))
        assert np.array_equal(h.cpu().numpy(), want_h) and np.array_equal(v.cpu().numpy(), want_v)
        flipped = np.ascontiguousarray(case.x_q[::-1])
        h2, v2 = hd.forward_i32_train(_t(flipped, cuda_device), _t(case.h0_q, cuda_device), reverse=True)
        assert np.array_equal(v2.cpu().numpy()[::-1], want_v)
        assert np.array_equal(h2.cpu().numpy()[:case.T][::-1], want_h[1:])


@pytest.mark.parametrize("order", ["stream", "w_stationary"])
@pytest.mark.parametrize("shape,name", [((3, 50, 20, 40), "default"), ((5, 70, 300, 200), "cfg2"),
                                        ((2, 300, 1024, 520), "default"), ((4, 33, 640, 136), "cfg3"),
                                        ((40, 64, 896, 300), "cfg2"), ((3, 9, 513, 64), "default")])
def test_input_gemm_tile_orders(oracle, cuda_device, shape, name, order):
    """Both tile orders of the tcgen05 input GEMM (W and x slabs streaming per tile; the slice
    of W resident in tensor memory for the whole launch, the MMAs' A operand read from there), K
    from 128 to 1024 padded bytes, more and fewer token tiles than CTAs per channel tile: bit-exact."""
    T, B, I, H = shape
    case = make_case(seed=51, T=T, B=B, I=I, H=H, checker=oracle, config=config_named(name))
    got, plan, _ = _run(case, cuda_device, opts=(("gemm", "tcgen05"), ("gemm_order", order)))
    assert "gemm=tcgen05_i8" in plan
    assert np.array_equal(got, _want(oracle, case))


@pytest.mark.parametrize("shape,chunk", [((11, 20, 32, 128), 4), ((9, 40, 64, 512), 2), ((13, 33, 40, 300), 5),
                                         ((7, 70, 24, 640), 7), ((10, 5, 16, 256), 1), ((6, 300, 48, 384), 4)])
@pytest.mark.parametrize("cfg", ["default", "cfg2"])
def test_timestep_chunks(oracle, cuda_device, shape, chunk, cfg):
    """W*x+bw computed and consumed a chunk of timesteps at a time (the GEMM of the next chunk on a second
    stream beside the recurrence of this one, each recurrence launch starting from the state the one
    before left): same bits as the whole sequence in one launch pair, ragged last chunk, initial state
    given, both directions, 32-bit, float and 8-bit outputs, two forwards in a row on one handle."""
    import copy
    import torch
    T, B, I, H = shape
    case = make_case(23, T, B, I, H, oracle, config_named(cfg), with_h0=True)
    want = _want(oracle, case)
    opts = (("rec", "mma"), ("exchange", "cluster"), ("t_chunk", str(chunk)))
    got, plan, _ = _run(case, cuda_device, opts=opts)
    assert f"t_chunks={-(-T // chunk)}" in plan and np.array_equal(got, want), plan
    # few SMs: the batch groups of a chunk take several launches, each leaving its rows' state behind
    got, plan, _ = _run(case, cuda_device, opts=opts + (("sm_limit", str(-(-H // 128))),))
    assert f"t_chunks={-(-T // chunk)}" in plan and np.array_equal(got, want), plan
    whole, plan1, _ = _run(case, cuda_device, opts=(("rec", "mma"), ("exchange", "cluster"), ("t_chunk", "0")))
    assert "t_chunks=1" in plan1 and np.array_equal(whole, want), plan1
    flipped = copy.copy(case)
    flipped.x_q = np.ascontiguousarray(case.x_q[::-1])
    rev, plan, _ = _run(case, cuda_device, reverse=True, opts=opts)
    assert np.array_equal(rev, _want(oracle, flipped)[::-1]), plan
    with gru_ops.Handle(case.I, case.H, device=cuda_device.index or 0) as hd:
        for k, v in opts:
            hd.set_option(k, v)
        hd.set_params(case.params)
        hd.set_weights_i32(*[_t(a, cuda_device) for a in case.wq])
        x, h0 = _t(case.x_q, cuda_device), _t(case.h0_q, cuda_device)
        first = hd.forward_i32(x, h0).cpu().numpy()
        second = hd.forward_i32(x, h0).cpu().numpy()
        assert np.array_equal(first, want) and np.array_equal(second, want)
        xf, hf = _t(case.x, cuda_device), _t(case.h0, cuda_device)
        f = hd.forward_f32(xf, hf)
        q8 = hd.forward_f32_q8(xf, hf)
        scale, zp, _ = hd.h_quant_meta()
        assert torch.equal((q8.to(torch.int32) - zp).to(torch.float32) * np.float32(scale), f), hd.describe_plan()
