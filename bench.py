#!/usr/bin/env python
"""Benchmark of the integer quantized GRU forward (tokens/s, batch x seq).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload cfg2]

One "step" is one forward pass of the workload over one batch of seeded synthetic input.
The default workload is the reference's bidirectional headline configuration: input 256,
hidden 512, batch 256 per GPU-unit, 200 timesteps; 8-bit per-channel symmetric weights, 8-bit
asymmetric activations, 16-bit gate outputs, MinMax calibration on 16 seeded batches.

Sharding (weak scaling): the global batch is 256 x N.  N = 1 runs both directions on one GPU;
for even N each direction gets N/2 GPUs and every GPU runs one direction on 512 rows - the
same work per GPU at every N.  Ranks never exchange data on the timed path.

Rank 0 prints one JSON line.  `value` is measured with inputs resident in HBM, `e2e` through
the same calls with pinned host buffers (host->device copy of x and device->host copy of
every output inside the timed region).  `--impl reference` times the reference's own CPU
integer path (oracle/_ref, else the C port) on the box's host cores instead.
"""
import argparse
import importlib
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402

WORKLOADS = {
    # name: (I, H, B per unit, T, bidirectional, config name, x distribution, calib batches)
    "cfg1": (64, 128, 32, 50, False, "sym8_tensor", "normal", 8),
    "cfg2": (256, 512, 256, 200, True, "cfg2", "normal", 16),
    "cfg3": (128, 256, 4096, 100, False, "cfg3", "outliers", 16),
    "cfg4": (1024, 1024, 64, 1000, False, "sym8_tensor", "normal", 4),
    "cfg5": (80, 256, 1, 16000, False, "cfg5", "ar1", 4),
}
# calibration method of each workload configuration: (method, percentile)
CALIBRATION = {"cfg1": ("minmax", 0.0), "cfg2": ("minmax", 0.0), "cfg3": ("percentile", 99.9),
               "cfg4": ("sqnr", 0.0), "cfg5": ("minmax", 0.0)}


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="cfg2", choices=sorted(WORKLOADS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--calib-batches", type=int, default=0,
                    help="override the number of calibration batches (profiling runs only)")
    ap.add_argument("--rows", type=int, default=0,
                    help="override the batch rows per GPU-unit (small profiling cases only)")
    return ap.parse_args()


class ClockSampler:
    """nvidia-smi clocks / throttle reasons of one GPU, sampled every 200 ms while running."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q,
                 "--format=csv,noheader,nounits", "-lms", "200"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *exc):
        if self.proc:
            time.sleep(0.25)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self):
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
            except (ValueError, IndexError):
                continue
            for n, v in zip(names, r[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                "samples": len(sm)}


def build_problem(wl, seed_base):
    """Seeded weights for each direction, in the reference's haste layout."""
    from tests.cases import gen_weights
    I, H = wl[0], wl[1]
    dirs = 2 if wl[4] else 1
    return [gen_weights(np.random.default_rng(seed_base + d), I, H) for d in range(dirs)]


def bytes_per_token(I, H, ih_bytes):
    # fp32 x read + W*x+bw written once and read once + fp32 h written
    return 4 * I + 2 * 3 * H * ih_bytes + 4 * H


# ----------------------------------------------------------------------------- our arm
def run_ours(args):
    import torch
    import torch.distributed as dist
    from __graft_entry__ import PKG_NAME, load_package
    load_package()
    gru_ops = importlib.import_module(PKG_NAME + ".gru_ops")
    params_mod = importlib.import_module(PKG_NAME + ".params")
    sharding = importlib.import_module(PKG_NAME + ".sharding")
    from tests.cases import config_named, gen_x

    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    if world != args.gpus and world > 1:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    I, H, B_unit, T, bidir, cfg_name, xdist, n_calib = WORKLOADS[args.workload]
    if args.calib_batches > 0:
        n_calib = args.calib_batches
    if args.rows > 0:
        B_unit = args.rows
    B_global = B_unit * world
    shards = sharding.plan_shards(world, B_global, bidir)
    me = shards[rank]
    cfg = config_named(cfg_name)
    weights = build_problem(WORKLOADS[args.workload], 1000 + int(args.workload[3:]) * 10)
    sms = torch.cuda.get_device_properties(dev).multi_processor_count

    # --- calibration over n_calib seeded batches of the unit shape, per direction: MinMax ranges
    # or 2048-bin histograms (Percentile / SQNR), as the workload's configuration says
    method, pct = CALIBRATION[args.workload]
    handles = []
    for d in me.directions:
        hd = gru_ops.Handle(I, H, device=local)
        if len(me.directions) > 1:
            hd.set_option("sm_limit", sms // 2)
        for kv in filter(None, os.environ.get("QGRU_OPTS", "").split(",")):   # tuning experiments
            hd.set_option(*kv.split("=", 1))
        W, R, bw, br = [torch.from_numpy(a).to(dev) for a in weights[d]]
        ranges = params_mod.Ranges(H)
        hist = params_mod.Histograms(H, device=local) if method != "minmax" else None
        for k in range(n_calib):
            xc = torch.from_numpy(gen_x(np.random.default_rng(100 * int(args.workload[3:]) + k), T,
                                        B_unit, I, xdist)).to(dev)
            xc = xc.flip(0).contiguous() if d == 1 else xc
            if hist is None:
                hd.calibrate_minmax(W, R, bw, br, xc, ranges)
            else:
                hd.calibrate_hist(W, R, bw, br, xc, hist, cfg.granularity_list())
        if hist is None:
            qp = params_mod.GRUQuantParams.from_ranges(ranges, cfg)
        else:
            qp = params_mod.GRUQuantParams.from_histograms(hist, cfg, method == "percentile", pct)
            hist.close()
        hd.set_params(qp)
        hd.set_weights_f32(W, R, bw, br)
        handles.append((hd, d == 1, torch.cuda.Stream(device=dev)))

    # --- this rank's input shard, resident on the device and pinned on the host
    rows = me.rows
    x_host = torch.from_numpy(gen_x(np.random.default_rng(int(args.workload[3:]) + 7919 * rank), T, rows, I,
                                    xdist)).pin_memory()
    x_dev = x_host.to(dev)
    outs = [torch.empty((T + 1, rows, H), dtype=torch.float32, device=dev) for _ in handles]
    outs_host = [torch.empty((T + 1, rows, H), dtype=torch.float32).pin_memory() for _ in handles]

    def step(x, into=None):
        cur = torch.cuda.current_stream(dev)
        for (hd, rev, st), o in zip(handles, into or outs):
            st.wait_stream(cur)
            with torch.cuda.stream(st):
                hd.forward_f32(x, None, reverse=rev, out=o, sync=False)
        for hd, rev, st in handles:
            cur.wait_stream(st)

    # End to end: every step copies its input from pinned host memory and its outputs back to
    # pinned host memory.  The three phases run on three streams over two sets of device buffers,
    # so the copy-in of step i+1 and the copy-out of step i-1 overlap the compute of step i (PCIe
    # is full duplex); each step's copies are still inside the timed region.
    # Two copy-out streams: one device-to-host copy alone reaches about 41 GB/s on this box, two
    # concurrent ones about 57 GB/s.
    copy_in = torch.cuda.Stream(device=dev)
    copy_outs = [torch.cuda.Stream(device=dev) for _ in range(2)]
    x_stage = [torch.empty_like(x_dev) for _ in range(2)]
    outs2 = [outs, [torch.empty_like(o) for o in outs]]
    ev_in = [torch.cuda.Event() for _ in range(2)]
    ev_done = [torch.cuda.Event() for _ in range(2)]
    ev_out = [[torch.cuda.Event() for _ in range(2)] for _ in range(2)]
    e2e_state = {"i": 0}

    def out_pieces(k):
        """(device piece, host piece) pairs of output set k, dealt over the two copy-out streams."""
        pairs = []
        for o, oh in zip(outs2[k], outs_host):
            if len(outs2[k]) == 1:
                half = o.shape[0] // 2
                pairs += [(o[:half], oh[:half]), (o[half:], oh[half:])]
            else:
                pairs.append((o, oh))
        return pairs

    def step_e2e():
        i = e2e_state["i"]
        k = i & 1
        e2e_state["i"] = i + 1
        cur = torch.cuda.current_stream(dev)
        copy_in.wait_stream(cur)                       # not before the timed region starts
        if i >= 2:
            copy_in.wait_event(ev_done[k])             # step i-2 has consumed this input buffer
        with torch.cuda.stream(copy_in):
            x_stage[k].copy_(x_host, non_blocking=True)
            ev_in[k].record(copy_in)
        cur.wait_event(ev_in[k])
        if i >= 2:
            for e in ev_out[k]:
                cur.wait_event(e)                      # step i-2's outputs have left these buffers
        step(x_stage[k], outs2[k])
        ev_done[k].record(cur)
        for n, (o, oh) in enumerate(out_pieces(k)):
            st = copy_outs[n % 2]
            st.wait_event(ev_done[k])
            with torch.cuda.stream(st):
                oh.copy_(o, non_blocking=True)
        for n, st in enumerate(copy_outs):
            ev_out[k][n].record(st)

    def e2e_drain():
        for st in copy_outs:
            torch.cuda.current_stream(dev).wait_stream(st)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    def timed(fn, steps, warmup, drain=None):
        for _ in range(warmup):
            fn()
        if drain:
            drain()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        if drain:
            drain()                                    # the last steps' copies end inside the region
        e1.record()
        barrier()
        ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    launches0 = sum(hd.launch_count() for hd, _, _ in handles)
    with ClockSampler(local) as clk:
        ms_total = timed(lambda: step(x_dev), args.steps, args.warmup)
    launches = sum(hd.launch_count() for hd, _, _ in handles) - launches0
    for hd, _, _ in handles:
        hd.synchronize()
    # per-kernel time of the timed steps, from events the library records on its launch stream
    nwin = min(args.steps, 64)
    wins = [hd.timing_window(nwin) for hd, _, _ in handles]
    ms_e2e = timed(step_e2e, max(3, args.steps // 2), 2, drain=e2e_drain)
    e2e_steps = max(3, args.steps // 2)
    for hd, _, _ in handles:
        hd.synchronize()

    tokens_step = B_global * T
    value = tokens_step * args.steps / (ms_total * 1e-3)
    e2e = tokens_step * e2e_steps / (ms_e2e * 1e-3)
    plan = handles[0][0].describe_plan()
    ih_bytes = 2 if "ih_bytes=2" in plan else 1

    result = None
    if rank == 0:
        peaks = {}
        try:
            peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        except (OSError, ValueError):
            pass
        hbm = peaks.get("hbm_gbs", 6650.0)
        peak_kind = "measured" if "hbm_gbs" in peaks else "fallback"
        # dominant kernel: the persistent recurrence kernel of one direction.  Algorithmic bytes
        # per launch = T * rows * (3H*b_ih read + 4H written as fp32 output); the 8-bit state adds
        # H per token only where it is exchanged through global memory (not in the cluster kernel)
        w = wins[0]
        rec_ms = w["recurrence_ms"] / max(1, w["calls"])
        gemm_ms = w["input_gemm_ms"] / max(1, w["calls"])
        cluster = "exchange=cluster_dsmem" in plan
        kernel = ("k_recurrence_cluster" if cluster else "k_recurrence_mma") if "rec=tcgen05" in plan \
            else ("k_recurrence_dp4a" if "path=int8" in plan else "k_linear_generic+k_gates_generic")
        rec_bytes = T * rows * (3 * H * ih_bytes + H * (4 if cluster else 5))
        # DRAM traffic of one launch from the ncu capture of this kernel on this workload
        # (dram__bytes_read.sum + dram__bytes_write.sum = 234.8 MB for 51200 tokens of cfg2),
        # scaled by the tokens of a launch; other kernels / workloads were not captured
        traffic = None
        if args.workload == "cfg2" and kernel == "k_recurrence_cluster" and ih_bytes == 2:
            traffic = 234.8e6 * (T * rows) / 51200.0
        achieved = rec_bytes / (rec_ms * 1e-3) / 1e9 if rec_ms > 0 else 0.0
        result = {
            "metric": "int-quant GRU fwd tokens/s (batch x seq)", "value": value, "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_total / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "int8 (int32 accumulate, 64-bit requantize)",
            "data": "synthetic",
            "config": {"workload": f"{args.workload}: {'bi' if bidir else 'uni'}directional GRU I={I} H={H} "
                                   f"global_batch={B_global} T={T}, bit widths '{cfg_name}', "
                                   f"{method}{' %g' % pct if method == 'percentile' else ''} calibration x{n_calib}",
                       "per_gpu": f"directions={list(me.directions)} rows={rows}",
                       "l2": "inputs larger than L2: x, W*x+bw and the fp32 outputs of one step "
                             f"total {(rows * T * bytes_per_token(I, H, ih_bytes) * len(handles)) / 1e6:.0f} MB > 126 MB",
                       "plan": plan},
            "roofline": {"bound": "hbm", "kernel": kernel + " (one direction)", "achieved": achieved,
                         "peak": hbm, "unit": "GB/s", "frac": achieved / hbm, "peak_kind": peak_kind,
                         "traffic": traffic, "us_per_timestep": rec_ms * 1e3 / T,
                         "input_gemm_ms": gemm_ms, "recurrence_ms": rec_ms,
                         "whole_forward_frac": (tokens_step / world * bytes_per_token(I, H, ih_bytes) * len(handles) /
                                                ((ms_total / args.steps) * 1e-3) / 1e9) / hbm},
            "e2e": {"value": e2e, "unit": "tokens/s",
                    "h2d_bytes_per_step": int(x_host.numel() * 4),
                    "d2h_bytes_per_step": int(sum(o.numel() * 4 for o in outs_host))},
            "gpu_launches": int(launches),
            "clocks": clk.summary(),
        }
        if world == 1 and not args.no_cpu_baseline:
            result["cpu_baseline"] = cpu_baseline(args.workload, budget_s=15.0)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    for hd, _, _ in handles:
        hd.close()
    if result is not None:
        print(json.dumps(result))


# ------------------------------------------------------------------ CPU baseline / reference arm
def cpu_problem(workload):
    """Quantized operands of one small batch for the CPU integer path (both directions)."""
    from oracle.binding import Oracle, reference_or_none
    from tests.cases import config_named, make_case
    I, H, B_unit, T, bidir, cfg_name, xdist, _ = WORKLOADS[workload]
    ref = reference_or_none()
    chk = ref or Oracle()
    cores = os.cpu_count() or 1
    rows = max(1, min(B_unit, 2 * cores))
    cases = []
    for d in range(2 if bidir else 1):
        # calibration on a short, narrow batch: it fixes the values, not the running time
        cal = make_case(1000 + d, min(T, 20), 4, I, H, chk, config_named(cfg_name), dist=xdist,
                        calib_batches=1, oracle=Oracle())
        x = np.random.default_rng(77 + d).standard_normal((T, rows, I)).astype(np.float32)
        x_q = chk.quantize(x, cal.params.c, 0)
        cases.append((cal, x_q))
    return chk, cases, rows, T, I, H, cores


def cpu_step(chk, cases, rows, T, I, H, cores):
    for cal, x_q in cases:
        chk.forward_i32(T, rows, I, H, cal.wq, x_q, None, cal.params.c, cal.params.scale_list(), threads=cores)


def cpu_baseline(workload, budget_s=15.0):
    chk, cases, rows, T, I, H, cores = cpu_problem(workload)
    t0 = time.perf_counter()
    cpu_step(chk, cases, rows, T, I, H, cores)
    one = time.perf_counter() - t0
    reps = max(1, min(10, int(budget_s / max(one, 1e-3)) - 1))
    t0 = time.perf_counter()
    for _ in range(reps):
        cpu_step(chk, cases, rows, T, I, H, cores)
    dt = (time.perf_counter() - t0) / reps
    return {"value": rows * T / dt, "unit": "tokens/s", "cores": min(cores, rows), "kind": chk.kind,
            "sample": f"{rows} of the batch rows x T={T}, {len(cases)} direction(s), batch rows split over "
                      f"{min(cores, rows)} host threads, {reps} repetitions"}


def run_reference(args):
    rank = int(os.environ.get("RANK", 0))
    if rank != 0:
        return
    chk, cases, rows, T, I, H, cores = cpu_problem(args.workload)
    for _ in range(args.warmup):
        cpu_step(chk, cases, rows, T, I, H, cores)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu_step(chk, cases, rows, T, I, H, cores)
    dt = time.perf_counter() - t0
    value = rows * T * args.steps / dt
    wl = WORKLOADS[args.workload]
    print(json.dumps({
        "impl": "reference", "metric": "int-quant GRU fwd tokens/s (batch x seq)", "value": value,
        "unit": "tokens/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "int32 containers, int64 accumulate (CPU)", "data": "synthetic",
        "config": {"workload": f"{args.workload}: {'bi' if wl[4] else 'uni'}directional GRU I={I} H={H} T={T}, "
                               f"bit widths '{wl[5]}'; each step = {rows} batch rows (bounded sample)"},
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": min(cores, rows), "kind": chk.kind,
                         "sample": f"{rows} batch rows x T={T}, {len(cases)} direction(s) per step"},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


if __name__ == "__main__":
    a = parse()
    if a.impl == "reference":
        run_reference(a)
    else:
        run_ours(a)
