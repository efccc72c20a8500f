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
every output inside the timed region).  After the timed regions every rank compares rows of
its GPU result, every timestep, bit for bit with the reference's CPU integer path (`check`);
with N > 1 the per-rank outputs are all-gathered once over NCCL and compared with the local
shards (`gather`); at every N the throughput configuration (batch 4096 split evenly over the N
GPUs, fixed total work) is timed as the `strong` block, and the recurrence is run once more
without its MMAs and cells to give the synchronisation floor of a timestep.  `--impl reference` times the
reference's own CPU integer path (oracle/_ref, else the C port) on the box's host cores.
"""
import argparse
import importlib
import json
import os
import re
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402

from __graft_entry__ import PKG_NAME, load_package  # noqa: E402

load_package()
workloads = importlib.import_module(PKG_NAME + ".workloads")
WORKLOADS, CALIBRATION = workloads.WORKLOADS, workloads.CALIBRATION

METRIC = "int-quant GRU fwd tokens/s (batch x seq)"
STRONG_WORKLOAD = "cfg3"      # batch 4096 sharded evenly over the GPUs: fixed total work


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="cfg2", choices=sorted(WORKLOADS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-check", action="store_true", help="skip the bit-exact comparison with the CPU path")
    ap.add_argument("--check-rows", type=int, default=0,
                    help="batch rows per direction compared with the CPU path (0: as many as ~10 s of CPU buy)")
    ap.add_argument("--no-strong", action="store_true", help="skip the fixed-total-work (cfg3, batch 4096 over N GPUs) block")
    ap.add_argument("--calib-batches", type=int, default=0,
                    help="override the number of calibration batches (profiling runs only)")
    ap.add_argument("--rows", type=int, default=0,
                    help="override the batch rows per GPU-unit (small profiling cases only)")
    ap.add_argument("--option", action="append", default=[], metavar="NAME=VALUE",
                    help="library option set on every handle (see qgru_set_option)")
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


def bytes_per_token(I, H, ih_bytes):
    # fp32 x read + W*x+bw written once and read once + fp32 h written
    return 4 * I + 2 * 3 * H * ih_bytes + 4 * H


def profiled_traffic_per_token(kernel, workload):
    """DRAM bytes per token of `kernel` on `workload` from the committed ncu summary
    profiles/<kernel>_<workload>.md (its line `dram_bytes_per_token: <number>`); None where no
    capture of that pair exists."""
    try:
        text = open(os.path.join(ROOT, "profiles", f"{kernel}_{workload}.md")).read()
    except OSError:
        return None
    m = re.search(r"dram_bytes_per_token:\s*([0-9.]+)", text)
    return float(m.group(1)) if m else None


# ----------------------------------------------------------------------------- our arm
class Job:
    """One rank's share of a workload: calibrated handles, resident input, output buffers."""

    def __init__(self, args, name, torch, dev, local, rank, world, global_batch, n_calib=0, options=()):
        gru_ops = importlib.import_module(PKG_NAME + ".gru_ops")
        sharding = importlib.import_module(PKG_NAME + ".sharding")
        self.torch, self.dev, self.name, self.rank, self.world = torch, dev, name, rank, world
        I, H, _, T, bidir = WORKLOADS[name][:5]
        self.I, self.H, self.T, self.bidir = I, H, T, bidir
        self.global_batch = global_batch
        self.shards = sharding.plan_shards(world, global_batch, bidir)
        self.me = self.shards[rank]
        self.rows = self.me.rows
        self.n_calib = n_calib or WORKLOADS[name][7]
        sms = torch.cuda.get_device_properties(dev).multi_processor_count
        weights = workloads.workload_weights(name)
        self.handles = []   # (handle, reverse, stream, quant params)
        for d in self.me.directions:
            hd = gru_ops.Handle(I, H, device=local)
            if len(self.me.directions) > 1:
                hd.set_option("sm_limit", sms // 2)
            for kv in options:
                hd.set_option(*kv.split("=", 1))
            wdev = [torch.from_numpy(a).to(dev) for a in weights[d]]
            qp = workloads.calibrate_workload(hd, name, d, wdev, lambda a: torch.from_numpy(a).to(dev),
                                              n_calib=self.n_calib)
            hd.set_params(qp)
            hd.set_weights_f32(*wdev)
            self.handles.append((hd, d == 1, torch.cuda.Stream(device=dev), qp))
        self.x_np = workloads.workload_input(name, rank, self.rows)
        self.x_host = torch.from_numpy(self.x_np).pin_memory()
        self.x_dev = self.x_host.to(dev)
        self.outs = [torch.empty((T + 1, self.rows, H), dtype=torch.float32, device=dev) for _ in self.handles]

    def step(self, x=None, into=None, narrow=False):
        torch, dev = self.torch, self.dev
        cur = torch.cuda.current_stream(dev)
        x = self.x_dev if x is None else x
        for (hd, rev, st, _), o in zip(self.handles, into or self.outs):
            st.wait_stream(cur)
            with torch.cuda.stream(st):
                if narrow:
                    hd.forward_f32_q8(x, None, reverse=rev, out=o, sync=False)
                else:
                    hd.forward_f32(x, None, reverse=rev, out=o, sync=False)
        for _, _, st, _ in self.handles:
            cur.wait_stream(st)

    def launch_count(self):
        return sum(h[0].launch_count() for h in self.handles)

    def synchronize(self):
        for h in self.handles:
            h[0].synchronize()

    def plan(self):
        return self.handles[0][0].describe_plan()

    def tokens_per_step(self):
        return self.global_batch * self.T

    def close(self):
        for h in self.handles:
            h[0].close()

    # -- bit-exact comparison of this rank's result with the CPU integer path
    def check(self, want_rows, threads):
        from oracle import check as ocheck
        chk = ocheck.checker()
        self.step()
        self.synchronize()
        self.torch.cuda.synchronize(self.dev)
        rows = ocheck.spread_rows(self.rows, want_rows)
        res = {"rows": 0, "steps": self.T, "mismatches": 0, "kind": chk.kind, "directions": len(self.handles)}
        for (hd, rev, _, qp), o in zip(self.handles, self.outs):
            r = ocheck.check_forward_rows(chk, hd, qp, self.x_np, o, rows, reverse=rev, threads=threads)
            res["rows"] += r["rows"]
            res["mismatches"] += r["mismatches"]
        return res

    def auto_check_rows(self, threads, budget_s=10.0):
        # the reference's CPU path runs about 0.5 G multiply-adds per second and thread
        macs_row = self.T * 3 * self.H * (self.I + self.H) * len(self.handles)
        n = int(budget_s * 0.5e9 * max(1, threads) / max(1, macs_row))
        return max(min(self.rows, 48), min(self.rows, n))

    # -- NCCL all-gather of every rank's output, compared with the local shard
    def gather_check(self):
        import torch.distributed as dist
        torch = self.torch
        sharding = importlib.import_module(PKG_NAME + ".sharding")
        self.step()
        self.synchronize()
        outs = []
        for (_, rev, _, _), o in zip(self.handles, self.outs):
            outs.append(o[:-1] if rev else o[1:])   # per-timestep outputs (the reverse result keeps its start in slot T)
        hns = [o[0:1] if rev else o[-1:] for (_, rev, _, _), o in zip(self.handles, self.outs)]
        local_out = torch.cat(outs, dim=-1) if len(outs) > 1 else outs[0].contiguous()
        local_hn = torch.cat(hns, dim=0) if len(hns) > 1 else hns[0].contiguous()
        full, full_hn = sharding.gather_outputs(local_out, local_hn, self.shards, self.rank, self.H,
                                                self.global_batch, self.T, self.bidir)
        ok = True
        for k, d in enumerate(self.me.directions):
            ok = ok and torch.equal(full[:, self.me.b0:self.me.b1, d * self.H:(d + 1) * self.H],
                                    local_out[:, :, k * self.H:(k + 1) * self.H])
            ok = ok and torch.equal(full_hn[d, self.me.b0:self.me.b1], local_hn[k])
        flag = torch.tensor([0 if ok else 1], device=self.dev)
        dist.all_reduce(flag)
        return int(flag.item()) == 0, list(full.shape)


def run_ours(args):
    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    if world != args.gpus and world > 1:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    I, H, B_unit, T, bidir, cfg_name, xdist, _ = WORKLOADS[args.workload]
    if args.rows > 0:
        B_unit = args.rows
    job = Job(args, args.workload, torch, dev, local, rank, world, B_unit * world, args.calib_batches, args.option)
    rows = job.rows
    method, pct = CALIBRATION[args.workload]

    # End to end: every step copies its input from pinned host memory and its outputs back to
    # pinned host memory.  The three phases run on three streams over two sets of device buffers,
    # so the copy-in of step i+1 and the copy-out of step i-1 overlap the compute of step i (PCIe
    # is full duplex); each step's copies are still inside the timed region.
    # Two copy-out streams: one device-to-host copy alone reaches about 41 GB/s on this box, two
    # concurrent ones about 57 GB/s.
    outs_host = [torch.empty((T + 1, rows, H), dtype=torch.float32).pin_memory() for _ in job.handles]
    copy_in = torch.cuda.Stream(device=dev)
    copy_outs = [torch.cuda.Stream(device=dev) for _ in range(2)]
    x_stage = [torch.empty_like(job.x_dev) for _ in range(2)]
    outs2 = [job.outs, [torch.empty_like(o) for o in job.outs]]
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
            x_stage[k].copy_(job.x_host, non_blocking=True)
            ev_in[k].record(copy_in)
        cur.wait_event(ev_in[k])
        if i >= 2:
            for e in ev_out[k]:
                cur.wait_event(e)                      # step i-2's outputs have left these buffers
        job.step(x_stage[k], outs2[k])
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

    launches0 = job.launch_count()
    with ClockSampler(local) as clk:
        ms_total = timed(job.step, args.steps, args.warmup)
    launches = job.launch_count() - launches0
    job.synchronize()
    # per-kernel time of the timed steps, from events the library records on its launch stream
    nwin = min(args.steps, 64)
    wins = [h[0].timing_window(nwin) for h in job.handles]
    e2e_steps = max(3, args.steps // 2)
    ms_e2e = timed(step_e2e, e2e_steps, 2, drain=e2e_drain)
    job.synchronize()
    # The same end-to-end loop with the outputs left in their 8-bit containers (qgru_forward_f32_q8): a
    # quarter of the device-to-host bytes.  Reported beside `e2e`, which stays the fp32 interface.
    e2e_narrow = None
    try:
        q8_dtype = torch.uint8 if job.handles[0][0].h_quant_meta()[2] else torch.int8
        n_outs = [[torch.empty((T + 1, rows, H), dtype=q8_dtype, device=dev) for _ in job.handles] for _ in range(2)]
        n_host = [torch.empty((T + 1, rows, H), dtype=q8_dtype).pin_memory() for _ in job.handles]
        n_state = {"i": 0}
        nev_in = [torch.cuda.Event() for _ in range(2)]
        nev_done = [torch.cuda.Event() for _ in range(2)]
        nev_out = [torch.cuda.Event() for _ in range(2)]

        def step_narrow():
            i = n_state["i"]
            k = i & 1
            n_state["i"] = i + 1
            cur = torch.cuda.current_stream(dev)
            copy_in.wait_stream(cur)
            if i >= 2:
                copy_in.wait_event(nev_done[k])
            with torch.cuda.stream(copy_in):
                x_stage[k].copy_(job.x_host, non_blocking=True)
                nev_in[k].record(copy_in)
            cur.wait_event(nev_in[k])
            if i >= 2:
                cur.wait_event(nev_out[k])
            job.step(x_stage[k], n_outs[k], narrow=True)
            nev_done[k].record(cur)
            st = copy_outs[0]
            st.wait_event(nev_done[k])
            with torch.cuda.stream(st):
                for o, oh in zip(n_outs[k], n_host):
                    oh.copy_(o, non_blocking=True)
            nev_out[k].record(st)

        ms_narrow = timed(step_narrow, e2e_steps, 2, drain=e2e_drain)
        job.synchronize()
        e2e_narrow = {"value": job.tokens_per_step() * e2e_steps / (ms_narrow * 1e-3), "unit": "tokens/s",
                      "h2d_bytes_per_step": int(T * rows * I * 4),
                      "d2h_bytes_per_step": int((T + 1) * rows * H * len(job.handles)),
                      "output": "8-bit quantized h (qgru_forward_f32_q8); dequantize with the h operator's scale / zero point",
                      "d2h_gb_per_s_this_rank": (T + 1) * rows * H * len(job.handles) * e2e_steps / (ms_narrow * 1e-3) / 1e9,
                      "h2d_gb_per_s_this_rank": T * rows * I * 4 * e2e_steps / (ms_narrow * 1e-3) / 1e9}
        del n_outs, n_host
    except Exception as ex:   # configurations outside the 8-bit storage plan have no narrow output
        e2e_narrow = {"unavailable": str(ex)[:120]}
    job.step()                # the plan text and timing ring describe the fp32 forward again
    job.synchronize()
    del x_stage, outs2, outs_host

    tokens_step = job.tokens_per_step()
    value = tokens_step * args.steps / (ms_total * 1e-3)
    e2e = tokens_step * e2e_steps / (ms_e2e * 1e-3)
    plan = job.plan()
    ih_bytes = 2 if "ih_bytes=2" in plan else (4 if "ih_bytes=4" in plan else 1)

    # ---- outside the timed regions: synchronisation floor, bit-exact check of this rank's rows, gather
    # check, strong block
    floor_us = None
    try:   # the same recurrence launch without its MMAs and cells: exchange, barriers and output stores only
        for h in job.handles:
            h[0].set_option("probe_floor", 1)
        for _ in range(3):
            job.step()
        job.synchronize()
        if "FLOOR PROBE" in job.plan():
            fw = job.handles[0][0].timing_window(2)
            floor_us = fw["recurrence_ms"] / max(1, fw["calls"]) * 1e3 / T
    except Exception:   # forms of the recurrence without the probe
        floor_us = None
    finally:
        for h in job.handles:
            h[0].set_option("probe_floor", 0)
        try:
            job.step()      # leaves the plan text and the timing ring describing the real kernel again
            job.synchronize()
        except Exception:
            pass
    cores = os.cpu_count() or 1
    threads = max(1, cores // world)
    check = None
    if not args.no_check:
        res = job.check(args.check_rows or job.auto_check_rows(threads), threads)
        tot = torch.tensor([res["rows"], res["mismatches"]], device=dev, dtype=torch.int64)
        if world > 1:
            dist.all_reduce(tot)
        check = {"status": "ok" if int(tot[1]) == 0 else "MISMATCH", "bit_exact": int(tot[1]) == 0,
                 "checked_rows": int(tot[0]), "timesteps": T, "ranks": world, "against": res["kind"],
                 "mismatching_values": int(tot[1])}
    gather = None
    if world > 1:
        ok, shape = job.gather_check()
        gather = {"status": "ok" if ok else "MISMATCH", "backend": "nccl", "gathered_shape": shape}
    job_rows, job_handles = job.rows, len(job.handles)
    job.close()
    del job
    torch.cuda.empty_cache()

    strong = None
    if not args.no_strong and args.workload == "cfg2":
        sI, sH, sB, sT = WORKLOADS[STRONG_WORKLOAD][:4]
        sj = Job(args, STRONG_WORKLOAD, torch, dev, local, rank, world, sB, 0, args.option)
        ms_s = timed(sj.step, args.steps, args.warmup)
        sj.synchronize()
        sw = sj.handles[0][0].timing_window(min(args.steps, 64))
        strong = {"workload": f"{STRONG_WORKLOAD}: unidirectional GRU I={sI} H={sH} global_batch={sB} T={sT}, "
                              f"batch split evenly over {world} GPUs ({sj.rows} rows each)",
                  "scaling": "strong", "value": sB * sT * args.steps / (ms_s * 1e-3), "unit": "tokens/s",
                  "ms_per_step": ms_s / args.steps, "n_gpus": world,
                  "us_per_timestep": sw["recurrence_ms"] / max(1, sw["calls"]) * 1e3 / sT, "plan": sj.plan()}
        if not args.no_check:
            res = sj.check(args.check_rows or sj.auto_check_rows(threads, 5.0), threads)
            tot = torch.tensor([res["rows"], res["mismatches"]], device=dev, dtype=torch.int64)
            if world > 1:
                dist.all_reduce(tot)
            strong["check"] = {"status": "ok" if int(tot[1]) == 0 else "MISMATCH", "checked_rows": int(tot[0]),
                               "timesteps": sT, "against": res["kind"]}
        sj.close()

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
            else ("k_recurrence_gemv" if "rec=gemv" in plan else
                  ("k_recurrence_dp4a" if "path=int8" in plan else "k_linear_generic+k_gates_generic"))
        rec_bytes = T * job_rows * (3 * H * ih_bytes + H * (4 if cluster or "rec=gemv" in plan else 5))
        per_token = profiled_traffic_per_token(kernel, args.workload)
        traffic = per_token * T * job_rows if per_token else None
        achieved = rec_bytes / (rec_ms * 1e-3) / 1e9 if rec_ms > 0 else 0.0
        result = {
            "metric": METRIC, "value": value, "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_total / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "int8 (int32 accumulate, 64-bit requantize)",
            "data": "synthetic",
            "config": {"workload": f"{args.workload}: {'bi' if bidir else 'uni'}directional GRU I={I} H={H} "
                                   f"global_batch={B_unit * world} T={T}, bit widths '{cfg_name}', "
                                   f"{method}{' %g' % pct if method == 'percentile' else ''} calibration "
                                   f"x{args.calib_batches or WORKLOADS[args.workload][7]}",
                       "per_gpu": f"directions={list(range(2)) if job_handles > 1 else 'one'} rows={job_rows}",
                       "l2": "inputs larger than L2: x, W*x+bw and the fp32 outputs of one step "
                             f"total {(job_rows * T * bytes_per_token(I, H, ih_bytes) * job_handles) / 1e6:.0f} MB > 126 MB"
                             if job_rows * T * bytes_per_token(I, H, ih_bytes) * job_handles > 126e6 else
                             "working set below L2 (126 MB): this workload is latency-bound by its T dependent steps, "
                             "not by memory; timed as is",
                       "plan": plan},
            "roofline": {"bound": "hbm", "kernel": kernel + " (one direction)", "achieved": achieved,
                         "peak": hbm, "unit": "GB/s", "frac": achieved / hbm, "peak_kind": peak_kind,
                         "traffic": traffic, "us_per_timestep": rec_ms * 1e3 / T,
                         "sync_floor_us_per_timestep": floor_us,
                         "sync_floor_frac": (floor_us / (rec_ms * 1e3 / T)) if floor_us and rec_ms > 0 else None,
                         "input_gemm_ms": gemm_ms, "recurrence_ms": rec_ms,
                         "whole_forward_frac": (tokens_step / world * bytes_per_token(I, H, ih_bytes) * job_handles /
                                                ((ms_total / args.steps) * 1e-3) / 1e9) / hbm},
            "e2e": {"value": e2e, "unit": "tokens/s",
                    "h2d_bytes_per_step": int(T * job_rows * I * 4),
                    "d2h_bytes_per_step": int((T + 1) * job_rows * H * 4 * job_handles)},
            "gpu_launches": int(launches),
            "clocks": clk.summary(),
        }
        result["e2e"]["d2h_gb_per_s_this_rank"] = (T + 1) * job_rows * H * 4 * job_handles * e2e_steps / (ms_e2e * 1e-3) / 1e9
        result["e2e"]["limited_by"] = "device-to-host copy of the fp32 outputs over PCIe (pinned host memory, two copy streams)"
        if e2e_narrow is not None:
            result["e2e_narrow"] = e2e_narrow
        if check is not None:
            result["check"] = check
        if gather is not None:
            result["gather"] = gather
        if strong is not None:
            result["strong"] = strong
        if world == 1 and not args.no_cpu_baseline:
            result["cpu_baseline"] = cpu_baseline(args.workload, budget_s=15.0)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if result is not None:
        print(json.dumps(result))
    if check is not None and not check["bit_exact"]:
        raise SystemExit("bench: the GPU result differs from the CPU integer path")


# ------------------------------------------------------------------ CPU baseline / reference arm
def cpu_problem(workload):
    """Quantized operands of one small batch for the CPU integer path (both directions)."""
    from oracle.binding import Oracle, reference_or_none
    from oracle.cases import make_case
    I, H, B_unit, T, bidir, cfg_name, xdist, _ = WORKLOADS[workload]
    ref = reference_or_none()
    chk = ref or Oracle()
    cores = os.cpu_count() or 1
    rows = max(1, min(B_unit, 2 * cores))
    cases = []
    for d in range(2 if bidir else 1):
        # calibration on a short, narrow batch: it fixes the values, not the running time
        cal = make_case(1000 + d, min(T, 20), 4, I, H, chk, workloads.config_named(cfg_name), dist=xdist,
                        calib_batches=1, oracle=Oracle())
        x = workloads.gen_x(np.random.default_rng(77 + d), T, rows, I, xdist)
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
        "impl": "reference", "metric": METRIC, "value": value,
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
