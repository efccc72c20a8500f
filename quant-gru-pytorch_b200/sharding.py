"""Partition of one GRU forward over several GPUs: one process per GPU, no data-path collective.

Rows of a batch never interact in a GRU and the two directions of a bidirectional layer are
independent until their outputs are concatenated, so the work is cut direction-major, then by
contiguous batch slices.  Every rank holds its direction's full weights and quant params
(a few MB).  A collective appears only when the caller asks for one gathered tensor:
``gather_outputs`` all-gathers the per-rank slices (NCCL on GPUs, gloo in the CPU tests).
The reference has no multi-GPU support at all; this module is new design.
"""
from dataclasses import dataclass

import torch
import torch.distributed as dist


@dataclass(frozen=True)
class Shard:
    rank: int
    directions: tuple      # (0,), (1,) or (0, 1)
    b0: int                # first batch row (inclusive)
    b1: int                # last batch row (exclusive)

    @property
    def rows(self):
        return self.b1 - self.b0


def plan_shards(world_size, batch, bidirectional):
    """Direction-major, then batch.  With two directions and an even world size each
    direction gets half the ranks; otherwise every rank runs every direction on its slice.
    Slices differ by at most one row; ranks beyond the batch size get an empty slice."""
    if world_size < 1 or batch < 1:
        raise ValueError("world_size and batch must be positive")
    if bidirectional and world_size % 2 == 0:
        per_dir = world_size // 2
        groups = [((0,), list(range(0, per_dir))), ((1,), list(range(per_dir, world_size)))]
    else:
        groups = [((0, 1) if bidirectional else (0,), list(range(world_size)))]
    shards = [None] * world_size
    for dirs, ranks in groups:
        n = len(ranks)
        for i, r in enumerate(ranks):
            shards[r] = Shard(r, dirs, batch * i // n, batch * (i + 1) // n)
    return shards


def slice_input(x, shard, batch_first=False):
    """The rows of x ([T,B,I] or [B,T,I]) a shard works on (a view, no copy)."""
    return x[shard.b0:shard.b1] if batch_first else x[:, shard.b0:shard.b1]


def gather_outputs(local_out, local_hn, shards, rank, hidden, batch, T, bidirectional, group=None):
    """All-gather per-rank results into output [T,B,D*H] and h_n [D,B,H] on every rank.

    local_out: [T, rows, len(directions)*H], local_hn: [len(directions), rows, H] of this rank.
    Slices are padded to the largest slice so one all_gather of equal-size tensors suffices."""
    world = len(shards)
    D = 2 if bidirectional else 1
    max_rows = max(s.rows for s in shards)
    nd_max = max(len(s.directions) for s in shards)
    me = shards[rank]
    pad_out = local_out.new_zeros((T, max_rows, nd_max * hidden))
    pad_hn = local_hn.new_zeros((nd_max, max_rows, hidden))
    if me.rows:
        pad_out[:, :me.rows, :local_out.shape[2]] = local_out
        pad_hn[:local_hn.shape[0], :me.rows] = local_hn
    outs = [torch.empty_like(pad_out) for _ in range(world)]
    hns = [torch.empty_like(pad_hn) for _ in range(world)]
    dist.all_gather(outs, pad_out, group=group)
    dist.all_gather(hns, pad_hn, group=group)
    output = local_out.new_zeros((T, batch, D * hidden))
    h_n = local_hn.new_zeros((D, batch, hidden))
    for s, o, hn in zip(shards, outs, hns):
        if not s.rows:
            continue
        for k, d in enumerate(s.directions):
            output[:, s.b0:s.b1, d * hidden:(d + 1) * hidden] = o[:, :s.rows, k * hidden:(k + 1) * hidden]
            h_n[d, s.b0:s.b1] = hn[k, :s.rows]
    return output, h_n


def run_sharded(forward_dir, x, shards, rank, hidden, bidirectional, gather=False, group=None):
    """Run this rank's share.  forward_dir(direction, x_slice) -> (out [T,rows,H], h_n [1,rows,H]).

    Returns the rank-local (output, h_n), or the gathered tensors when gather=True."""
    me = shards[rank]
    T, B = x.shape[0], x.shape[1]
    xs = slice_input(x, me)
    outs, hns = [], []
    for d in me.directions:
        if me.rows:
            o, hn = forward_dir(d, xs)
        else:
            o = x.new_zeros((T, 0, hidden), dtype=x.dtype)
            hn = x.new_zeros((1, 0, hidden), dtype=x.dtype)
        outs.append(o)
        hns.append(hn)
    local_out = torch.cat(outs, dim=-1) if len(outs) > 1 else outs[0]
    local_hn = torch.cat(hns, dim=0) if len(hns) > 1 else hns[0]
    if not gather:
        return local_out, local_hn
    return gather_outputs(local_out, local_hn, shards, rank, hidden, B, T, bidirectional, group)


def merge_ranges(ranges, group=None):
    """Union of MinMax calibration ranges collected on different ranks (element-wise min/max
    all-reduce of the range vector); every rank ends with the same ranges."""
    import numpy as np
    from .params import NUM_OPS, WEIGHT_OPS
    C3 = 3 * ranges.hidden
    mins = torch.from_numpy(np.concatenate([ranges.min_v] + [ranges.ch_min[n] for n in WEIGHT_OPS]).copy())
    maxs = torch.from_numpy(np.concatenate([ranges.max_v] + [ranges.ch_max[n] for n in WEIGHT_OPS]).copy())
    if dist.get_backend(group) == "nccl":
        mins, maxs = mins.cuda(), maxs.cuda()
    dist.all_reduce(mins, op=dist.ReduceOp.MIN, group=group)
    dist.all_reduce(maxs, op=dist.ReduceOp.MAX, group=group)
    mins, maxs = mins.cpu().numpy(), maxs.cpu().numpy()
    ranges.min_v[:] = mins[:NUM_OPS]
    ranges.max_v[:] = maxs[:NUM_OPS]
    for k, n in enumerate(WEIGHT_OPS):
        ranges.ch_min[n][:] = mins[NUM_OPS + k * C3:NUM_OPS + (k + 1) * C3]
        ranges.ch_max[n][:] = maxs[NUM_OPS + k * C3:NUM_OPS + (k + 1) * C3]
    return ranges
