"""Host logic of the multi-GPU partition, run as world_size-2/3/4 gloo ranks on the CPU.

The per-rank forward is stood in by the oracle (a rank's CUDA forward gives the same integers,
as the GPU parity tests show); what is exercised here is the partition (direction-major, then
batch), the optional all-gather of outputs and the min/max union of calibration ranges."""
import importlib
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from __graft_entry__ import PKG_NAME, load_package

load_package()
sharding = importlib.import_module(PKG_NAME + ".sharding")


def test_plan_shards_covers_batch_once():
    for world in (1, 2, 3, 4, 8):
        for batch in (1, 5, 64, 257):
            for bidir in (False, True):
                shards = sharding.plan_shards(world, batch, bidir)
                assert [s.rank for s in shards] == list(range(world))
                for d in ((0, 1) if bidir else (0,)):
                    rows = sorted((s.b0, s.b1) for s in shards if d in s.directions and s.rows)
                    assert rows[0][0] == 0 and rows[-1][1] == batch
                    assert all(a[1] == b[0] for a, b in zip(rows, rows[1:]))
                sizes = [s.rows for s in shards]
                if bidir and world % 2 == 0:
                    assert all(s.directions in ((0,), (1,)) for s in shards)
                assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        sharding.plan_shards(0, 4, False)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, bidir, batch, result_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        load_package()
        from oracle.binding import Oracle
        from tests.cases import config_named, make_case, params_mod
        orc = Oracle()
        T, I, H = 5, 12, 16
        cases = [make_case(50 + d, T, batch, I, H, orc, config_named("cfg2")) for d in range(2 if bidir else 1)]
        x_q = torch.from_numpy(cases[0].x_q)

        def forward_dir(d, xs):
            c = cases[d]
            xin = xs.numpy()[::-1].copy() if d == 1 else xs.numpy()
            h = orc.forward_i32(T, xs.shape[1], I, H, c.wq, xin, None, c.params.c, c.params.scale_list())
            out = h[1:][::-1].copy() if d == 1 else h[1:]
            return torch.from_numpy(np.ascontiguousarray(out)), torch.from_numpy(h[-1:].copy())

        shards = sharding.plan_shards(world, batch, bidir)
        out, hn = sharding.run_sharded(forward_dir, x_q, shards, rank, H, bidir, gather=True)
        # every rank must hold the full, identical result
        want_o, want_h = [], []
        for d in range(len(cases)):
            o, h = forward_dir(d, x_q)
            want_o.append(o)
            want_h.append(h)
        assert torch.equal(out, torch.cat(want_o, -1)) and torch.equal(hn, torch.cat(want_h, 0))
        local_o, _ = sharding.run_sharded(forward_dir, x_q, shards, rank, H, bidir, gather=False)
        assert local_o.shape[1] == shards[rank].rows

        # calibration ranges collected on different ranks are merged to the same union
        r = params_mod.Ranges(H)
        r.min_v[:] = -1.0 - rank
        r.max_v[:] = 2.0 + rank
        for n in params_mod.WEIGHT_OPS:
            r.ch_min[n][:] = -0.5 * (rank + 1)
            r.ch_max[n][:] = 0.25 * (rank + 1)
        sharding.merge_ranges(r)
        assert np.all(r.min_v == -float(world)) and np.all(r.max_v == 1.0 + world)
        assert np.all(r.ch_min["R"] == -0.5 * world) and np.all(r.ch_max["bw"] == 0.25 * world)
        open(os.path.join(result_dir, f"ok{rank}"), "w").close()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,bidir,batch", [(2, True, 6), (2, False, 5), (3, True, 7), (4, True, 3)])
def test_sharded_forward_with_gather_gloo(tmp_path, world, bidir, batch):
    mp.spawn(_worker, args=(world, _free_port(), bidir, batch, str(tmp_path)), nprocs=world, join=True)
    assert all(os.path.exists(tmp_path / f"ok{r}") for r in range(world))
