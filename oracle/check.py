"""TEST INFRASTRUCTURE: compare a full-size GPU forward with the CPU integer path on a row subset.

Batch rows of a GRU never interact, so any subset of the rows of a large GPU result can be
checked against the reference's CPU integer forward (cpu::ForwardPassQuantCPU::Run,
src/gru_forward_cpu_quant.cc:290-340 of the reference; oracle/_ref when it is built, else the
C restatement) run on just those rows - every timestep, bit for bit.  Used by the full-size
parity tests and by bench.py's post-run check; never by the product.
"""
import os

import numpy as np

from .binding import Oracle, reference_or_none
from .cases import OP


def spread_rows(B, n, group=16):
    """Up to n row indices of [0, B): the whole first and last group of `group` rows (the first
    and last tile of a batch-tiled kernel, the last one possibly ragged) and the rest evenly
    spaced in between."""
    if n >= B:
        return np.arange(B)
    first = list(range(min(group, B)))
    last = list(range(max(0, B - group), B))
    rest = max(0, n - len(first) - len(last))
    mid = np.linspace(group, B - group - 1, rest).astype(int).tolist() if rest > 0 and B > 2 * group else []
    return np.array(sorted(set(first + mid + last)), dtype=np.int64)


def checker():
    """The compiled reference if present, else the C port."""
    return reference_or_none() or Oracle()


def check_forward_rows(chk, handle, qp, x, out, rows, reverse=False, threads=None):
    """Compare rows `rows` of a GPU forward with the CPU integer path.

    handle: gru_ops.Handle after set_params/set_weights (its quantized weights are read back);
    qp: the GRUQuantParams it runs with; x: numpy [T, B, I] fp32 (the GPU's input);
    out: the GPU result [(T+1), B, H], torch or numpy, fp32 (dequantized) or int32.
    Returns {"rows": n, "steps": T, "mismatches": count, "kind": ...}."""
    T, B, I = x.shape
    H = handle.hidden_size
    rows = np.asarray(rows)
    wq = [t.cpu().numpy() for t in handle.get_weights_i32()]
    xs = np.ascontiguousarray(x[:, rows, :])
    if reverse:
        xs = np.ascontiguousarray(xs[::-1])
    x_q = chk.quantize(xs, qp.c, OP["x"])
    threads = threads or min(len(rows), os.cpu_count() or 1)
    want = chk.forward_i32(T, len(rows), I, H, wq, x_q, None, qp.c, qp.scale_list(), threads=max(1, threads))
    if reverse:   # slot k of the reverse result is the state after consuming x[k]; slot T the initial one
        want = np.ascontiguousarray(want[::-1])
    got = out[:, rows, :] if isinstance(out, np.ndarray) else out[:, rows.tolist(), :].cpu().numpy()
    if got.dtype == np.float32:
        want_f = chk.dequantize(want, qp.c, OP["h"])
        bad = int(np.count_nonzero(got.view(np.uint32) != want_f.view(np.uint32)))
    else:
        bad = int(np.count_nonzero(got != want))
    return {"rows": int(len(rows)), "steps": int(T), "mismatches": bad, "kind": chk.kind}
