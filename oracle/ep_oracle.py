"""CPU oracle for the expert-parallel protocol. TEST INFRASTRUCTURE ONLY.

Restates in plain PyTorch on the CPU (a) the seven operations the reference's expert-parallel
runtime calls (`TorchOps`, switchyard/ep.py:31-64) and (b) the placement rule of its dispatch
(switchyard/ep.py:174-224, 239-262): which sorted rows go to which rank, how the per-expert
offsets are rebased, and where results return. The product's `ExpertParallel` takes an `ops`
object; the tests hand it `TorchOps` to run the whole protocol on CPU "ranks". The product
itself never constructs this class.

Parity status: pinned by `tests/golden/make_golden.py` (outputs of the unmodified reference's
`ExpertParallel(["cpu"]*R)` stored as fixtures) and `tests/test_oracle.py`.
"""

from __future__ import annotations

import torch

from . import moe_oracle as mo


class TorchOps:
    """switchyard/ep.py:31-64: route, sort, ffn, combine, gather_to, copy_to, host."""

    def route(self, h, router, k, norm):
        idx, w = mo.route_reference(h, router, k, norm)
        return idx.int(), w

    def sort(self, idx, w, E):
        return mo.sort_by_expert(idx, w, E)

    def ffn(self, x, a_rows, offsets, counts, wsorted, gate_up, down, rows, host_counts=None):
        xs = x[a_rows.long()] if a_rows is not None else x
        return mo.run_sorted(xs, counts.long(), gate_up, down) * wsorted[:, None]

    def combine(self, y, pos_of, idx, N):
        # rows are sorted by expert, so adding them in row order adds each token's k results
        # in expert order (switchyard/ep.py:48-55)
        k = idx.shape[1]
        token = torch.empty(idx.numel(), dtype=torch.int64)
        token[pos_of.long()] = torch.arange(idx.numel()) // k
        out = torch.zeros(N, y.shape[1], dtype=y.dtype)
        out.index_add_(0, token, y)
        return out

    def gather_to(self, src, index, dst):
        dst.copy_(src[index.long()])

    def copy_to(self, dst, src):
        dst.copy_(src)

    def host(self, t):
        return t.tolist()


def single_device_layer(h, router, gate_up, down, k, norm, ops=None):
    """The one-device comparand of the reference's CPU protocol test
    (tests/test_ep.py:19-24)."""
    ops = ops or TorchOps()
    idx, w = ops.route(h, router, k, norm)
    counts, offsets, token, wsorted, pos_of = ops.sort(idx, w, gate_up.shape[0])
    y = ops.ffn(h, token, offsets, counts, wsorted, gate_up, down, idx.numel())
    return ops.combine(y, pos_of, idx, h.shape[0])


def dispatch_placement(offsets, counts, token, wsorted, R):
    """Placement rule of the dispatch (switchyard/ep.py:190-223). For a sender whose sorted
    rows are described by (offsets [E+1], counts [E], token [M], wsorted [M]) and R ranks
    owning E/R contiguous experts each, returns for every destination d a dict with
      seg      (a, b): the sender's sorted rows bound for d (contiguous),
      token    token[a:b]          (the rows of h to ship, in order),
      offsets  offsets[d*per:(d+1)*per+1] - a   (rebased per-expert offsets, int32),
      counts   counts[d*per:(d+1)*per],
      w        wsorted[a:b].
    Results for those rows come back into the sender's y[a:b] (switchyard/ep.py:259-260)."""
    E = counts.numel()
    per = E // R
    off = offsets.tolist()
    out = []
    for d in range(R):
        a, b = off[d * per], off[(d + 1) * per]
        out.append(dict(seg=(a, b), token=token[a:b].clone(),
                        offsets=(offsets[d * per:(d + 1) * per + 1] - a).to(offsets.dtype),
                        counts=counts[d * per:(d + 1) * per].clone(), w=wsorted[a:b].clone()))
    return out


def expert_parallel_layer(hs, router, gate_up, down, k, norm, ops=None):
    """A direct (no threads, no inboxes) restatement of one expert-parallel layer: every rank
    routes and sorts its own tokens, each destination runs its experts on each sender's
    segment separately, results return to the sender's rows, the sender combines.
    hs: list of [N_r,H]; gate_up/down: the FULL expert stacks. Returns outputs per rank and
    the number of rows that crossed ranks."""
    ops = ops or TorchOps()
    R = len(hs)
    E = gate_up.shape[0]
    per = E // R
    outs, crossed = [], 0
    for r, h in enumerate(hs):
        idx, w = ops.route(h, router, k, norm)
        counts, offsets, token, wsorted, pos_of = ops.sort(idx, w, E)
        y = torch.empty(idx.numel(), h.shape[1], dtype=h.dtype)
        for d, p in enumerate(dispatch_placement(offsets, counts, token, wsorted, R)):
            a, b = p["seg"]
            if b == a:
                continue
            x = h[p["token"].long()]
            y[a:b] = ops.ffn(x, None, p["offsets"], p["counts"], p["w"],
                             gate_up[d * per:(d + 1) * per], down[d * per:(d + 1) * per], b - a)
            crossed += (b - a) if d != r else 0
        outs.append(ops.combine(y, pos_of, idx, h.shape[0]))
    return outs, crossed
