"""Where the experts live when they are split over ranks: measuring per-expert load without
stalling the device, and choosing a placement that evens out the rows each rank computes.

With expert parallelism the rank that holds the busiest experts finishes last and every other
rank waits for its results in the combine, so the layer's time is the busiest rank's time. On
eight GPUs a rank holds only eight experts, and one expert with four times the mean load is no
longer averaged away. A placement is a permutation of the experts: rank r holds
placement[r*E/R:(r+1)*E/R]; the router's rows are permuted the same way, so the model computes
the same function (`ep_dist.DistributedExpertParallel(placement=...)`, and the reference's
`serve.ParallelModel(placement=...)`, switchyard/serve.py:14-33).

Same role as switchyard/balance.py:11-40 (`rank_loads`, `imbalance`, `greedy`, `contiguous`);
`balanced` goes one step further than its greedy pass: after dealing the experts out by
decreasing load it keeps swapping pairs of experts between the busiest rank and the others
while that lowers the maximum."""

import torch


def contiguous(n_experts):
    """The default placement: rank r holds experts r*E/R .. (r+1)*E/R - 1."""
    return list(range(n_experts))


def rank_rows(load, placement, ranks):
    """Rows each rank computes for one layer: load[e] rows for expert e, rank r holding
    placement[r*E/R:(r+1)*E/R]. Returns a float64 tensor [ranks]."""
    load = torch.as_tensor(load, dtype=torch.float64)
    per = len(placement) // ranks
    index = torch.as_tensor(list(placement), dtype=torch.int64).view(ranks, per)
    return load[index].sum(1)


def imbalance(rows):
    """Busiest rank over the mean: 1.0 is perfect, and it is what the layer's time scales with."""
    rows = torch.as_tensor(rows, dtype=torch.float64)
    total = rows.sum().item()
    return rows.max().item() * rows.numel() / total if total > 0 else 1.0


def balanced(load, ranks, sweeps=8):
    """A placement with E/R experts per rank whose busiest rank is as light as a greedy deal
    plus pairwise swaps can make it, and never heavier than with contiguous blocks. load:
    per-expert rows (any sequence or tensor)."""
    load = [float(x) for x in torch.as_tensor(load, dtype=torch.float64).tolist()]
    E = len(load)
    assert E % ranks == 0, "experts must split evenly over the ranks"
    per = E // ranks
    held = [[] for _ in range(ranks)]
    weight = [0.0] * ranks
    # deal: heaviest expert first, to the lightest rank that still has a free slot
    for e in sorted(range(E), key=lambda e: (-load[e], e)):
        r = min((r for r in range(ranks) if len(held[r]) < per), key=lambda r: (weight[r], r))
        held[r].append(e)
        weight[r] += load[e]
    # refine: swap one expert of the busiest rank with one of another rank if the pair's
    # maximum drops; stop when no swap helps
    for _ in range(sweeps * ranks):
        top = max(range(ranks), key=lambda r: weight[r])
        best = None
        for other in range(ranks):
            if other == top:
                continue
            for a in held[top]:
                for b in held[other]:
                    delta = load[a] - load[b]
                    if delta <= 0:
                        continue
                    new_max = max(weight[top] - delta, weight[other] + delta)
                    if new_max < weight[top] - 1e-12 and (best is None or new_max < best[0]):
                        best = (new_max, other, a, b)
        if best is None:
            break
        _, other, a, b = best
        held[top][held[top].index(a)] = b
        held[other][held[other].index(b)] = a
        weight[top] += load[b] - load[a]
        weight[other] += load[a] - load[b]
    placement = [e for r in range(ranks) for e in sorted(held[r])]
    # never hand back something worse than the default: on a load that happens to suit the
    # contiguous blocks the deal can end above them
    if max(weight) > rank_rows(load, contiguous(E), ranks).max().item() + 1e-9:
        return contiguous(E)
    return placement


class LoadMeter:
    """Adds up per-expert row counts on the device. `add(counts)` takes the sort's `counts`
    tensor (int32 [E]) of a layer and costs one small addition on the current stream; nothing is
    read back until `read()`. One meter per layer gives per-layer placements."""

    def __init__(self, n_experts, device):
        self.total = torch.zeros(n_experts, dtype=torch.int64, device=device)

    def add(self, counts):
        self.total += counts

    def read(self):
        """Per-expert rows so far as a list (waits for the device)."""
        return self.total.tolist()

    def reset(self):
        self.total.zero_()
