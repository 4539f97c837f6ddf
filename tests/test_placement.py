"""Expert placement (switchyard_b200.placement): the cases of the reference's placement tests
(tests/test_ep.py:141-160) on this package's functions, the refinement beyond the greedy deal,
and the device-side load meter on the CPU."""

import torch

from switchyard_b200 import placement as pl


def test_balanced_placement_evens_out_a_skewed_load():
    load = torch.tensor([100.0, 90, 80, 70] + [10.0] * 12)
    assert pl.imbalance(pl.rank_rows(load, pl.contiguous(16), 2)) > 1.3
    p = pl.balanced(load, 2)
    assert sorted(p) == list(range(16))
    assert pl.imbalance(pl.rank_rows(load, p, 2)) < 1.03


def test_eight_ranks_with_a_zipf_load():
    from switchyard_b200 import synthetic
    # the benchmark's skew: expected rows per expert under the Zipf router bias
    bias = synthetic.zipf_bias()
    load = torch.softmax(bias.double() * 1.3, 0) * 65536  # busiest expert about four times the mean
    before = pl.imbalance(pl.rank_rows(load, pl.contiguous(64), 8))
    p = pl.balanced(load, 8)
    after = pl.imbalance(pl.rank_rows(load, p, 8))
    assert sorted(p) == list(range(64)) and all(len(set(p[r * 8:(r + 1) * 8])) == 8 for r in range(8))
    assert before > 1.2 and after < 1.05
    assert pl.rank_rows(load, p, 8).sum().item() == torch.as_tensor(load).sum().item()


def test_swaps_improve_on_the_greedy_deal():
    # a load where dealing heaviest-first leaves one rank heavier than a swap can make it
    load = [9.0, 8, 7, 6, 5, 5, 4, 4, 1, 1, 1, 1]
    p = pl.balanced(load, 3, sweeps=0)
    q = pl.balanced(load, 3)
    assert pl.imbalance(pl.rank_rows(load, q, 3)) <= pl.imbalance(pl.rank_rows(load, p, 3))
    assert sorted(q) == list(range(12))


def test_degenerate_loads():
    assert pl.imbalance([0, 0]) == 1.0
    assert pl.balanced([0.0] * 8, 4) == list(range(8))
    assert pl.balanced([5.0, 1, 1, 1], 4) == [0, 1, 2, 3]


def test_load_meter_accumulates():
    m = pl.LoadMeter(4, "cpu")
    m.add(torch.tensor([1, 0, 2, 0], dtype=torch.int32))
    m.add(torch.tensor([0, 5, 0, 0], dtype=torch.int32))
    assert m.read() == [1, 5, 2, 0]
    m.reset()
    assert m.read() == [0, 0, 0, 0]


def test_properties_on_random_loads():
    """Whatever the load: a permutation with E/R experts per rank, never heavier than contiguous
    blocks, every row accounted for."""
    from hypothesis import given, settings, strategies as st

    @settings(max_examples=150, deadline=None)
    @given(st.sampled_from([2, 4, 8]), st.integers(1, 4), st.data())
    def check(ranks, per, data):
        E = ranks * per
        load = data.draw(st.lists(st.integers(0, 5000), min_size=E, max_size=E))
        got = pl.balanced(load, ranks)
        assert sorted(got) == list(range(E))
        rows = pl.rank_rows(load, got, ranks)
        assert rows.max().item() <= pl.rank_rows(load, pl.contiguous(E), ranks).max().item() + 1e-9
        assert rows.sum().item() == float(sum(load))

    check()
