"""The expert-parallel host logic (segments, mailboxes, rebased offsets, return placement,
barriers, threads, capacity drop, trace, failure handling) on CPU "ranks". The package has no
CPU operations of its own; the seven protocol operations are injected from the oracle. Cases
follow the reference's tests/test_ep.py."""

import math

import numpy as np
import pytest
import torch

import cases
from oracle import ep_oracle as eo
from oracle import moe_oracle as mo
from switchyard_b200.ep import ExpertParallel


def T(a):
    return torch.from_numpy(np.asarray(a))


def split(gu, dn, R):
    per = gu.shape[0] // R
    return [gu[r * per:(r + 1) * per] for r in range(R)], [dn[r * per:(r + 1) * per] for r in range(R)]


@pytest.mark.parametrize("name", list(cases.EP_CASES))
def test_layer_is_bit_identical_to_one_device_and_to_the_reference(golden, name):
    R, sizes = cases.EP_CASES[name]
    router, gu, dn, hs = cases.ep_inputs(R, sizes)
    torch.set_num_threads(1)
    ep = ExpertParallel(["cpu"] * R, cases.EP_E, cases.EP_K, False, ops=eo.TorchOps())
    gus, dns = split(gu, dn, R)
    outs = ep.layer(hs, [router] * R, gus, dns)
    for r, (h, o) in enumerate(zip(hs, outs)):
        assert torch.equal(o, eo.single_device_layer(h, router, gu, dn, cases.EP_K, False))
        assert torch.equal(o, T(golden[f"ep/{name}/out/{r}"]))  # the reference's own output
        if h.shape[0]:
            idx, w = mo.route_reference(h, router, cases.EP_K, False)
            assert torch.allclose(o, mo.experts_reference(h, idx, w, gu, dn), atol=1e-5)
    assert ep.stats["dispatched_rows"] == int(golden[f"ep/{name}/dispatched_rows"])
    assert ep.stats["local_rows"] == int(golden[f"ep/{name}/local_rows"])
    if R > 1 and sum(sizes) > 4:
        assert ep.stats["dispatched_rows"] > 0
    threaded = ep.layer_threaded(hs, [router] * R, gus, dns)
    assert all(torch.equal(a, b) for a, b in zip(outs, threaded))
    # a second layer reuses the mailboxes
    again = ep.layer(hs, [router] * R, gus, dns)
    assert all(torch.equal(a, b) for a, b in zip(outs, again))


@pytest.mark.parametrize("name", ["r2_0", "r4_2"])
def test_mailbox_contents_match_the_reference(golden, name):
    R, sizes = cases.EP_CASES[name]
    router, gu, dn, hs = cases.ep_inputs(R, sizes)
    ep = ExpertParallel(["cpu"] * R, cases.EP_E, cases.EP_K, False, ops=eo.TorchOps())
    sh = ep.new_state()
    for r in range(R):
        ep.phase_send(sh, r, hs[r], router)
    for d in range(R):
        for r in range(R):
            m, pre = sh["inbox"][d][r], f"ep/{name}/inbox/{d}/{r}"
            if m is None:
                assert pre + "/x" not in golden.files
                continue
            assert torch.equal(m["x"], T(golden[pre + "/x"]))
            assert torch.equal(m["offsets"], T(golden[pre + "/offsets"]))
            assert torch.equal(m["counts"], T(golden[pre + "/counts"]))
            assert torch.equal(m["w"], T(golden[pre + "/w"]))
            assert m["rows"] == m["x"].shape[0]
        assert [list(s) for s in sh["st"][d]["seg"]] == golden[f"ep/{name}/seg/{d}"].tolist()


def test_eight_ranks():
    R = 8
    g = cases.gen(3)
    E, k, H, I = 64, 8, 32, 16
    router = torch.randn(E, H, generator=g)
    gu, dn = torch.randn(E, 2 * I, H, generator=g) * 0.3, torch.randn(E, H, I, generator=g) * 0.3
    hs = [torch.randn(n, H, generator=g) for n in (3, 0, 17, 1, 9, 30, 2, 8)]
    ep = ExpertParallel(["cpu"] * R, E, k, False, ops=eo.TorchOps())
    gus, dns = split(gu, dn, R)
    for outs in (ep.layer(hs, [router] * R, gus, dns), ep.layer_threaded(hs, [router] * R, gus, dns)):
        for h, o in zip(hs, outs):
            assert torch.equal(o, eo.single_device_layer(h, router, gu, dn, k, False))
    assert ep.owner(0) == 0 and ep.owner(63) == 7 and ep.owner(8) == 1


def test_a_failing_rank_does_not_hang_the_others():
    ep = ExpertParallel(["cpu", "cpu"], 4, 2, False, ops=eo.TorchOps())

    def fn(r):
        if r == 1:
            raise ValueError("boom")
        ep.barrier.wait()

    with pytest.raises(ValueError, match="boom"):
        ep.run_ranks(fn)
    assert ep.run_ranks(lambda r: r) == [0, 1]  # usable again


def _dropped_reference(h, router, gu, dn, k, cf):
    idx, w = mo.route_reference(h, router, k, False)
    E, M = router.shape[0], idx.numel()
    cap = math.ceil(cf * M / E)
    w = w.clone()
    seen = [0] * E
    for t in range(idx.shape[0]):
        for s in range(k):
            e = int(idx[t, s])
            if seen[e] >= cap:
                w[t, s] = 0
            seen[e] += 1
    return mo.experts_reference(h, idx, w, gu, dn), sum(max(0, c - cap) for c in seen)


@pytest.mark.parametrize("cf", cases.CAPACITY_FACTORS)
def test_capacity_drops_rows_past_each_experts_capacity_in_token_order(golden, cf):
    router, gu, dn, hs = cases.capacity_inputs()
    torch.set_num_threads(1)
    E, k, R = cases.EP_E, cases.EP_K, 2
    ep = ExpertParallel(["cpu"] * R, E, k, False, ops=eo.TorchOps())
    ep.capacity_factor = cf
    gus, dns = split(gu, dn, R)
    outs = ep.layer(hs, [router] * R, gus, dns)
    dropped = 0
    for r, (h, o) in enumerate(zip(hs, outs)):
        want, d = _dropped_reference(h, router, gu, dn, k, cf)
        dropped += d
        assert torch.allclose(o, want, atol=1e-5)
        assert torch.equal(o, T(golden[f"cap/{cf}/out/{r}"]))
    assert ep.stats["dropped_rows"] == dropped == int(golden[f"cap/{cf}/dropped"])
    assert ep.stats["routed_rows"] == sum(h.shape[0] for h in hs) * k == int(golden[f"cap/{cf}/routed"])
    assert (dropped == 0) == (cf == 100.0)


def test_trace_counts_every_routed_row():
    router, gu, dn, hs = cases.ep_inputs(2, (9, 9))
    ep = ExpertParallel(["cpu"] * 2, cases.EP_E, cases.EP_K, False, ops=eo.TorchOps())
    ep.trace = []
    gus, dns = split(gu, dn, 2)
    for _ in range(3):
        ep.layer(hs, [router] * 2, gus, dns)
    assert len(ep.trace) == 3 * 2
    for r, counts in ep.trace:
        assert int(counts.sum()) == 9 * cases.EP_K
