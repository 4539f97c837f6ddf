"""Pins the CPU oracle (oracle/) against the stored outputs of the unmodified reference
(tests/golden/reference_vectors.npz, made by tests/golden/make_golden.py) and against the
reference's one literal known-answer vector. Runs without a GPU."""

import numpy as np
import pytest
import torch

import cases
from oracle import ep_oracle as eo
from oracle import moe_oracle as mo


def T(a):
    return torch.from_numpy(np.asarray(a))


def test_plan_known_answer():
    # the literal vector of the reference's tests/test_model.py:49-57
    idx = torch.tensor([[2, 0], [0, 1], [2, 1]])
    w = torch.tensor([[.6, .4], [.7, .3], [.5, .5]])
    p = mo.plan(idx, w, 4)
    assert p.counts.tolist() == [2, 2, 2, 0]
    assert p.offsets.tolist() == [0, 2, 4, 6, 6]
    assert p.token.tolist() == [0, 1, 1, 2, 0, 2]
    assert p.slot.tolist() == [1, 0, 1, 1, 0, 0]
    assert torch.allclose(p.weight, torch.tensor([.4, .7, .3, .5, .6, .5]))
    counts, offsets, token, wsorted, pos_of = mo.sort_by_expert(idx.int(), w, 4)
    assert counts.tolist() == [2, 2, 2, 0] and offsets.tolist() == [0, 2, 4, 6, 6]
    assert token.tolist() == [0, 1, 1, 2, 0, 2]
    assert pos_of.tolist() == [4, 0, 1, 2, 5, 3]


@pytest.mark.parametrize("name", list(cases.ROUTE_CASES))
@pytest.mark.parametrize("norm", [False, True])
def test_route_rules_match_the_reference(golden, name, norm):
    E, k, N = cases.ROUTE_CASES[name]
    logits = cases.route_logits(E, N)
    assert cases.checksum(logits) == golden[f"route/{name}/logits_sum"]
    ridx = T(golden[f"route/{name}/norm{int(norm)}/idx"]).long()
    rw = T(golden[f"route/{name}/norm{int(norm)}/w"])
    # the restated reference math reproduces the stored reference output exactly
    torch.set_num_threads(1)
    idx2, w2 = mo.route_reference(logits, torch.eye(E, dtype=logits.dtype), k, norm)
    assert torch.equal(idx2, ridx) and torch.equal(w2, rw)
    # the kernel rule picks the same experts except where candidates tie to within rounding
    # (the allowance of the reference's tests/test_kernels_cuda.py:28-38)
    kidx, kw = mo.route_kernel_rule(logits, k, norm)
    probs = torch.softmax(logits.float(), -1)
    same = (kidx.long().sort(-1).values == ridx.sort(-1).values).all(-1)
    for t in torch.nonzero(~same).flatten().tolist():
        mine, ref = set(kidx[t].tolist()), set(ridx[t].tolist())
        gap = (probs[t, list(mine - ref)].sum() - probs[t, list(ref - mine)].sum()).abs().item()
        assert gap < 1e-6, (t, mine ^ ref, gap)
    assert same.float().mean().item() > 0.99
    assert (kw.float().sort(-1).values - rw.float().sort(-1).values)[same].abs().max().item() < 1e-3
    # kernel rule properties: descending probability, lower index first on exact ties
    p = torch.gather(probs, 1, kidx.long())
    ev = torch.exp(logits.float() - logits.float().max(-1, keepdim=True).values)
    e_sel = torch.gather(ev, 1, kidx.long())
    assert (e_sel[:, :-1] >= e_sel[:, 1:]).all()
    tie = e_sel[:, :-1] == e_sel[:, 1:]
    assert (kidx[:, :-1][tie] < kidx[:, 1:][tie]).all()
    del p


def test_route_kernel_rule_breaks_ties_to_the_lower_index():
    logits = torch.zeros(3, 64, dtype=torch.float16)
    logits[1, 40:] = 1.0
    logits[2, ::2] = 0.5
    idx, w = mo.route_kernel_rule(logits, 8, False)
    assert idx[0].tolist() == list(range(8))
    assert idx[1].tolist() == list(range(40, 48))
    assert idx[2].tolist() == list(range(0, 16, 2))
    assert abs(w[0, 0].item() - 1 / 64) < 1e-4


@pytest.mark.parametrize("name", list(cases.SORT_CASES))
def test_sort_matches_the_reference(golden, name):
    E, k, N, seed = cases.SORT_CASES[name]
    idx, w = cases.sort_inputs(E, k, N, seed)
    assert cases.checksum(idx.float()) + cases.checksum(w) == golden[f"sort/{name}/in_sum"]
    got = mo.sort_by_expert(idx, w, E)
    for g, key in zip(got, ("counts", "offsets", "token", "wsorted", "pos_of")):
        assert torch.equal(g, T(golden[f"sort/{name}/{key}"])), key
    p = mo.plan(idx, w, E)
    assert torch.equal(p.slot.int(), T(golden[f"sort/{name}/slot"]))


@pytest.mark.parametrize("name", list(cases.LAYER_CASES))
def test_expert_math_matches_the_reference(golden, name):
    spec = cases.LAYER_CASES[name]
    h, router, gu, dn = cases.layer_inputs(**spec)
    assert sum(cases.checksum(t) for t in (h, router, gu, dn)) == golden[f"layer/{name}/in_sum"]
    torch.set_num_threads(1)
    ridx, rw = mo.route_reference(h, router, spec["k"], False)
    assert torch.equal(ridx.int(), T(golden[f"layer/{name}/ridx"]))
    assert torch.equal(rw, T(golden[f"layer/{name}/rw"]))
    want = mo.experts_reference(h.float(), ridx, rw.float(), gu.float(), dn.float())
    assert torch.equal(want, T(golden[f"layer/{name}/want_fp32"]))
    assert torch.equal(mo.experts_grouped(h.float(), ridx, rw.float(), gu.float(), dn.float()), want)
    if h.dtype != torch.float32:
        # the kernel-rule layer (rounding points of the CUDA epilogues, expert-order combine)
        # stays inside the reference's own tolerance: err <= max(2 * err of the 16-bit loop, 2e-3)
        loop16 = T(golden[f"layer/{name}/loop16"]).float()
        counts, offsets, token, wsorted, pos_of = mo.sort_by_expert(ridx.int(), rw, gu.shape[0])
        y = mo.ffn_sorted_kernel_rule(h, token, offsets, wsorted, gu, dn)
        got = mo.combine_expert_order(y, pos_of, ridx.int(), h.shape[0]).float()
        err, err16 = (got - want).abs().max().item(), (loop16 - want).abs().max().item()
        assert err <= max(2 * err16, 2e-3), (err, err16)


def test_combine_rules_agree_in_float32():
    # in float32 the expert-order combine and the reference's index_add_ combine coincide
    g = cases.gen(7)
    idx, w = cases.sort_inputs(16, 4, 50, 9)
    counts, offsets, token, wsorted, pos_of = mo.sort_by_expert(idx, w.float(), 16)
    y = torch.randn(idx.numel(), 24, generator=g)
    a = mo.combine_expert_order(y, pos_of, idx, 50)
    b = eo.TorchOps().combine(y, pos_of, idx, 50)
    assert torch.equal(a, b)


@pytest.mark.parametrize("name", list(cases.EP_CASES))
def test_expert_parallel_oracle_matches_the_reference(golden, name):
    R, sizes = cases.EP_CASES[name]
    router, gu, dn, hs = cases.ep_inputs(R, sizes)
    torch.set_num_threads(1)
    outs, crossed = eo.expert_parallel_layer(hs, router, gu, dn, cases.EP_K, False)
    for r, o in enumerate(outs):
        assert torch.equal(o, T(golden[f"ep/{name}/out/{r}"]))
        assert torch.equal(o, eo.single_device_layer(hs[r], router, gu, dn, cases.EP_K, False))
    assert crossed == int(golden[f"ep/{name}/dispatched_rows"])
    # placement: what lands in inbox[d][r], bit for bit
    ops = eo.TorchOps()
    for r, h in enumerate(hs):
        idx, w = ops.route(h, router, cases.EP_K, False)
        counts, offsets, token, wsorted, pos_of = ops.sort(idx, w, cases.EP_E)
        place = eo.dispatch_placement(offsets, counts, token, wsorted, R)
        assert [list(p["seg"]) for p in place] == golden[f"ep/{name}/seg/{r}"].tolist()
        for d, p in enumerate(place):
            pre = f"ep/{name}/inbox/{d}/{r}"
            if d == r or p["seg"][0] == p["seg"][1]:
                assert pre + "/x" not in golden.files
                continue
            assert torch.equal(h[p["token"].long()], T(golden[pre + "/x"]))
            assert torch.equal(p["offsets"], T(golden[pre + "/offsets"]))
            assert torch.equal(p["counts"], T(golden[pre + "/counts"]))
            assert torch.equal(p["w"], T(golden[pre + "/w"]))
