"""Parity of the CUDA kernels, called through the C ABI (switchyard_b200.kernels), against the
CPU oracle and the stored outputs of the reference. Cases follow the reference's
tests/test_kernels_cuda.py and add bf16, the multi-block sort, row-grouping independence and
the full OLMoE layer shape.

Tolerances (written where they are used):
  * routing indices, sort outputs, combine: bit-exact;
  * routing weights: within one unit in the last place of the 16-bit result of the oracle;
  * layer output vs the float32 expert loop: max-abs error <= max(2 * error of the 16-bit
    PyTorch loop, 2e-3), the reference's own bound."""

import numpy as np
import pytest
import torch

import cases
from oracle import moe_oracle as mo

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def T(a):
    return torch.from_numpy(np.asarray(a))


@pytest.fixture(scope="module")
def K():
    from switchyard_b200 import kernels
    kernels.ext()
    yield kernels
    assert kernels.ext().device_status(DEV) == 0  # no kernel gave up on a wait


def force_tile(K, tile):
    """0 = automatic, 1 = one CTA per tile, 2 = CTA pairs."""
    assert K.ext().lib.sy_force_compute_tile(tile) == 0


def layer_logits(K, h, router):
    """The router logits moe_layer routes on: the library GEMM's, or (SWITCHYARD_FUSED_ROUTER=1) the
    ones the fused routing launch computes and reports."""
    if K.FUSED_ROUTER and K.fused_routing_applies(h.shape[0], router.shape[0], h.shape[1], 8):
        return K.ext().route_fused(h, router, 8, False, logits=True)[7]
    return torch.nn.functional.linear(h, router)


def ulp16(t):
    """Spacing of the 16-bit format at |t| (as float32)."""
    mant = 10 if t.dtype == torch.float16 else 7
    f = t.float().abs().clamp_min(2.0 ** -14)
    return torch.exp2(torch.floor(torch.log2(f)) - mant)


# ------------------------------------------------------------------------------ route
@pytest.mark.parametrize("name", list(cases.ROUTE_CASES))
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_route_is_bit_exact_against_the_kernel_rule(K, golden, name, dtype):
    E, k, N = cases.ROUTE_CASES[name]
    logits = cases.route_logits(E, N, dtype=dtype)
    for norm in (False, True):
        idx, w = K.ext().route(logits.to(DEV), k, norm)
        oidx, ow = mo.route_kernel_rule(logits, k, norm)
        assert idx.dtype == torch.int32 and w.dtype == dtype
        assert torch.equal(idx.cpu(), oidx)
        assert ((w.cpu().float() - ow.float()).abs() <= ulp16(ow)).all()
        if dtype == torch.float16:
            # against the reference's softmax + topk, with its own tie allowance
            ridx = T(golden[f"route/{name}/norm{int(norm)}/idx"]).long()
            rw = T(golden[f"route/{name}/norm{int(norm)}/w"])
            probs = torch.softmax(logits.float(), -1)
            same = (idx.cpu().long().sort(-1).values == ridx.sort(-1).values).all(-1)
            for t in torch.nonzero(~same).flatten().tolist():
                mine, ref = set(idx[t].tolist()), set(ridx[t].tolist())
                gap = (probs[t, list(mine - ref)].sum() - probs[t, list(ref - mine)].sum()).abs().item()
                assert gap < 1e-6
            assert same.float().mean().item() > 0.99
            assert (w.cpu().float().sort(-1).values - rw.float().sort(-1).values)[same].abs().max().item() < 1e-3


def test_route_ties_and_empty(K):
    logits = torch.zeros(3, 64, dtype=torch.float16)
    logits[1, 40:] = 1.0
    logits[2, ::2] = 0.5
    idx, w = K.ext().route(logits.to(DEV), 8, False)
    assert idx.cpu().tolist() == [list(range(8)), list(range(40, 48)), list(range(0, 16, 2))]
    idx, w = K.ext().route(torch.empty(0, 64, dtype=torch.float16, device=DEV), 8, False)
    assert idx.shape == (0, 8) and w.shape == (0, 8)
    with pytest.raises(RuntimeError):
        K.ext().route(torch.zeros(2, 200, dtype=torch.float16, device=DEV), 8, False)
    with pytest.raises(RuntimeError):
        K.ext().route(torch.zeros(2, 64, dtype=torch.float32, device=DEV), 8, False)


def test_route_through_the_router_gemm(K):
    h, router, _, _ = cases.layer_inputs(300)
    hd, rd = h.to(DEV), router.to(DEV)
    idx, w = K.route(hd, rd, 8, False)
    logits = torch.nn.functional.linear(hd, rd).cpu()  # the same fp16 logits the kernel saw
    oidx, ow = mo.route_kernel_rule(logits, 8, False)
    assert torch.equal(idx.cpu(), oidx)


def test_route_never_leaves_the_expert_range(K):
    """Rows of NaN, of -inf and of +inf have no valid softmax; the picks must still be experts
    in [0, E) (the k lowest, weight 0 where nothing is valid), so that nothing downstream
    indexes out of range."""
    logits = cases.route_logits(64, 6).clone()
    logits[1] = float("nan")
    logits[2] = float("-inf")
    logits[3, 5] = float("nan")
    logits[4] = float("inf")
    for norm in (False, True):
        idx, w = K.ext().route(logits.to(DEV), 8, norm)
        idx, w = idx.cpu(), w.cpu()
        assert ((idx >= 0) & (idx < 64)).all()
        for t in range(6):
            assert len(set(idx[t].tolist())) == 8
        assert idx[1].tolist() == list(range(8)) and idx[2].tolist() == list(range(8))
        assert (w[1] == 0).all() and (w[2] == 0).all()
        oidx, _ = mo.route_kernel_rule(logits[[0, 5]], 8, norm)
        assert torch.equal(idx[[0, 5]], oidx)  # ordinary rows are untouched


@pytest.mark.parametrize("N,E,k,H,dtype", [(1, 64, 8, 2048, torch.float16), (8, 64, 8, 2048, torch.float16),
                                           (64, 64, 8, 2048, torch.float16), (37, 64, 8, 256, torch.bfloat16),
                                           (200, 128, 8, 512, torch.float16), (50, 16, 4, 96, torch.float16),
                                           (1024, 8, 2, 64, torch.float16)])
def test_route_fused_is_the_kernel_rule_on_its_own_logits(K, N, E, k, H, dtype):
    """Router GEMM + route + sort in one launch. Contract: the routing is the kernel rule applied
    to the logits the launch writes out, the sort is sort_by_expert of that routing (both bit for
    bit), and those logits are the library GEMM's up to the 16-bit rounding of a differently
    ordered float32 sum. Against softmax + topk of the library GEMM's logits the reference's own
    tie allowance applies (tests/test_kernels_cuda.py:28-38)."""
    g = cases.gen(N + E)
    h = torch.randn(N, H, generator=g).to(dtype).to(DEV)
    router = (torch.randn(E, H, generator=g) * H ** -0.5 * 3).to(dtype).to(DEV)
    bias = (torch.randn(E, generator=g) * 0.3).to(dtype).to(DEV)
    for norm, b in ((False, None), (True, None), (False, bias)):
        a = K.ext().route_fused(h, router, k, norm, b, logits=True)
        again = K.ext().route_fused(h, router, k, norm, b, logits=True)
        assert all(torch.equal(x, y) for x, y in zip(a, again))  # the ticket comes back to zero; same bits
        idx, w, counts, offsets, token, wsorted, pos_of, logits = a
        oidx, ow = mo.route_kernel_rule(logits.cpu(), k, norm)
        assert torch.equal(idx.cpu(), oidx)
        assert ((w.cpu().float() - ow.float()).abs() <= ulp16(ow)).all()
        for got, want in zip((counts, offsets, token, wsorted, pos_of), K.ext().sort_by_expert(idx, w, E)):
            assert torch.equal(got, want)
        # the logits: the float32 dot products rounded to 16 bits (one step of slack for a sum that
        # lands on a rounding boundary, one more for the bias add); the library GEMM, which may
        # reduce in lower precision, is only required to be close
        exact = (h.float() @ router.float().t()).to(dtype)
        lib = torch.nn.functional.linear(h, router)
        if b is not None:
            exact, lib = exact + b, lib + b
        assert ((logits.float() - exact.float()).abs() <= (2 if b is not None else 1) * ulp16(exact) + 2e-5).all()
        assert ((logits.float() - lib.float()).abs() <= 16 * ulp16(lib) + 1e-3).all()
        if b is None and not norm:
            probs = torch.softmax(exact.float(), -1).cpu()
            ridx = probs.topk(k, -1).indices
            same = (idx.cpu().long().sort(-1).values == ridx.sort(-1).values).all(-1)
            for t in torch.nonzero(~same).flatten().tolist():
                mine, ref = set(idx[t].tolist()), set(ridx[t].tolist())
                gap = (probs[t, list(mine - ref)].sum() - probs[t, list(ref - mine)].sum()).abs().item()
                # only near-ties may differ: logits one 16-bit step apart
                assert gap < (0.02 if dtype == torch.float16 else 0.12) * probs[t, list(ref - mine)].sum().item()
            assert same.float().mean().item() >= (0.97 if dtype == torch.float16 else 0.9)
    assert K.ext().device_status() == 0


def test_route_fused_rows_do_not_depend_on_the_batch(K):
    """A token's logits (and so its routing) depend on its own row only: the same token routed
    alone, in a batch of 64 and at another position gives identical bits."""
    g = cases.gen(77)
    h = torch.randn(64, 2048, generator=g).half().to(DEV)
    router = (torch.randn(64, 2048, generator=g) * 0.02).half().to(DEV)
    full = K.ext().route_fused(h, router, 8, False, logits=True)
    for t in (0, 17, 63):
        one = K.ext().route_fused(h[t:t + 1].contiguous(), router, 8, False, logits=True)
        assert torch.equal(one[7][0], full[7][t]) and torch.equal(one[0][0], full[0][t]) and torch.equal(one[1][0], full[1][t])
    rolled = K.ext().route_fused(torch.roll(h, 5, 0).contiguous(), router, 8, False, logits=True)
    assert torch.equal(torch.roll(full[7], 5, 0), rolled[7])


# ------------------------------------------------------------------------------ sort
@pytest.mark.parametrize("name", list(cases.SORT_CASES))
def test_sort_matches_the_reference_bit_for_bit(K, golden, name):
    E, k, N, seed = cases.SORT_CASES[name]
    idx, w = cases.sort_inputs(E, k, N, seed)
    a = K.ext().sort_by_expert(idx.to(DEV), w.to(DEV), E)
    b = K.ext().sort_by_expert(idx.to(DEV), w.to(DEV), E)
    assert all(torch.equal(x, y) for x, y in zip(a, b))  # same result every run
    for got, key in zip(a, ("counts", "offsets", "token", "wsorted", "pos_of")):
        assert torch.equal(got.cpu(), T(golden[f"sort/{name}/{key}"])), key


@pytest.mark.parametrize("N,E,k", [(1025, 64, 8), (1100, 64, 8), (8192, 64, 8), (20000, 128, 4), (70001, 16, 2)])
def test_sort_with_several_blocks(K, N, E, k):
    idx, w = cases.sort_inputs(E, k, N, N)
    a = K.ext().sort_by_expert(idx.to(DEV), w.to(DEV), E)
    want = mo.sort_by_expert(idx, w, E)
    for got, ref in zip(a, want):
        assert torch.equal(got.cpu(), ref)
    # a permutation: every choice has exactly one row
    assert torch.equal(a[4].cpu().long().sort().values, torch.arange(N * k))


def test_sort_bf16_weights(K):
    idx, w = cases.sort_inputs(64, 8, 333, 11)
    w = w.to(torch.bfloat16)
    a = K.ext().sort_by_expert(idx.to(DEV), w.to(DEV), 64)
    want = mo.sort_by_expert(idx, w, 64)
    for got, ref in zip(a, want):
        assert torch.equal(got.cpu(), ref)


@pytest.mark.parametrize("N", [40, 3000])
def test_an_expert_id_out_of_range_is_skipped_everywhere(K, N):
    """A choice whose expert id is outside [0, E) gets no row: the sort leaves it out of the
    counts, marks pos_of with -1 and sets status 6; the combine adds nothing for it. No kernel
    reads through the bad index."""
    E, k, H = 64, 8, 256
    idx, w = cases.sort_inputs(E, k, N, 21)
    bad = idx.clone()
    bad[3, 2], bad[N - 1, 0], bad[N // 2, 7] = 1 << 30, -5, E
    counts, offsets, token, wsorted, pos_of = K.ext().sort_by_expert(bad.to(DEV), w.to(DEV), E)
    assert K.ext().device_status() == 6
    flat = bad.flatten()
    valid = (flat >= 0) & (flat < E)
    assert int(counts.sum()) == int(valid.sum()) == N * k - 3 and int(offsets[-1]) == N * k - 3
    assert (pos_of.cpu()[~valid] == -1).all() and (pos_of.cpu()[valid] >= 0).all()
    assert torch.equal(counts.cpu().long(), torch.bincount(flat[valid].long(), minlength=E))
    y = torch.randn(N * k, H, generator=cases.gen(5)).half()
    got = K.ext().combine(y.to(DEV), pos_of, bad.to(DEV), N).cpu()
    rows = pos_of.cpu().view(N, k)
    for t in (3, N - 1, N // 2, 0):
        order = sorted((int(bad[t, j]), j) for j in range(k) if rows[t, j] >= 0)
        acc = torch.zeros(H)
        for _, j in order:
            acc += y[rows[t, j]].float()
        assert torch.equal(got[t], acc.half())
    assert K.ext().device_status() == 0


@pytest.mark.parametrize("N,E,k,dtype", [(1, 64, 8, torch.float16), (64, 64, 8, torch.float16), (300, 128, 8, torch.bfloat16),
                                         (1024, 64, 8, torch.float16), (77, 60, 4, torch.float16)])
def test_route_sort_in_one_launch_equals_the_two_calls(K, N, E, k, dtype):
    logits = cases.route_logits(E, N, dtype=dtype).to(DEV)
    for norm in (False, True):
        idx, w = K.ext().route(logits, k, norm)
        want = [idx, w] + K.ext().sort_by_expert(idx, w, E)
        for _ in range(2):  # several blocks route, the last one sorts; the ticket returns to zero
            got = K.ext().route_sort(logits, k, norm)
            for a, b in zip(got, want):
                assert torch.equal(a, b)
    with pytest.raises(RuntimeError):
        K.ext().route_sort(cases.route_logits(64, 1025).to(DEV), 8, False)  # more choices than one block sorts


# ------------------------------------------------------------------------------ combine
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("N,E,k,H", [(50, 16, 4, 24 * 8), (333, 64, 8, 256), (64, 64, 8, 2048), (1, 64, 8, 2048)])
def test_combine_adds_in_expert_order(K, dtype, N, E, k, H):
    idx, w = cases.sort_inputs(E, k, N, 9)
    counts, offsets, token, wsorted, pos_of = mo.sort_by_expert(idx, w, E)
    y = torch.randn(N * k, H, generator=cases.gen(5)).to(dtype)
    got = K.ext().combine(y.to(DEV), pos_of.to(DEV), idx.to(DEV), N)
    assert torch.equal(got.cpu(), mo.combine_expert_order(y, pos_of, idx, N))


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("N,E,k,H", [(50, 16, 4, 24 * 8), (64, 64, 8, 2048), (1, 64, 8, 2048)])
def test_combine_with_a_residual_is_the_separate_addition(K, dtype, N, E, k, H):
    idx, w = cases.sort_inputs(E, k, N, 9)
    counts, offsets, token, wsorted, pos_of = mo.sort_by_expert(idx, w, E)
    y = torch.randn(N * k, H, generator=cases.gen(5)).to(dtype)
    x = (torch.randn(N, H, generator=cases.gen(6)) * 3).to(dtype)
    got = K.ext().combine(y.to(DEV), pos_of.to(DEV), idx.to(DEV), N, x.to(DEV))
    assert torch.equal(got.cpu(), x + mo.combine_expert_order(y, pos_of, idx, N))  # two roundings, as the caller's add
    with pytest.raises(RuntimeError):
        K.ext().combine(y.to(DEV), pos_of.to(DEV), idx.to(DEV), N, x[:, :8].contiguous().to(DEV))


@pytest.mark.parametrize("mode", ["gemv", "gemm"])
def test_layer_with_a_residual_is_the_layer_plus_the_residual(K, mode):
    spec = cases.LAYER_CASES["n64"]
    h, router, gu, dn = (t.to(DEV) for t in cases.layer_inputs(**spec))
    x = torch.randn(h.shape, generator=cases.gen(3)).to(h.dtype).to(DEV)
    k = spec["k"]
    assert torch.equal(K.moe_layer(h, router, gu, dn, k, False, mode, residual=x),
                       x + K.moe_layer(h, router, gu, dn, k, False, mode))


# ------------------------------------------------------------------------------ layer
def layer_errors(K, h, router, gu, dn, mode, ridx, rw, want, loop16):
    got = K.experts(h.to(DEV), ridx.int().to(DEV), rw.to(DEV), gu.to(DEV), dn.to(DEV), mode).float().cpu()
    err = (got - want).abs().max().item()
    err16 = (loop16.float() - want).abs().max().item()
    rel = ((got - want).norm() / want.norm().clamp_min(1e-20)).item()
    return err, err16, rel


@pytest.mark.parametrize("name", [n for n in cases.LAYER_CASES if n != "tiny"])
@pytest.mark.parametrize("mode", ["gemv", "gemm"])
def test_layer_matches_the_stored_reference(K, golden, name, mode):
    spec = cases.LAYER_CASES[name]
    h, router, gu, dn = cases.layer_inputs(**spec)
    ridx = T(golden[f"layer/{name}/ridx"]).long()
    rw = T(golden[f"layer/{name}/rw"])
    want = T(golden[f"layer/{name}/want_fp32"])
    loop16 = T(golden[f"layer/{name}/loop16"])
    err, err16, rel = layer_errors(K, h, router, gu, dn, mode, ridx, rw, want, loop16)
    assert err <= max(2 * err16, 2e-3), (err, err16, rel)


@pytest.mark.parametrize("N", [1, 7, 64, 333, 2048])
@pytest.mark.parametrize("skew", [0.0, 2.0])
@pytest.mark.parametrize("mode", ["gemv", "gemm"])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_layer_matches_the_fp32_expert_loop(K, N, skew, mode, dtype):
    h, router, gu, dn = cases.layer_inputs(N, skew=skew, dtype=dtype)
    ridx, rw = mo.route_reference(h, router, 8, False)
    want = mo.experts_reference(h.float(), ridx, rw.float(), gu.float(), dn.float())
    loop16 = mo.experts_reference(h, ridx, rw, gu, dn)
    err, err16, rel = layer_errors(K, h, router, gu, dn, mode, ridx, rw, want, loop16)
    floor = 2e-3 if dtype == torch.float16 else 1.6e-2  # bf16 has 3 fewer mantissa bits
    assert err <= max(2 * err16, floor), (err, err16, rel)


@pytest.mark.parametrize("mode", ["gemv", "gemm"])
@pytest.mark.parametrize("N", [5, 150, 700])
def test_sizes_that_fill_no_tile(K, mode, N):
    """hidden 200 (three 64-wide k blocks and a tail of 8), expert width 72 (less than any tile's
    columns), 16 experts, top-4: every tile is ragged in k, in columns and in rows."""
    h, router, gu, dn = cases.layer_inputs(N, E=16, k=4, H=200, I=72, seed=3, skew=1.0)
    ridx, rw = mo.route_reference(h, router, 4, False)
    want = mo.experts_reference(h.float(), ridx, rw.float(), gu.float(), dn.float())
    loop16 = mo.experts_reference(h, ridx, rw, gu, dn)
    err, err16, rel = layer_errors(K, h, router, gu, dn, mode, ridx, rw, want, loop16)
    assert err <= max(2 * err16, 2e-3), (err, err16, rel)
    assert K.ext().device_status() == 0


def test_empty_experts_and_a_single_token(K):
    h, router, gu, dn = cases.layer_inputs(1)
    out = K.moe_layer(h.to(DEV), router.to(DEV), gu.to(DEV), dn.to(DEV), 8, False)
    ridx, rw = mo.route_kernel_rule(layer_logits(K, h.to(DEV), router.to(DEV)).cpu(), 8, False)
    ridx = ridx.long()
    want = mo.experts_reference(h.float(), ridx, rw.float(), gu.float(), dn.float())
    assert (out.float().cpu() - want).abs().max().item() < 2e-3
    out0 = K.moe_layer(h[:0].to(DEV), router.to(DEV), gu.to(DEV), dn.to(DEV), 8, False)
    assert out0.shape == (0, 256)


@pytest.mark.parametrize("mode", ["gemv", "gemm"])
def test_a_rows_bits_do_not_depend_on_its_group(K, mode):
    """The property expert parallelism rests on: the same (row, expert) computed inside
    different groupings (all rows at once; split into two ffn calls at an arbitrary point, as a
    local and a received segment would be) gives identical bits."""
    h, router, gu, dn = cases.layer_inputs(97, skew=2.0)
    ridx, rw = mo.route_reference(h, router, 8, False)
    counts, offsets, token, wsorted, pos_of = mo.sort_by_expert(ridx.int(), rw, 64)
    hd, gud, dnd = h.to(DEV), gu.to(DEV), dn.to(DEV)
    M = token.numel()
    full = K.ffn(hd, token.to(DEV), offsets.to(DEV), counts.to(DEV), wsorted.to(DEV), gud, dnd, M, mode)
    # split every expert's rows in two parts: part A gets the first third, part B the rest
    off = offsets.tolist()
    partA, partB = [], []
    for e in range(64):
        a, b = off[e], off[e + 1]
        cut = a + (b - a) // 3
        partA += list(range(a, cut))
        partB += list(range(cut, b))
    for part in (partA, partB):
        rows = torch.tensor(part, dtype=torch.long)
        e_of = torch.bucketize(rows, offsets[1:].long(), right=True)
        cnt = torch.bincount(e_of, minlength=64).int()
        offs = torch.zeros(65, dtype=torch.int32)
        offs[1:] = torch.cumsum(cnt, 0)
        y = K.ffn(hd, token[rows].contiguous().to(DEV), offs.to(DEV), cnt.to(DEV), wsorted[rows].contiguous().to(DEV),
                  gud, dnd, len(part), mode)
        assert torch.equal(y.cpu(), full.cpu()[rows])


@pytest.mark.parametrize("mode", ["gemv", "gemm"])
@pytest.mark.parametrize("N,skew", [(1, 0.0), (64, 0.0), (97, 2.0), (700, 2.0)])
def test_fused_ffn_equals_the_two_grouped_calls(K, mode, N, skew):
    """ffn() runs both projections in one launch; bit for bit the same as grouped_gemv /
    grouped_gemm called twice (the reference's structure), several times in a row (the kernel's
    per-expert counters must come back to zero)."""
    h, router, gu, dn = cases.layer_inputs(N, skew=skew)
    ridx, rw = mo.route_reference(h, router, 8, False)
    counts, offsets, token, wsorted, pos_of = mo.sort_by_expert(ridx.int(), rw, 64)
    hd, gud, dnd = h.to(DEV), gu.to(DEV), dn.to(DEV)
    tok, off, ws = token.to(DEV), offsets.to(DEV), wsorted.to(DEV)
    M = token.numel()
    E = K.ext()
    if mode == "gemv":
        act = E.grouped_gemv(hd, tok, gud, off, M, True, None)
        want = E.grouped_gemv(act, None, dnd, off, M, False, ws)
    else:
        act = E.grouped_gemm(hd, tok, gud, off, None, 0, M, True, None)
        want = E.grouped_gemm(act, None, dnd, off, None, 0, M, False, ws)
    for _ in range(3):
        got = K.ffn(hd, tok, off, counts.to(DEV), ws, gud, dnd, M, mode)
        assert torch.equal(got, want)
    if mode == "gemv":
        # ... and with the combine folded into the down projection's epilogue: the bits of combine()
        out = E.combine(want, pos_of.to(DEV), ridx.int().to(DEV), N)
        for _ in range(3):
            got = E.expert_ffn_combine(hd, tok, gud, dnd, off, ws, pos_of.to(DEV), 8)
            assert torch.equal(got, out)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("N,E,k,H,I", [(64, 64, 8, 2048, 1024), (5, 16, 4, 200, 72), (130, 8, 2, 256, 128), (1, 64, 8, 2048, 1024)])
def test_fused_combine_equals_the_combine_kernel(K, dtype, N, E, k, H, I):
    """expert_ffn_combine against expert_ffn + combine at the benchmark's shape and at sizes that
    fill no tile (hidden 200: a ragged last column block), with many rows per expert (E=8)."""
    h, router, gu, dn = cases.layer_inputs(N, E=E, k=k, H=H, I=I, seed=4, skew=1.0, dtype=dtype)
    ridx, rw = mo.route_reference(h, router, k, False)
    counts, offsets, token, wsorted, pos_of = (t.to(DEV) for t in mo.sort_by_expert(ridx.int(), rw, E))
    hd, gud, dnd = h.to(DEV), gu.to(DEV), dn.to(DEV)
    X = K.ext()
    y = X.expert_ffn(hd, token, gud, dnd, offsets, N * k, wsorted, 0)
    want = X.combine(y, pos_of, ridx.int().to(DEV), N)
    for _ in range(2):
        assert torch.equal(X.expert_ffn_combine(hd, token, gud, dnd, offsets, wsorted, pos_of, k), want)
    assert X.device_status() == 0


@pytest.mark.parametrize("N,skew,dtype", [(64, 0.0, torch.float16), (333, 2.0, torch.float16), (2048, 2.0, torch.float16),
                                          (3000, 1.0, torch.bfloat16)])
def test_compute_tiles_and_row_sources_agree_bit_for_bit(K, N, skew, dtype):
    """The compute shape has two tiles (one CTA; a CTA pair, sy_force_compute_tile) and two ways to
    fetch token rows (gathered through a_rows; contiguous rows by TMA). All four combinations
    run the same MMAs in the same k order: identical bits, separately and fused."""
    h, router, gu, dn = cases.layer_inputs(N, skew=skew, dtype=dtype)
    ridx, rw = mo.route_reference(h, router, 8, False)
    counts, offsets, token, wsorted, pos_of = mo.sort_by_expert(ridx.int(), rw, 64)
    hd, gud, dnd = h.to(DEV), gu.to(DEV), dn.to(DEV)
    tok, off, ws = token.to(DEV), offsets.to(DEV), wsorted.to(DEV)
    M = token.numel()
    E = K.ext()
    hs = hd[tok.long()].contiguous()
    want_act = want = None
    try:
        for tile in (1, 2):
            force_tile(K, tile)
            for x, rows in ((hd, tok), (hs, None)):
                act = E.grouped_gemm(x, rows, gud, off, None, 0, M, True, None)
                y = E.grouped_gemm(act, None, dnd, off, None, 0, M, False, ws)
                fused = E.expert_ffn(x, rows, gud, dnd, off, M, ws, 1)
                if want is None:
                    want_act, want = act, y
                assert torch.equal(act, want_act) and torch.equal(y, want) and torch.equal(fused, want)
    finally:
        force_tile(K, 0)
    assert E.device_status() == 0


# ------------------------------------------------------------------------------ OLMoE shapes
@pytest.fixture(scope="module")
def olmoe():
    from switchyard_b200 import synthetic
    router, gu, dn = synthetic.layer_weights("cpu", torch.float16, seed=0)
    return router, gu, dn


@pytest.mark.parametrize("tokens", [1, 8, 32, 64])
@pytest.mark.parametrize("mode", ["gemv", "gemm"])
def test_olmoe_decode_layer(K, olmoe, tokens, mode):
    """The benchmark's layer (hidden 2048, 64 experts of width 1024, top-8) at the decode
    sweep's token counts, against the float32 expert loop."""
    from switchyard_b200 import synthetic
    router, gu, dn = olmoe
    h = synthetic.hidden_states(tokens, "cpu", torch.float16, seed=1)
    rd, gud, dnd = router.to(DEV), gu.to(DEV), dn.to(DEV)
    out = K.moe_layer(h.to(DEV), rd, gud, dnd, 8, False, mode).cpu()
    logits = layer_logits(K, h.to(DEV), rd).cpu()
    idx, w = mo.route_kernel_rule(logits, 8, False)
    want = mo.experts_reference(h.float(), idx.long(), w.float(), gu.float(), dn.float())
    loop16 = mo.experts_reference(h, idx.long(), w, gu, dn)
    err = (out.float() - want).abs().max().item()
    err16 = (loop16.float() - want).abs().max().item()
    rel = ((out.float() - want).norm() / want.norm()).item()
    assert err <= max(2 * err16, 2e-3), (err, err16, rel)
    assert rel < 5e-3


# ------------------------------------------------------------------------------ transport
@pytest.mark.parametrize("tokens,dtype", [(1024, torch.bfloat16), (4096, torch.bfloat16), (8192, torch.bfloat16),
                                          (2048, torch.float16)])
def test_olmoe_prefill_layer_at_full_size(K, olmoe, tokens, dtype):
    """The prefill configuration at its real sizes (hidden 2048, 64 experts of width 1024, top-8,
    Zipf-skewed routing: the busiest expert gets about four times the mean), checked on a sample
    of tokens against the float32 expert loop. The tile is first the library's own choice (one
    CTA below 768 rows per expert on average, CTA pairs from there: 8192 tokens take pairs), then
    each tile forced: all three must give the same bits."""
    from switchyard_b200 import synthetic
    router, gu, dn = (t.to(dtype) for t in olmoe)
    h = synthetic.hidden_states(tokens, "cpu", dtype, seed=tokens)
    rd, gud, dnd, hd = router.to(DEV), gu.to(DEV), dn.to(DEV), h.to(DEV)
    logits = (torch.nn.functional.linear(hd, rd) + synthetic.zipf_bias().to(DEV).to(dtype)).contiguous()
    idx, w = K.ext().route(logits, 8, False)
    outs = [K.experts(hd, idx, w, gud, dnd, "gemm")]
    try:
        for tile in (1, 2):
            force_tile(K, tile)
            outs.append(K.experts(hd, idx, w, gud, dnd, "gemm"))
    finally:
        force_tile(K, 0)
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])
    assert K.ext().device_status() == 0
    counts = torch.bincount(idx.flatten().long().cpu(), minlength=64)
    assert counts.max().item() > 3 * counts.float().mean().item()  # the skew is there
    sample = torch.arange(0, tokens, tokens // 16)
    hs, ids, ws = h[sample], idx.cpu()[sample].long(), w.cpu()[sample]
    want = mo.experts_reference(hs.float(), ids, ws.float(), gu.float(), dn.float())
    loop16 = mo.experts_reference(hs, ids, ws, gu, dn)
    got = outs[0].cpu()[sample].float()
    err = (got - want).abs().max().item()
    err16 = (loop16.float() - want).abs().max().item()
    floor = 2e-3 if dtype == torch.float16 else 1.6e-2
    assert err <= max(2 * err16, floor), (err, err16)


def test_graphed_layer_replays_the_same_bits(K):
    """GraphedLayer captures moe_layer once per batch size; replays, from device or pinned host
    input, give moe_layer's bits for new inputs of that size."""
    _, router, gu, dn = cases.layer_inputs(8)
    rd, gud, dnd = router.to(DEV), gu.to(DEV), dn.to(DEV)
    layer = K.GraphedLayer(rd, gud, dnd, 8, False, "auto")
    for N in (5, 40, 5, 40, 200):
        for seed in (1, 2):
            h = torch.randn(N, rd.shape[1], generator=cases.gen(1000 * seed + N)).half()
            want = K.moe_layer(h.to(DEV), rd, gud, dnd, 8, False, "auto")
            assert torch.equal(layer(h.to(DEV)), want)
            out = torch.empty(N, rd.shape[1], dtype=torch.float16).pin_memory()
            layer(h.pin_memory(), out=out)
            torch.cuda.synchronize()
            assert torch.equal(out, want.cpu())
    assert len(layer.graphs) == 3
    # the same pair of pinned buffers again: the copies are inside the replayed graph
    hin = torch.empty(40, rd.shape[1], dtype=torch.float16).pin_memory()
    hout = torch.empty(40, rd.shape[1], dtype=torch.float16).pin_memory()
    for seed in (5, 6, 7):
        hin.copy_(torch.randn(40, rd.shape[1], generator=cases.gen(seed)).half())
        assert layer(hin, out=hout) is hout
        torch.cuda.synchronize()
        assert torch.equal(hout, K.moe_layer(hin.to(DEV), rd, gud, dnd, 8, False, "auto").cpu())
    assert (40, hin.data_ptr(), hout.data_ptr()) in layer.staged
    layer.check()  # no replayed kernel gave up on a wait


def test_a_wait_that_runs_out_ends_in_a_status_code(K):
    """The bounded-wait path, exercised without hanging anything: a one-block kernel waits for a
    flag that nothing sets, with the limit lowered to 2 ms. It returns by itself, the status word
    reads 5 (a flag never came), sy_device_status answers SY_ERR_DEVICE, check_device raises, and
    the next layer on the same stream runs and is correct."""
    X = K.ext()
    flags = torch.zeros(4, dtype=torch.int32, device=DEV)
    epoch = torch.zeros(1, dtype=torch.int32, device=DEV)
    stream = torch.cuda.current_stream().cuda_stream
    default = X.lib.sy_wait_limit_ns()
    assert default == 2_000_000_000
    try:
        X.set_wait_limit(0.002)
        assert X.lib.sy_wait_limit_ns() == 2_000_000
        assert X.lib.sy_ep_wait(flags.data_ptr(), 4, epoch.data_ptr(), 1, stream) == 0  # waits for flags >= 1
        assert X.device_status() == 5
        assert X.device_status() == 0  # reading clears it
        X.lib.sy_ep_wait(flags.data_ptr(), 4, epoch.data_ptr(), 1, stream)
        with pytest.raises(RuntimeError, match="device status 5"):
            X.check_device()
        flags.fill_(1)
        assert X.lib.sy_ep_wait(flags.data_ptr(), 4, epoch.data_ptr(), 1, stream) == 0  # the flags are there: no timeout
        assert X.device_status() == 0
    finally:
        X.lib.sy_set_wait_limit_ns(default)
    h, router, gu, dn = cases.layer_inputs(9)
    got = K.moe_layer(h.to(DEV), router.to(DEV), gu.to(DEV), dn.to(DEV), 8, False, "gemv")
    again = K.moe_layer(h.to(DEV), router.to(DEV), gu.to(DEV), dn.to(DEV), 8, False, "gemv")
    assert torch.equal(got, again) and X.device_status() == 0


def test_gather_rows_and_copy(K):
    src = torch.randn(100, 256, generator=cases.gen(1)).half().to(DEV)
    index = torch.randint(0, 100, (37,), generator=cases.gen(2)).int().to(DEV)
    dst = torch.empty(37, 256, dtype=torch.float16, device=DEV)
    K.ext().gather_rows(src, index, dst)
    assert torch.equal(dst, src[index.long()])
    other = torch.empty_like(dst)
    K.ext().copy_async(other, dst)
    assert torch.equal(other, dst)
    with pytest.raises(RuntimeError):
        K.ext().gather_rows(src, index, torch.empty(36, 256, dtype=torch.float16, device=DEV))
