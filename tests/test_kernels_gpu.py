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


@pytest.mark.parametrize("N,E,k,dtype", [(1, 64, 8, torch.float16), (64, 64, 8, torch.float16), (300, 128, 8, torch.bfloat16),
                                         (1024, 64, 8, torch.float16), (77, 60, 4, torch.float16)])
def test_route_sort_in_one_launch_equals_the_two_calls(K, N, E, k, dtype):
    logits = cases.route_logits(E, N, dtype=dtype).to(DEV)
    for norm in (False, True):
        idx, w = K.ext().route(logits, k, norm)
        want = [idx, w] + K.ext().sort_by_expert(idx, w, E)
        got = K.ext().route_sort(logits, k, norm)
        for a, b in zip(got, want):
            assert torch.equal(a, b)
    with pytest.raises(RuntimeError):
        K.ext().route_sort(cases.route_logits(64, 1025).to(DEV), 8, False)  # more than one block sorts


# ------------------------------------------------------------------------------ combine
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("N,E,k,H", [(50, 16, 4, 24 * 8), (333, 64, 8, 256), (64, 64, 8, 2048), (1, 64, 8, 2048)])
def test_combine_adds_in_expert_order(K, dtype, N, E, k, H):
    idx, w = cases.sort_inputs(E, k, N, 9)
    counts, offsets, token, wsorted, pos_of = mo.sort_by_expert(idx, w, E)
    y = torch.randn(N * k, H, generator=cases.gen(5)).to(dtype)
    got = K.ext().combine(y.to(DEV), pos_of.to(DEV), idx.to(DEV), N)
    assert torch.equal(got.cpu(), mo.combine_expert_order(y, pos_of, idx, N))


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
    ridx, rw = mo.route_reference(h, router, 8, False)
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


@pytest.mark.parametrize("N,skew,dtype", [(64, 0.0, torch.float16), (333, 2.0, torch.float16), (2048, 2.0, torch.float16),
                                          (3000, 1.0, torch.bfloat16)])
def test_compute_tiles_and_row_sources_agree_bit_for_bit(K, monkeypatch, N, skew, dtype):
    """The compute shape has two tiles (one CTA; a CTA pair, SY_GEMM_TILE=pair) and two ways to
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
    for tile in ("single", "pair"):
        monkeypatch.setenv("SY_GEMM_TILE", tile)
        for x, rows in ((hd, tok), (hs, None)):
            act = E.grouped_gemm(x, rows, gud, off, None, 0, M, True, None)
            y = E.grouped_gemm(act, None, dnd, off, None, 0, M, False, ws)
            fused = E.expert_ffn(x, rows, gud, dnd, off, M, ws, 1)
            if want is None:
                want_act, want = act, y
            assert torch.equal(act, want_act) and torch.equal(y, want) and torch.equal(fused, want)
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
    logits = torch.nn.functional.linear(h.to(DEV), rd).cpu()
    idx, w = mo.route_kernel_rule(logits, 8, False)
    want = mo.experts_reference(h.float(), idx.long(), w.float(), gu.float(), dn.float())
    loop16 = mo.experts_reference(h, idx.long(), w, gu, dn)
    err = (out.float() - want).abs().max().item()
    err16 = (loop16.float() - want).abs().max().item()
    rel = ((out.float() - want).norm() / want.norm()).item()
    assert err <= max(2 * err16, 2e-3), (err, err16, rel)
    assert rel < 5e-3


# ------------------------------------------------------------------------------ transport
@pytest.mark.parametrize("tokens,dtype", [(4096, torch.bfloat16), (2048, torch.float16)])
def test_olmoe_prefill_layer_at_full_size(K, olmoe, tokens, dtype):
    """The prefill configuration at its real size (hidden 2048, 64 experts of width 1024, top-8,
    Zipf-skewed routing: the busiest expert gets about four times the mean), checked on a sample
    of tokens against the float32 expert loop; both compute tiles must give the same bits."""
    import os
    from switchyard_b200 import synthetic
    router, gu, dn = (t.to(dtype) for t in olmoe)
    h = synthetic.hidden_states(tokens, "cpu", dtype, seed=tokens)
    rd, gud, dnd, hd = router.to(DEV), gu.to(DEV), dn.to(DEV), h.to(DEV)
    logits = (torch.nn.functional.linear(hd, rd) + synthetic.zipf_bias().to(DEV).to(dtype)).contiguous()
    idx, w = K.ext().route(logits, 8, False)
    outs = []
    for tile in ("single", "pair"):
        os.environ["SY_GEMM_TILE"] = tile
        try:
            outs.append(K.experts(hd, idx, w, gud, dnd, "gemm"))
        finally:
            os.environ.pop("SY_GEMM_TILE", None)
    assert torch.equal(outs[0], outs[1])
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
