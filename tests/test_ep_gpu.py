"""The expert-parallel layer on GPUs: bit-identical to the one-GPU layer run with the same
kernel mode on each rank's tokens. Cases follow the reference's tests/test_ep_cuda.py: several
ranks sharing one GPU (the window engine ordered by stream events: the same dispatch, expert and
combine kernels without a second GPU), real peer-to-peer ordered by device-side flags when more
GPUs are visible, and the ordering of the layer after its caller."""

import pytest
import torch

import cases

pytestmark = pytest.mark.gpu


def n_gpus():
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


def weights(E=64, H=256, I=128, seed=0, dtype=torch.float16):
    g = cases.gen(seed)
    router = (torch.randn(E, H, generator=g) * 0.2).to(dtype)
    gu = (torch.randn(E, 2 * I, H, generator=g) * H ** -0.5).to(dtype)
    dn = (torch.randn(E, H, I, generator=g) * I ** -0.5).to(dtype)
    return router.cuda(0), gu.cuda(0), dn.cuda(0)


def run(devices, sizes, mode, E=64, k=8, dtype=torch.float16, H=256, I=128):
    from switchyard_b200 import kernels
    from switchyard_b200.ep import CudaOps, ExpertParallel
    router, gu, dn = weights(E, H, I, dtype=dtype)
    R, per = len(devices), E // len(devices)
    g = cases.gen(1)
    hs0 = [torch.randn(n, router.shape[1], generator=g).to(dtype).cuda(0) for n in sizes]
    hs = [h.to(d) for h, d in zip(hs0, devices)]
    ep = ExpertParallel(devices, E, k, False, ops=CudaOps(mode))
    args = ([router.to(d) for d in devices], [gu[r * per:(r + 1) * per].to(devices[r]) for r in range(R)],
            [dn[r * per:(r + 1) * per].to(devices[r]) for r in range(R)])
    outs = ep.layer(hs, *args)
    threaded = ep.layer_threaded(hs, *args)
    again = ep.layer(hs, *args)  # mailboxes reused
    for d in devices:
        torch.cuda.synchronize(d)
    for h, o, t, a in zip(hs0, outs, threaded, again):
        want = kernels.moe_layer(h, router, gu, dn, k, False, mode)
        assert torch.equal(o.to("cuda:0"), want)
        assert torch.equal(t.to("cuda:0"), want)
        assert torch.equal(a.to("cuda:0"), want)
    assert kernels.ext().device_status("cuda:0") == 0
    ep.check()
    assert ep.windows and ep.host_ordered == (len(set(str(d) for d in devices)) < len(devices))
    stats = ep.stats  # counted on the device, read here
    assert stats["dispatched_rows"] + stats["local_rows"] == 3 * sum(sizes) * k
    if R == 1:
        assert stats["dispatched_rows"] == 0
    return ep


@pytest.mark.parametrize("mode", ["gemv", "gemm"])
@pytest.mark.parametrize("sizes", [(1, 1), (7, 30), (0, 5), (200, 200)])
def test_two_ranks_on_one_gpu(mode, sizes):
    run(["cuda:0", "cuda:0"], sizes, mode)


@pytest.mark.parametrize("mode", ["gemv", "gemm"])
def test_four_and_eight_ranks_on_one_gpu(mode):
    run(["cuda:0"] * 4, (3, 50, 0, 17), mode)
    run(["cuda:0"] * 8, (3, 50, 0, 17, 1, 1, 64, 9), mode)


def test_bf16_ranks_on_one_gpu():
    run(["cuda:0", "cuda:0"], (33, 12), "gemv", dtype=torch.bfloat16)


def test_one_rank_and_growing_batches():
    run(["cuda:0"], (40,), "gemv")
    from switchyard_b200.ep import CudaOps, ExpertParallel
    ep = ExpertParallel(["cuda:0", "cuda:0"], 64, 8, False, ops=CudaOps("gemv"))
    ep.max_tokens = 8   # small windows: layer() must grow them; layer_rank() cannot and says so
    router, gu, dn = weights(64)
    args = ([router, router], [gu[:32].contiguous(), gu[32:].contiguous()], [dn[:32].contiguous(), dn[32:].contiguous()])
    from switchyard_b200 import kernels
    for n in (4, 20, 100, 7):
        h = torch.randn(n, 256, generator=cases.gen(n)).half().cuda(0)
        outs = ep.layer([h, h[: n // 2]], *args)
        assert torch.equal(outs[0], kernels.moe_layer(h, router, gu, dn, 8, False, "gemv"))
    assert ep.max_tokens == 128
    big = torch.randn(200, 256, generator=cases.gen(1)).half().cuda(0)
    with pytest.raises(RuntimeError, match="reserve"):
        ep.phase_send(ep.new_state(), 0, big, router)
    ep.reserve(200)
    outs = ep.layer([big, big[:3]], *args)
    assert torch.equal(outs[0], kernels.moe_layer(big, router, gu, dn, 8, False, "gemv"))


@pytest.mark.parametrize("mode", ["gemv", "gemm"])
def test_two_ranks_at_the_benchmark_shape(mode):
    """OLMoE's layer sizes (hidden 2048, width 1024), 256 tokens per rank; in the compute shape
    2048 per rank as well."""
    sizes = (256, 256) if mode == "gemv" else (2048, 300)
    devices = ["cuda:0", "cuda:1"] if n_gpus() > 1 else ["cuda:0", "cuda:0"]
    run(devices, sizes, mode, H=2048, I=1024)


def test_capacity_factor_and_trace_on_the_gpu():
    """Rows past an expert's capacity get weight 0 in token order; the counts come from the
    device when stats is read. Against the layer computed with those weights zeroed by hand."""
    import math
    from switchyard_b200 import kernels
    from switchyard_b200.ep import CudaOps, ExpertParallel
    router, gu, dn = weights(64)
    router[:4] += 0.5  # a few popular experts, so that the limit bites
    ep = ExpertParallel(["cuda:0", "cuda:0"], 64, 8, False, ops=CudaOps("gemv"))
    ep.capacity_factor, ep.trace = 1.0, []
    hs = [torch.randn(n, 256, generator=cases.gen(n)).half().cuda(0) for n in (60, 33)]
    outs = ep.layer(hs, [router, router], [gu[:32].contiguous(), gu[32:].contiguous()],
                    [dn[:32].contiguous(), dn[32:].contiguous()])
    dropped = 0
    for h, o in zip(hs, outs):
        idx, w = kernels.route_and_sort(h, router, 8, False)[:2]  # the routing the ranks use for this batch size
        cap = math.ceil(1.0 * idx.numel() / 64)
        w, seen = w.clone().cpu(), [0] * 64
        for t in range(idx.shape[0]):
            for s in range(8):
                e = int(idx[t, s])
                if seen[e] >= cap:
                    w[t, s] = 0
                    dropped += 1
                seen[e] += 1
        assert torch.equal(o, kernels.experts(h, idx, w.cuda(0), gu, dn, "gemv"))
    assert dropped > 0 and ep.stats["dropped_rows"] == dropped and ep.stats["routed_rows"] == 93 * 8
    assert len(ep.trace) == 2 and all(int(c.sum()) == n * 8 for (_, c), n in zip(ep.trace, (60, 33)))


@pytest.mark.skipif(n_gpus() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("mode", ["gemv", "gemm"])
@pytest.mark.parametrize("sizes", [(1, 1), (7, 30), (0, 5), (200, 200), (1000, 3)])
def test_two_gpus_peer_to_peer(mode, sizes):
    ep = run(["cuda:0", "cuda:1"], sizes, mode)
    assert ep.peer
    if sum(sizes) > 2:
        assert ep.stats["dispatched_rows"] > 0


@pytest.mark.skipif(n_gpus() < 4, reason="needs four GPUs")
def test_all_visible_gpus_peer_to_peer():
    n = 8 if n_gpus() >= 8 else 4
    ep = run([f"cuda:{i}" for i in range(n)], tuple(range(5, 5 + 11 * n, 11)), "gemv")
    assert ep.peer and ep.stats["dispatched_rows"] > 0


@pytest.mark.parametrize("threaded", [False, True])
def test_the_layer_waits_for_its_input(threaded):
    # h is written on the caller's stream after a long GPU sleep; a layer that does not order
    # its stream after the caller's reads the old contents (zeros).
    from switchyard_b200 import kernels
    from switchyard_b200.ep import CudaOps, ExpertParallel
    devices = ["cuda:0", "cuda:1"] if n_gpus() > 1 else ["cuda:0", "cuda:0"]
    router, gu, dn = weights(64)
    g = cases.gen(3)
    real = [torch.randn(16, router.shape[1], generator=g).half().cuda(0) for _ in devices]
    torch.cuda.synchronize()
    hs = [torch.zeros(16, router.shape[1], dtype=torch.half, device=d) for d in devices]
    ep = ExpertParallel(devices, 64, 8, False, ops=CudaOps("gemv"))
    args = ([router.to(d) for d in devices], [gu[r * 32:(r + 1) * 32].to(d) for r, d in enumerate(devices)],
            [dn[r * 32:(r + 1) * 32].to(d) for r, d in enumerate(devices)])
    for d in devices:
        torch.cuda.synchronize(d)
    for h, x, d in zip(hs, real, devices):
        with torch.cuda.device(d):
            torch.cuda._sleep(100_000_000)  # tens of milliseconds
            h.copy_(x)
    outs = ep.layer_threaded(hs, *args) if threaded else ep.layer(hs, *args)
    for d in devices:
        torch.cuda.synchronize(d)
    for x, o in zip(real, outs):
        assert torch.equal(o.to("cuda:0"), kernels.moe_layer(x, router, gu, dn, 8, False, "gemv"))
