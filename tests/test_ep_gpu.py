"""The expert-parallel layer on GPUs: bit-identical to the one-GPU layer run with the same
kernel mode on each rank's tokens. Cases follow the reference's tests/test_ep_cuda.py: several
ranks sharing one GPU (streams, events, mailboxes and kernels without a second GPU), real
peer-to-peer when more GPUs are visible, and the ordering of the layer after its caller."""

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


def run(devices, sizes, mode, E=64, k=8, dtype=torch.float16):
    from switchyard_b200 import kernels
    from switchyard_b200.ep import CudaOps, ExpertParallel
    router, gu, dn = weights(E, dtype=dtype)
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
