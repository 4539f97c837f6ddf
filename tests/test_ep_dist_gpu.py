"""The one-process-per-GPU expert-parallel layer (switchyard_b200.ep_dist) on real GPUs: every
rank's output is bit-identical to the single-GPU layer run with the same mode on that rank's
tokens. Needs at least two GPUs (kernels that wait for another rank's flag must not share a GPU
with the kernels that set it); ranks are child processes, rendezvous on 127.0.0.1."""

import os
import socket

import pytest
import torch

import cases

pytestmark = pytest.mark.gpu


def n_gpus():
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, sizes_per_layer, mode, dtype_name, fused, out):
    try:
        _rank_main(rank, world, port, sizes_per_layer, mode, dtype_name, fused, out)
    except BaseException:  # report instead of leaving the parent waiting for a result
        import traceback
        out.put((rank, False, traceback.format_exc()))


def _rank_main(rank, world, port, sizes_per_layer, mode, dtype_name, fused, out):
    import torch.distributed as dist
    from switchyard_b200 import kernels
    from switchyard_b200.ep_dist import DistributedExpertParallel
    dtype = getattr(torch, dtype_name)
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    try:
        E, k, H, I = 64, 8, 256, 128
        g = cases.gen(0)
        router = (torch.randn(E, H, generator=g) * 0.2).to(dtype).cuda()
        gu = (torch.randn(E, 2 * I, H, generator=g) * H ** -0.5).to(dtype).cuda()
        dn = (torch.randn(E, H, I, generator=g) * I ** -0.5).to(dtype).cuda()
        per = E // world
        my_gu, my_dn = gu[rank * per:(rank + 1) * per].contiguous(), dn[rank * per:(rank + 1) * per].contiguous()
        ep = DistributedExpertParallel(E, k, False, H, I, max_tokens=max(max(s) for s in sizes_per_layer), dtype=dtype,
                                       mode=mode, fused_transport=fused)
        ok = True
        for layer_no, sizes in enumerate(sizes_per_layer):
            hs = [torch.randn(n, H, generator=cases.gen(100 * layer_no + r)).to(dtype) for r, n in enumerate(sizes)]
            h = hs[rank].cuda()
            got = ep.layer(h, router, my_gu, my_dn)
            want = kernels.moe_layer(h, router, gu, dn, k, False, mode)
            torch.cuda.synchronize()
            ok = ok and torch.equal(got, want)
        status = kernels.ext().device_status()
        ep.close()
        out.put((rank, ok, status))
    finally:
        dist.destroy_process_group()


def run(world, sizes_per_layer, mode, dtype_name="float16", fused=True):
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, sizes_per_layer, mode, dtype_name, fused, out))
             for r in range(world)]
    for p in procs:
        p.start()
    results = []
    for _ in procs:
        results.append(out.get(timeout=120))
    for p in procs:
        p.join(timeout=30)
    for rank, ok, status in sorted(results, key=lambda r: r[0]):
        assert status == 0, f"rank {rank}: {status}"  # a status code of a bounded wait, or a traceback
        assert ok, f"rank {rank}: output differs from the single-GPU layer"


@pytest.mark.skipif(n_gpus() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("mode", ["gemv", "gemm"])
def test_two_ranks_bit_identical(mode):
    run(2, [(1, 1), (7, 30), (0, 5), (200, 200), (64, 3), (33, 0)], mode)


@pytest.mark.skipif(n_gpus() < 2, reason="needs two GPUs")
def test_two_ranks_bf16():
    run(2, [(33, 12), (12, 33)], "gemv", "bfloat16")


@pytest.mark.skipif(n_gpus() < 2, reason="needs two GPUs")
def test_two_ranks_with_every_transport_step_as_its_own_launch():
    run(2, [(7, 30), (0, 5), (64, 3)], "gemv", fused=False)


@pytest.mark.skipif(n_gpus() < 4, reason="needs four GPUs")
@pytest.mark.parametrize("mode", ["gemv", "gemm"])
def test_four_ranks_bit_identical(mode):
    run(4, [(3, 50, 0, 17), (64, 64, 64, 64), (1, 0, 0, 1)], mode)


@pytest.mark.skipif(n_gpus() < 8, reason="needs eight GPUs")
def test_eight_ranks_bit_identical():
    run(8, [(3, 50, 0, 17, 1, 1, 64, 9), (256,) * 8], "gemv")
