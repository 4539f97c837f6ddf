"""The one-process-per-GPU expert-parallel layer (switchyard_b200.ep_dist) on real GPUs: every
rank's output is bit-identical to the single-GPU layer run with the same mode on that rank's
tokens. Ranks are child processes, rendezvous on 127.0.0.1. With one rank (every expert local,
every row "sent" to the rank's own mailbox) the whole transport runs on a single GPU; with more
ranks each needs its own GPU (kernels that wait for another rank's flag must not share a GPU
with the kernels that set it)."""

import socket

import pytest
import torch

import cases

pytestmark = pytest.mark.gpu

SMALL = dict(E=64, k=8, H=256, I=128, std=None)
OLMOE = dict(E=64, k=8, H=2048, I=1024, std=0.02)   # the benchmark's layer


def n_gpus():
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, sizes_per_layer, mode, dtype_name, shape, opts, out):
    try:
        _rank_main(rank, world, port, sizes_per_layer, mode, dtype_name, shape, opts, out)
    except BaseException:  # report instead of leaving the parent waiting for a result
        import traceback
        out.put((rank, False, traceback.format_exc()))


def _weights(shape, dtype, device):
    """The full layer, generated on the device from one seed (the same on every rank)."""
    E, H, I = shape["E"], shape["H"], shape["I"]
    g = torch.Generator(device=device).manual_seed(0)
    rs, gs, ds = (0.2, H ** -0.5, I ** -0.5) if shape["std"] is None else (shape["std"],) * 3
    router = (torch.randn(E, H, device=device, generator=g) * rs).to(dtype)
    gu = torch.empty(E, 2 * I, H, dtype=dtype, device=device)
    dn = torch.empty(E, H, I, dtype=dtype, device=device)
    for e in range(E):
        gu[e] = (torch.randn(2 * I, H, device=device, generator=g) * gs).to(dtype)
        dn[e] = (torch.randn(H, I, device=device, generator=g) * ds).to(dtype)
    return router, gu, dn


def _rank_main(rank, world, port, sizes_per_layer, mode, dtype_name, shape, opts, out):
    import torch.distributed as dist
    from switchyard_b200 import kernels, synthetic
    from switchyard_b200.ep_dist import DistributedExpertParallel
    dtype = getattr(torch, dtype_name)
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    try:
        E, k, H, I = shape["E"], shape["k"], shape["H"], shape["I"]
        router, gu, dn = _weights(shape, dtype, f"cuda:{rank}")
        per = E // world
        placement = opts.get("placement")
        mine = list(range(rank * per, (rank + 1) * per)) if placement is None else placement[rank * per:(rank + 1) * per]
        my_gu, my_dn = gu[mine].contiguous(), dn[mine].contiguous()
        order = list(range(E)) if placement is None else placement
        bias = synthetic.zipf_bias(E) if opts.get("zipf") else None
        ep = DistributedExpertParallel(E, k, False, H, I, max_tokens=max(max(s) for s in sizes_per_layer), dtype=dtype,
                                       mode=mode, logit_bias=bias, placement=placement)
        dbias = None if bias is None else bias.to("cuda").to(dtype)[order].contiguous()
        # the comparand: the single-GPU layer with all experts in placement order (a token's
        # expert outputs are then added in the same order on both sides)
        r1, g1, d1 = router[order].contiguous(), gu[order].contiguous(), dn[order].contiguous()
        ok, rows = True, 0
        for layer_no, sizes in enumerate(sizes_per_layer):
            h = torch.randn(sizes[rank], H, generator=cases.gen(100 * layer_no + rank)).to(dtype).cuda()
            x = torch.randn(h.shape, generator=cases.gen(7 + layer_no)).to(dtype).cuda() if opts.get("residual") else None
            got = ep.layer(h, router, my_gu, my_dn, residual=x)
            srt = kernels.route_and_sort(h, r1, k, False, dbias)
            want = kernels._sorted_experts(h, srt, g1, d1, k, ep.mode)
            if x is not None:
                want = x + want  # the caller's own 16-bit addition
            torch.cuda.synchronize()
            ok = ok and torch.equal(got, want)
            rows += sizes[rank] * k
        sent, kept = ep.row_counts()
        ok = ok and sent + kept == rows and (world > 1 or sent == 0)
        status = kernels.ext().device_status()
        ep.close()
        out.put((rank, ok, status))
    finally:
        dist.destroy_process_group()


def run(world, sizes_per_layer, mode, dtype_name="float16", shape=SMALL, **opts):
    assert world <= n_gpus(), f"{world} ranks need {world} GPUs"  # never start ranks that cannot get a device
    results = cases.spawn_ranks(_worker, world, (_free_port(), sizes_per_layer, mode, dtype_name, shape, opts))
    for rank, ok, status in results:
        assert status == 0, f"rank {rank}: {status}"  # a status code of a bounded wait, or a traceback
        assert ok, f"rank {rank}: output differs from the single-GPU layer"
    assert len(results) == world


# ---- one rank: the whole transport on a single GPU
@pytest.mark.parametrize("mode", ["gemv", "gemm"])
@pytest.mark.parametrize("dtype_name", ["float16", "bfloat16"])
def test_one_rank_equals_the_single_gpu_layer(mode, dtype_name):
    run(1, [(1,), (7,), (0,), (200,), (64,), (333,)], mode, dtype_name)


@pytest.mark.parametrize("dtype_name", ["float16", "bfloat16"])
def test_one_rank_adds_the_residual_in_the_combine(dtype_name):
    run(1, [(1,), (0,), (64,), (333,)], "gemv", dtype_name, residual=True)


def test_auto_mode_is_resolved_once_for_all_batch_sizes():
    # mode="auto" is fixed from max_tokens, which every rank shares, so a layer with few tokens is
    # computed in the same shape as one with many and equals the single-GPU layer of THAT mode
    run(1, [(3,), (200,), (1,)], "auto")


@pytest.mark.skipif(n_gpus() < 2, reason="needs two GPUs")
def test_two_ranks_in_auto_mode_with_unequal_batches():
    run(2, [(3, 200), (64, 1), (0, 130)], "auto")


def test_one_rank_at_the_benchmark_shape():
    run(1, [(64,), (256,), (8,)], "gemv", shape=OLMOE, zipf=True)
    # compute shape: 300 tokens share tiles across senders; from 192 rows per expert and sender the
    # senders' rows are tiled on their own (TMA rows), from 768 with CTA pairs
    run(1, [(300,), (2048,), (6200,)], "gemm", shape=OLMOE, zipf=True)


def test_one_rank_with_a_placement():
    g = cases.gen(9)
    run(1, [(50,), (3,)], "gemv", placement=torch.randperm(64, generator=g).tolist())


# ---- several ranks, one GPU each
@pytest.mark.skipif(n_gpus() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("mode", ["gemv", "gemm"])
def test_two_ranks_bit_identical(mode):
    run(2, [(1, 1), (7, 30), (0, 5), (200, 200), (64, 3), (33, 0)], mode)


@pytest.mark.skipif(n_gpus() < 2, reason="needs two GPUs")
def test_two_ranks_add_the_residual_in_the_combine():
    run(2, [(5, 9), (0, 3), (64, 64)], "gemv", residual=True)


@pytest.mark.skipif(n_gpus() < 2, reason="needs two GPUs")
def test_two_ranks_bf16():
    run(2, [(33, 12), (12, 33)], "gemv", "bfloat16")


@pytest.mark.skipif(n_gpus() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("mode", ["gemv", "gemm"])
def test_two_ranks_at_the_benchmark_shape(mode):
    """256 tokens per GPU at OLMoE's sizes with the Zipf-skewed routing (configs[2]); in the compute
    shape also 2048 tokens per GPU: thousands of rows per rank through the mailbox ranges."""
    run(2, [(256, 256), (64, 1)] + ([(2048, 2048)] if mode == "gemm" else []), mode, shape=OLMOE, zipf=True)


@pytest.mark.skipif(n_gpus() < 2, reason="needs two GPUs")
def test_two_ranks_with_a_placement():
    g = cases.gen(9)
    run(2, [(50, 20), (3, 0)], "gemv", placement=torch.randperm(64, generator=g).tolist())


@pytest.mark.skipif(n_gpus() < 4, reason="needs four GPUs")
@pytest.mark.parametrize("mode", ["gemv", "gemm"])
def test_four_ranks_bit_identical(mode):
    run(4, [(3, 50, 0, 17), (64, 64, 64, 64), (1, 0, 0, 1)], mode)


@pytest.mark.skipif(n_gpus() < 8, reason="needs eight GPUs")
def test_eight_ranks_bit_identical():
    run(8, [(3, 50, 0, 17, 1, 1, 64, 9), (256,) * 8], "gemv")
    run(8, [(256,) * 8], "gemv", shape=OLMOE, zipf=True)
