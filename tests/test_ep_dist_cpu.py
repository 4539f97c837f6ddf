"""The one-process-per-rank expert-parallel protocol (switchyard_b200.ep_dist) in two, four
and eight real processes over gloo, without a GPU: the device side is replaced by the host-memory mock of
oracle/ep_dist_mock.py (windows in /dev/shm mapped by the peers, polling flag waits), so what
runs is the product's own host logic: window layout, pointer tables, argument order, device-side
epochs, mailbox reuse over several layers, a rank with zero tokens, a permuted expert placement, the residual handed to the combine.
Every rank's output must equal the one-process layer computed with the same row-at-a-time
arithmetic."""

import socket

import pytest
import torch

import cases


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, sizes_per_layer, placement, residual, out):
    import torch.distributed as dist
    from oracle import ep_dist_mock as mock
    from switchyard_b200.ep_dist import DistributedExpertParallel
    torch.set_num_threads(1)
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    backend = mock.MockBackend()
    try:
        E, k, H, I = 16, 4, 32, 16
        g = cases.gen(0)
        router = torch.randn(E, H, generator=g).half()
        gu = (torch.randn(E, 2 * I, H, generator=g) * 0.3).half()
        dn = (torch.randn(E, H, I, generator=g) * 0.3).half()
        per = E // world
        ep = DistributedExpertParallel(E, k, False, H, I, max_tokens=max(max(s) for s in sizes_per_layer),
                                       dtype=torch.float16, mode="gemv", backend=backend, placement=placement)
        # this rank's experts: a contiguous block, or its block of the placement
        mine = list(range(rank * per, (rank + 1) * per)) if placement is None else placement[rank * per:(rank + 1) * per]
        my_gu, my_dn = gu[mine].contiguous(), dn[mine].contiguous()
        # the one-process comparand computes the same function; with a placement a token's expert
        # outputs are added in placement order, so the comparand is given the permuted layer
        order = list(range(E)) if placement is None else placement
        ok, sent = True, 0
        for layer_no, sizes in enumerate(sizes_per_layer):
            h = torch.randn(sizes[rank], H, generator=cases.gen(100 * layer_no + rank)).half()
            x = torch.randn(h.shape, generator=cases.gen(7 + layer_no)).half() if residual else None
            got = ep.layer(h, router, my_gu, my_dn, residual=x)
            want = mock.single_layer(h, router[order], gu[order], dn[order], k, False)
            ok = ok and torch.equal(got, want if x is None else x + want)
        sent, kept = ep.row_counts()
        ok = ok and sent + kept == sum(s[rank] for s in sizes_per_layer) * k
        ep.close()
        out.put((rank, ok, ""))
    except BaseException:
        import traceback
        out.put((rank, False, traceback.format_exc()))
    finally:
        backend.cleanup()
        dist.destroy_process_group()


PLACEMENT = [5, 12, 0, 9, 3, 14, 7, 1, 10, 2, 15, 6, 11, 4, 13, 8]


@pytest.mark.parametrize("world,sizes,placement,residual", [(2, [(5, 9), (0, 3), (12, 12), (1, 0)], None, False),
                                                            (2, [(5, 9), (0, 3), (1, 0)], PLACEMENT, True),
                                                            (4, [(3, 7, 0, 2), (8, 8, 8, 8)], None, False),
                                                            (8, [(2, 0, 5, 1, 3, 4, 0, 6), (4,) * 8], None, False)])
def test_protocol_over_gloo_processes(world, sizes, placement, residual):
    results = cases.spawn_ranks(_rank_main, world, (_free_port(), sizes, placement, residual), limit=180)
    for rank, ok, err in results:
        assert not err, f"rank {rank}:\n{err}"
        assert ok, f"rank {rank}: output differs from the one-process layer"
    assert len(results) == world


def test_window_layout_is_aligned_and_disjoint():
    from switchyard_b200.ep_dist import window_layout
    lay = window_layout(8, 8, 2048, 2048, 2048, 2)
    names = ["arrive", "ret", "epoch", "counters", "stats", "meta", "w", "x", "y"]
    offs = [lay[n] for n in names] + [lay["total"]]
    assert offs == sorted(offs) and all(o % 256 == 0 for o in offs)
    assert lay["x"] - lay["w"] >= 8 * 2048 * 2 and lay["y"] - lay["x"] >= 8 * 2048 * 2048 * 2
    assert lay["total"] - lay["y"] >= 2048 * 2048 * 2
