"""Seeded inputs shared by the golden-vector generator, the CPU tests and the GPU tests.
Everything is generated on the CPU with torch.Generator so that the same bits are available on
every machine; `checksum` guards against a changed random stream."""

import numpy as np
import torch

# name -> (E, k, N): the (experts, top-k) pairs of the reference's routing test
# (tests/test_kernels_cuda.py:21-22) on 300 tokens.
ROUTE_CASES = {"e8k2": (8, 2, 300), "e64k8": (64, 8, 300), "e60k4": (60, 4, 300), "e128k8": (128, 8, 300)}

# name -> (E, k, N, seed)
SORT_CASES = {"n999": (64, 8, 999, 0), "n1": (64, 8, 1, 1), "n0": (64, 8, 0, 2), "e16k4": (16, 4, 77, 3),
              "n4100": (64, 8, 4100, 4), "skew": (64, 8, 513, 5)}

# name -> layer_inputs kwargs: shapes of the reference's layer test (tests/test_kernels_cuda.py:11-19)
LAYER_CASES = {
    "n1": dict(N=1, E=64, k=8, H=256, I=128, seed=0, skew=0.0),
    "n7": dict(N=7, E=64, k=8, H=256, I=128, seed=0, skew=0.0),
    "n64": dict(N=64, E=64, k=8, H=256, I=128, seed=0, skew=0.0),
    "n333": dict(N=333, E=64, k=8, H=256, I=128, seed=0, skew=0.0),
    "n64skew": dict(N=64, E=64, k=8, H=256, I=128, seed=0, skew=2.0),
    "tiny": dict(N=40, E=8, k=3, H=16, I=12, seed=0, skew=0.0, dtype=torch.float32),
}

EP_E, EP_K, EP_H, EP_I = 16, 4, 24, 12
# name -> (R, sizes): the reference's CPU protocol cases (tests/test_ep.py:26-28)
EP_CASES = {f"r{R}_{i}": (R, sizes[:R]) for R in (1, 2, 4)
            for i, sizes in enumerate([(5, 9, 1, 13), (0, 3, 7, 2), (40, 40, 40, 40)])}
CAPACITY_FACTORS = (0.5, 1.0, 1.25, 100.0)


def gen(seed):
    return torch.Generator().manual_seed(seed)


def checksum(t):
    """A float64 sum of a tensor's values: cheap fingerprint of regenerated inputs."""
    return np.float64(t.double().sum().item())


def to_np(t):
    """numpy view of a tensor; bfloat16 is stored as its int16 bit pattern."""
    return t.view(torch.int16).numpy() if t.dtype == torch.bfloat16 else t.numpy()


def route_logits(E, N, seed=0, dtype=torch.float16):
    """Router logits with the spread of N(0,1) hidden states times N(0,0.2) router rows at
    H=256 (std ~3), rounded to the 16-bit dtype."""
    g = gen(seed + 1000 * E)
    h = torch.randn(N, 256, generator=g)
    router = torch.randn(E, 256, generator=g) * 0.2
    return (h @ router.t()).to(dtype)


def sort_inputs(E, k, N, seed):
    """idx [N,k] int32 with k distinct experts per token (skewed towards low ids), w fp16."""
    g = gen(seed)
    scores = torch.rand(N, E, generator=g) + torch.linspace(0.6, 0, E)[None]
    idx = scores.topk(k, dim=1).indices.int()
    w = torch.rand(N, k, generator=g).half()
    return idx, w


def layer_inputs(N, E=64, k=8, H=256, I=128, seed=0, skew=0.0, dtype=torch.float16):
    g = gen(seed)
    h = torch.randn(N, H, generator=g).to(dtype)
    router = torch.randn(E, H, generator=g) * 0.2
    router[: max(1, E // 8)] += skew  # a few popular experts
    gu = (torch.randn(E, 2 * I, H, generator=g) * H ** -0.5).to(dtype)
    dn = (torch.randn(E, H, I, generator=g) * I ** -0.5).to(dtype)
    return h, router.to(dtype), gu, dn


def ep_inputs(R, sizes, seed=0):
    g = gen(seed)
    router = torch.randn(EP_E, EP_H, generator=g)
    gu = torch.randn(EP_E, 2 * EP_I, EP_H, generator=g) * 0.3
    dn = torch.randn(EP_E, EP_H, EP_I, generator=g) * 0.3
    hs = [torch.randn(n, EP_H, generator=g) for n in sizes]
    return router, gu, dn, hs


def capacity_inputs(seed=1):
    g = gen(seed)
    router = torch.randn(EP_E, EP_H, generator=g) * 2  # skewed enough to overflow some experts
    gu = torch.randn(EP_E, 2 * EP_I, EP_H, generator=g) * 0.3
    dn = torch.randn(EP_E, EP_H, EP_I, generator=g) * 0.3
    hs = [torch.randn(n, EP_H, generator=g) for n in (30, 17)]
    return router, gu, dn, hs


def spawn_ranks(worker, world, args, limit=300):
    """Runs worker(rank, world, *args, out) in `world` spawned processes and returns what they
    put on `out`: one (rank, ok, detail) each, detail a string (a traceback) when the rank failed.
    Never leaves a rank behind and never waits for one that cannot report: the children are
    daemons, a rank that reports a failure or ends silently stops the wait for the others (they
    may be waiting for it in a collective), and whatever is still alive afterwards is killed."""
    import queue
    import time
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    procs = [ctx.Process(target=worker, args=(r, world) + tuple(args) + (out,), daemon=True) for r in range(world)]
    for p in procs:
        p.start()
    results, failed = [], False
    deadline = time.monotonic() + limit
    try:
        while len(results) < world and not failed:
            try:
                results.append(out.get(timeout=1.0))
                failed = isinstance(results[-1][2], str) and bool(results[-1][2])
            except queue.Empty:
                gone = [p for p in procs if p.exitcode is not None]
                if len(gone) > len(results):  # a rank has ended without reporting (it could not even start)
                    try:
                        results.append(out.get(timeout=3.0))  # its report may still be on its way
                        failed = isinstance(results[-1][2], str) and bool(results[-1][2])
                    except queue.Empty:
                        results.append((-1, False, f"a rank ended without a report (exit code {gone[0].exitcode})"))
                        failed = True
                elif time.monotonic() > deadline:
                    results.append((-1, False, f"a rank did not report within {limit} s"))
                    failed = True
        for p in procs:
            p.join(timeout=1 if failed else 30)
    finally:
        for p in procs:  # exactly the processes started above
            if p.is_alive():
                p.kill()
                p.join(timeout=10)
    return sorted(results, key=lambda r: r[0])
