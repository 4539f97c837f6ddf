"""`bench.py --gpus N` for N > 1: the same decode sweep as at N = 1, expert-parallel.

One process per GPU (launched by torch.distributed.run), NCCL process group for set-up and for
the max-over-ranks of the timings only. Every rank holds E/N experts of each resident weight
set and T tokens of its own (T = 1, 8, 32, 64: weak scaling in tokens); a step is one
expert-parallel layer at each T through `DistributedExpertParallel.layer` (dispatch and return
by kernels writing into peer memory, no collective on the data path).

  value  aggregate expert-weight GB/s: over all ranks, experts that received at least one row
         (from any rank) x 3*H*I*2 bytes, divided by the slowest rank's device time;
  e2e    the same with each rank's hidden states copied from pinned host memory and its output
         copied back every pass."""

import json
import os
import statistics

import torch
import torch.distributed as dist

SWEEP = (1, 8, 32, 64)
H, I, E, TOPK = 2048, 1024, 64, 8
EXPERT_BYTES = 3 * H * I * 2
LAYERS = 8
METRIC, UNIT = "moe_layer_decode_expert_weight_GBps", "GB/s"


def rank_weights(device, dtype, seed, lo, hi, experts=None):
    """Experts [lo, hi) of the weight set `seed`, or the listed `experts` in that order (same
    values as synthetic.layer_weights gives for the whole set: the generator is advanced past the
    experts this rank does not hold)."""
    mine = list(range(lo, hi)) if experts is None else [int(e) for e in experts]
    slot = {e: i for i, e in enumerate(mine)}
    g = torch.Generator(device=device).manual_seed(seed)
    router = (torch.randn(E, H, device=device, generator=g) * 0.02).to(dtype)
    gate_up = torch.empty(len(mine), 2 * I, H, device=device, dtype=dtype)
    down = torch.empty(len(mine), H, I, device=device, dtype=dtype)
    for e in range(max(mine) + 1):
        a = torch.randn(2 * I, H, device=device, generator=g)
        b = torch.randn(H, I, device=device, generator=g)
        if e in slot:
            gate_up[slot[e]] = (a * 0.02).to(dtype)
            down[slot[e]] = (b * 0.02).to(dtype)
    return router, gate_up, down


def check_bit_identity(ep, kernels, layer, full, hs, rank, world, order=None):
    """Every rank's expert-parallel output against the single-GPU layer on the same tokens with
    the whole expert set (same mode): must be the same bits. With a placement the single-GPU
    layer gets its experts (and router rows) in placement order, so that a token's expert
    outputs are added in the same order on both sides. Collective; returns (ok on every rank,
    rows each rank sent / kept during the check)."""
    ok = True
    if order is not None:
        full = (full[0][order].contiguous(), full[1][order].contiguous(), full[2][order].contiguous())
    for h in hs:
        got = ep.layer(h, layer[0], layer[1], layer[2])
        want = kernels.moe_layer_with_bias(h, full[0], full[1], full[2], TOPK, False, ep.mode, ep.bias)
        torch.cuda.synchronize()
        ok = ok and bool(torch.equal(got, want))
    agreed = torch.tensor([1 if ok else 0], device=hs[0].device)
    dist.all_reduce(agreed, op=dist.ReduceOp.MIN)
    sent, kept = ep.row_counts()
    rows = torch.zeros(world, 2, dtype=torch.int64, device=hs[0].device)
    rows[rank, 0], rows[rank, 1] = sent, kept
    dist.all_reduce(rows)
    return bool(int(agreed)), rows.tolist()


def run(args):
    from . import kernels, synthetic
    from .ep_dist import DistributedExpertParallel
    import bench  # the repo-root script: clock sampler and peaks

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev)
    dtype, mode = torch.float16, "gemv"
    per = E // world
    layers = [rank_weights(dev, dtype, 100 + l, rank * per, (rank + 1) * per) for l in range(LAYERS)]
    hs = {T: synthetic.hidden_states(T, dev, dtype, seed=1000 * rank + T) for T in SWEEP}
    ep = DistributedExpertParallel(E, TOPK, False, H, I, max_tokens=max(SWEEP), dtype=dtype, mode=mode, device=dev)
    # before anything is timed: the expert-parallel layer must give the single-GPU layer's bits
    full = synthetic.layer_weights(dev, dtype, seed=100)
    identical, check_rows = check_bit_identity(ep, kernels, layers[0], full, [hs[T] for T in SWEEP], rank, world)
    del full
    torch.cuda.empty_cache()
    if not identical:
        if rank == 0:
            print(json.dumps({"error": "expert-parallel output differs from the single-GPU layer", "n_gpus": world}), flush=True)
        dist.destroy_process_group()
        raise SystemExit(1)

    # experts used per (T, layer) over ALL ranks' tokens: fixed by the seeds; for the byte count
    used = {}
    for T in SWEEP:
        for l, (router, _, _) in enumerate(layers):
            idx, _ = kernels.route(hs[T], router, TOPK, False)
            seen = torch.zeros(E, dtype=torch.int32, device=dev)
            seen[idx.flatten().long()] = 1
            dist.all_reduce(seen, op=dist.ReduceOp.MAX)
            used[(T, l)] = int(seen.sum())
    stream = torch.cuda.Stream(dev)
    pass_no = [0]

    # warm-up, then one CUDA graph per STEP (the four passes of a step back to back, a step starting
    # at weight set 0 and one at set 4) and, for the per-T breakdown, one graph per T holding that
    # T's pass over each of the eight weight sets; every rank builds and replays them in the same order
    keep = []
    with torch.cuda.stream(stream):
        for T in SWEEP:
            for router, gu, dn in layers:
                ep.layer(hs[T], router, gu, dn)
        stream.synchronize()
        dist.barrier()
        step_graphs, step_bytes = [], []
        for first in range(0, LAYERS, len(SWEEP)):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream):
                for i, T in enumerate(SWEEP):
                    keep.append(ep.layer(hs[T], *layers[(first + i) % LAYERS]))
            step_graphs.append(g)
            step_bytes.append(sum(used[(T, (first + i) % LAYERS)] for i, T in enumerate(SWEEP)) * EXPERT_BYTES)
        t_graphs = {}
        for T in SWEEP:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream):
                for l in range(LAYERS):
                    keep.append(ep.layer(hs[T], *layers[l]))
            t_graphs[T] = g
    torch.cuda.synchronize()
    dist.barrier()

    with torch.cuda.stream(stream):
        for i in range(args.warmup):
            step_graphs[i % len(step_graphs)].replay()
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()
        sampler = bench.ClockSampler(dev.index).__enter__() if rank == 0 else None
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record(stream)
        for i in range(args.steps):
            step_graphs[i % len(step_graphs)].replay()
        t1.record(stream)
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()
        per_T = []
        for T in SWEEP:
            for _ in range(2):
                t_graphs[T].replay()
            torch.cuda.synchronize()
            dist.barrier()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(stream)
            for _ in range(args.steps):
                t_graphs[T].replay()
            b.record(stream)
            torch.cuda.synchronize()
            per_T.append(a.elapsed_time(b))
            dist.barrier()
        clocks = sampler.stop() if sampler else None
    times = torch.tensor([t0.elapsed_time(t1)] + per_T, dtype=torch.float64, device=dev)
    dist.all_reduce(times, op=dist.ReduceOp.MAX)
    total_ms = float(times[0])
    per_T_ms = {T: float(times[1 + i]) for i, T in enumerate(SWEEP)}
    per_T_bytes = {T: sum(used[(T, l)] for l in range(LAYERS)) * EXPERT_BYTES * args.steps for T in SWEEP}
    total_bytes = sum(step_bytes[i % len(step_graphs)] for i in range(args.steps))
    del step_graphs, t_graphs, keep

    # end to end with host buffers
    host_in = {T: hs[T].cpu().pin_memory() for T in SWEEP}
    host_out = {T: torch.empty(T, H, dtype=dtype).pin_memory() for T in SWEEP}
    dev_in = {T: torch.empty_like(hs[T]) for T in SWEEP}

    def e2e_step():
        nbytes = 0
        for T in SWEEP:
            l = pass_no[0] % LAYERS
            pass_no[0] += 1
            router, gu, dn = layers[l]
            dev_in[T].copy_(host_in[T], non_blocking=True)
            out = ep.layer(dev_in[T], router, gu, dn)
            host_out[T].copy_(out, non_blocking=True)
            nbytes += used[(T, l)] * EXPERT_BYTES
        torch.cuda.current_stream().synchronize()
        return nbytes

    with torch.cuda.stream(stream):
        for _ in range(args.warmup):
            e2e_step()
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        e2e_bytes = sum(e2e_step() for _ in range(args.steps))
        e1.record(stream)
        torch.cuda.synchronize()
        dist.barrier()
    e2e_t = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=dev)
    dist.all_reduce(e2e_t, op=dist.ReduceOp.MAX)
    status = torch.tensor([kernels.ext().device_status(dev)], device=dev)
    dist.all_reduce(status, op=dist.ReduceOp.MAX)
    assert int(status) == 0, "a kernel gave up on a bounded wait"
    ep.close()

    if rank == 0:
        peak, peak_src = bench.peaks()
        io_bytes = sum(T * H * 2 for T in SWEEP) * world
        value = total_bytes / (total_ms / 1e3) / 1e9
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": total_ms / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": bench.CONFIG,
            "arm": {"mode": mode, "parallelism": f"ep{world}: {per} experts per GPU, T tokens PER GPU (weak scaling in "
                                                 "tokens), attention data-parallel; dispatch and return by kernels "
                                                 "writing into peer memory, no collective on the data path",
                    "timing": "CUDA events on each rank's stream around K replays of CUDA graphs holding one step (the four "
                              "layer passes back to back), max over ranks; `sweep`: per T, replays of one graph holding "
                              "that T's pass over each of the eight weight sets"},
            "ep_bit_identical": identical,
            "ep_check": {"what": "every rank's layer output == kernels.moe_layer on its own tokens with all 64 experts, "
                                 "T=1,8,32,64, torch.equal, before timing",
                         "rows_sent_kept_per_rank": check_rows},
            "sweep": [{"tokens_per_gpu": T, "us_per_layer": per_T_ms[T] / (args.steps * LAYERS) * 1e3,
                       "expert_weight_GBps": per_T_bytes[T] / (per_T_ms[T] / 1e3) / 1e9,
                       "tokens_per_s": T * world * args.steps * LAYERS / (per_T_ms[T] / 1e3)} for T in SWEEP],
            "clocks": clocks,
            "e2e": {"value": e2e_bytes / (float(e2e_t) / 1e3) / 1e9, "unit": UNIT, "h2d_bytes_per_step": io_bytes,
                    "d2h_bytes_per_step": io_bytes, "ms_per_step": float(e2e_t) / args.steps,
                    "api": "switchyard_b200.ep_dist.DistributedExpertParallel.layer, host buffers pinned"},
            # this library's kernels per layer and rank: route_fused, dispatch, expert FFN, combine
            "gpu_launches": args.steps * 4 * len(SWEEP) * world,
            "roofline": {"bound": "hbm", "achieved": value / world, "peak": peak, "unit": "GB/s",
                         "frac": value / world / peak, "traffic": None, "peak_source": peak_src,
                         "kernel": "whole expert-parallel layer, per GPU (the weight-stream kernel is profiled at N=1)"},
        }
        print(json.dumps(line), flush=True)
    dist.destroy_process_group()


# ------------------------------------------------------------------------------------------
# The other benchmark configurations (the default bench line is the
# decode sweep above): config 3 = 256 tokens per GPU, fp16, Zipf-skewed routing;
# config 4 = prefill, 1024 / 4096 / 8192 tokens per GPU, bf16, same skew.
def run_config(args):
    from . import kernels, synthetic
    import bench

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    if args.config == "ep256":
        dtype, sizes, mode = torch.float16, (256,), kernels.auto_mode(256 * TOPK, E)
    else:
        dtype, sizes, mode = torch.bfloat16, (1024, 4096, 8192), "gemm"
    per = E // world
    n_sets = 3
    bias = synthetic.zipf_bias()
    # --placement balanced: measure the per-expert load of this configuration's routing on every
    # rank (largest batch, routing only), add it up over the ranks, and deal the experts out so
    # that every rank computes about the same number of rows (switchyard_b200.placement)
    place, balance = None, None
    if world > 1 and getattr(args, "placement", "contiguous") == "balanced":
        from . import placement as pl
        router0 = rank_weights(dev, dtype, 100, 0, 1)[0]
        hb = synthetic.hidden_states(sizes[-1], dev, dtype, seed=1000 * rank + sizes[-1])
        meter = pl.LoadMeter(E, dev)
        meter.add(kernels.route_and_sort(hb, router0, TOPK, False, bias.to(dev).to(dtype))[2])
        dist.all_reduce(meter.total)
        load = meter.read()
        place = pl.balanced(load, world)
        balance = {"rows_per_rank_contiguous": pl.rank_rows(load, pl.contiguous(E), world).tolist(),
                   "rows_per_rank_balanced": pl.rank_rows(load, place, world).tolist(),
                   "imbalance_contiguous": pl.imbalance(pl.rank_rows(load, pl.contiguous(E), world)),
                   "imbalance_balanced": pl.imbalance(pl.rank_rows(load, place, world))}
        del hb, meter
    mine = None if place is None else place[rank * per:(rank + 1) * per]
    layers = [rank_weights(dev, dtype, 100 + l, rank * per, (rank + 1) * per, mine) for l in range(n_sets)]
    out = []
    for T in sizes:
        h = synthetic.hidden_states(T, dev, dtype, seed=1000 * rank + T)
        if world > 1:
            from .ep_dist import DistributedExpertParallel
            m = kernels.auto_mode(T * world * TOPK, E) if getattr(args, "mode", "auto") == "auto" else args.mode
            ep = DistributedExpertParallel(E, TOPK, False, H, I, max_tokens=T, dtype=dtype, mode=m, device=dev,
                                           logit_bias=bias, placement=place)
            full = synthetic.layer_weights(dev, dtype, seed=100)
            identical, rows_rank = check_bit_identity(ep, kernels, layers[0], full, [h], rank, world, place)
            del full
            torch.cuda.empty_cache()
            if not identical:
                raise SystemExit(f"rank {rank}: expert-parallel output differs from the single-GPU layer at T={T}")
            run = lambda l: ep.layer(h, *layers[l])
            mode_used = m
        else:
            b = bias.to(dev).to(dtype)

            def run(l):
                router, gu, dn = layers[l]
                return kernels.moe_layer_with_bias(h, router, gu, dn, TOPK, False, mode, b)
            mode_used = mode
            identical, rows_rank = None, None
        stream = torch.cuda.Stream(dev)
        with torch.cuda.stream(stream):
            for i in range(max(args.warmup, 3)):
                run(i % n_sets)
            torch.cuda.synchronize()
            # one CUDA graph per weight set: the host's launch cost (some 100 us for the layer's
            # dozen launches and allocations) would otherwise bound the smaller batches
            graphs, keep = [], []
            for l in range(n_sets):
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=stream):
                    keep.append(run(l))
                graphs.append(g)
            for i in range(max(args.warmup, 3)):
                graphs[i % n_sets].replay()
            torch.cuda.synchronize()
            if world > 1:
                dist.barrier()
            t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0.record(stream)
            for i in range(args.steps):
                graphs[i % n_sets].replay()
            t1.record(stream)
            torch.cuda.synchronize()
            del graphs, keep
        ms = torch.tensor([t0.elapsed_time(t1) / args.steps], dtype=torch.float64, device=dev)
        # routing skew actually achieved (rank 0's tokens)
        idx, _ = kernels.ext().route((torch.nn.functional.linear(h, layers[0][0]) + bias.to(dev).to(dtype)).contiguous(),
                                     TOPK, False)
        skew = synthetic.busiest_over_mean(idx)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
            ep.close()
        ms = float(ms)
        rows = T * world * TOPK
        out.append({"tokens_per_gpu": T, "ms_per_layer": ms, "tokens_per_s": T * world / (ms / 1e3),
                    "tflops": rows * 12582912 / (ms / 1e3) / 1e12, "tflops_per_gpu": rows * 12582912 / (ms / 1e3) / 1e12 / world,
                    "mode": mode_used, "busiest_over_mean": skew, "ep_bit_identical": identical,
                    "rows_sent_kept_per_rank": rows_rank})
    if rank == 0:
        print(json.dumps({"config": args.config, "n_gpus": world, "dtype": str(dtype).replace("torch.", ""),
                          "placement": getattr(args, "placement", "contiguous"), "balance": balance,
                          "steps": args.steps, "timing": "CUDA events around CUDA-graph replays of the whole layer, max over ranks",
                          "results": out, "device_status": kernels.ext().device_status(dev)}), flush=True)
    if world > 1:
        dist.destroy_process_group()


# ------------------------------------------------------------------------------------------
# configs[2] through the reference-shaped host: ONE process, a thread and a stream per GPU
# (`ep.ExpertParallel.layer_threaded`), 256 tokens per GPU, fp16, Zipf routing. Launches are eager
# (a layer driven by several host threads is not captured in one graph), so the figure includes
# the host's launch cost; `bench.py --config ep256` under torchrun is the one-process-per-GPU
# form of the same layer, replayed from graphs.
def run_threads(args):
    import time
    from . import kernels, synthetic
    from .ep import CudaOps, ExpertParallel

    n = args.gpus
    if torch.cuda.device_count() < n:
        raise SystemExit(f"--host threads needs {n} visible GPUs in this process")
    devices = [torch.device("cuda", i) for i in range(n)]
    dtype, T = torch.float16, 256
    per = E // n
    mode = kernels.auto_mode(T * n * TOPK, E) if args.mode == "auto" else args.mode
    bias = synthetic.zipf_bias()
    sets = 3
    weights = [[rank_weights(d, dtype, 100 + l, r * per, (r + 1) * per) for r, d in enumerate(devices)] for l in range(sets)]
    hs = [synthetic.hidden_states(T, d, dtype, seed=1000 * r + T) for r, d in enumerate(devices)]
    ep = ExpertParallel(devices, E, TOPK, False, ops=CudaOps(mode, logit_bias=bias))
    ep.reserve(T)

    def layer(l):
        w = weights[l % sets]
        return ep.layer_threaded(hs, [x[0] for x in w], [x[1] for x in w], [x[2] for x in w])

    # bit-identity against the single-GPU layer on rank 0's tokens
    full = synthetic.layer_weights(devices[0], dtype, seed=100)
    want = kernels.moe_layer_with_bias(hs[0], full[0], full[1], full[2], TOPK, False, mode, bias.to(devices[0]).to(dtype))
    identical = bool(torch.equal(layer(0)[0], want))
    del full
    for i in range(max(args.warmup, 3)):
        layer(i)
    for d in devices:
        torch.cuda.synchronize(d)
    t0 = time.perf_counter()
    for i in range(args.steps):
        layer(i)
    for d in devices:
        torch.cuda.synchronize(d)
    ms = (time.perf_counter() - t0) / args.steps * 1e3
    ep.check()
    rows = T * n * TOPK
    print(json.dumps({"config": "ep256", "host": "one process, a thread per GPU (ep.ExpertParallel.layer_threaded), eager launches",
                      "n_gpus": n, "dtype": "float16", "mode": mode, "steps": args.steps, "tokens_per_gpu": T,
                      "ms_per_layer": ms, "tokens_per_s": T * n / (ms / 1e3), "tflops_per_gpu": rows * 12582912 / (ms / 1e3) / 1e12 / n,
                      "timing": "host wall clock around K layers, all GPUs synchronised before and after",
                      "ep_bit_identical_rank0": identical, "stats": ep.stats}), flush=True)


# ------------------------------------------------------------------------------------------
# config 5: the full random-init OLMoE-1B-7B architecture, fp16: 128-token prompts of uniform
# random ids, 32 greedy decode tokens, `batch` requests dealt round-robin to the ranks
# (attention data-parallel, experts expert-parallel). tok/s = batch * new / wall(generate),
# prefill included, as the reference's bench/serve.py:81-85 computes it; decode-only tok/s too.
def run_model(args):
    import time
    from . import kernels, olmoe

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    c = olmoe.Config()
    per = c.experts // world
    dtype, new, plen = torch.float16, 32, 128
    w = olmoe.random_weights(c, dev, dtype, seed=0, experts=range(rank * per, (rank + 1) * per))
    results = []
    for batch in (8, 64):
        if batch % world:
            continue
        mine = batch // world
        g = torch.Generator().manual_seed(7)
        prompts = [torch.randint(0, c.vocab, (plen,), generator=g).tolist() for _ in range(batch)][rank::world]
        if world > 1:
            from .ep_dist import DistributedExpertParallel
            ep = DistributedExpertParallel(c.experts, c.top_k, c.norm_topk_prob, c.hidden, c.intermediate,
                                           max_tokens=mine * plen, dtype=dtype, mode="auto", device=dev)
            moe = lambda i, h, x: ep.layer(h, w["layers"][i]["router"], w["layers"][i]["gate_up"],
                                           w["layers"][i]["down"], residual=x)
        else:
            moe = lambda i, h, x: kernels.moe_layer(h, w["layers"][i]["router"], w["layers"][i]["gate_up"],
                                                    w["layers"][i]["down"], c.top_k, c.norm_topk_prob, residual=x)
        dec = olmoe.Decoder(c, w, moe, moe_adds_residual=True)  # the residual add rides in the combine launch
        session = olmoe.Session(dec, mine, plen + new)
        dec.generate(prompts, 4, graph=True, session=session)  # warm-up: libraries, allocator, graph capture
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        marks = []
        t0 = time.perf_counter()
        out = dec.generate(prompts, new, graph=True, marks=marks, session=session)
        torch.cuda.synchronize()
        t1 = time.perf_counter()
        times = torch.tensor([t1 - t0, marks[1][1] - marks[0][1]], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(times, op=dist.ReduceOp.MAX)
            ep.close()
        wall, decode = float(times[0]), float(times[1])
        results.append({"batch": batch, "requests_per_gpu": mine, "wall_s": wall, "tok_per_s": batch * new / wall,
                        "decode_tok_per_s": batch * (new - 1) / decode, "ms_per_decode_step": decode / (new - 1) * 1e3,
                        "first_tokens": out[0][:4]})
    if rank == 0:
        print(json.dumps({"config": "model", "model": "OLMoE-1B-7B architecture, random init, fp16", "n_gpus": world,
                          "prompt_tokens": plen, "new_tokens": new, "parallelism": f"dp{world} attention, ep{world} experts",
                          "decode": "one CUDA graph per decode step (all layers)", "results": results,
                          "device_status": kernels.ext().device_status(dev)}), flush=True)
    if world > 1:
        dist.destroy_process_group()
