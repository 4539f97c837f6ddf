"""Benchmark of the MoE layer hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload at N=1 (the decode sweep the headline metric is quoted on): one OLMoE-1B-7B MoE layer
(hidden 2048, 64 experts of width 1024, top-8, no renormalisation) in fp16 on the
weight-streaming path, at T = 1, 8, 32 and 64 tokens. A step is one pass of the layer at each
T. Every pass runs on a different layer's weights (LAYERS weight sets are resident and used
in rotation), so a pass never finds its weights in L2.

  value   expert-weight GB/s: bytes of the expert weights the passes had to read (experts that
          received a row x 3*H*I*2 bytes, the reference's bench/kernels.py formula) / time of
          the whole layer passes (router GEMM to combine), inputs resident in HBM, each pass
          replayed from a CUDA graph;
  e2e     the same through the public Python API with HOST buffers: hidden states copied from
          pinned memory, `kernels.moe_layer`, result copied back, every pass;
  roofline the dominant kernel (the fused expert FFN of T=64: both weight streams in one launch)
          alone: algorithmic bytes per launch / its CUDA-event duration, against the measured
          HBM copy bandwidth;
  prefill the same layer in bf16 at 4096 and 8192 tokens with Zipf-skewed routing (compute-bound:
          the tensor-core shape of the expert kernel), TFLOP/s against the measured cuBLAS rate;
  cpu_baseline / --impl reference: the reference's float32 expert loop (`switchyard.moe`,
          imported unchanged from `baseline/_ref` when `python tests/fetch_reference.py` has put
          a copy there; otherwise its restatement in oracle/moe_oracle.py) on the same sweep, on
          the host cores.

`--case MODE:T[...]` runs three passes of one layer shape and nothing else: the small,
self-ending workload that the ncu summaries under profiles/ are captured from.

Prints ONE JSON line on rank 0."""

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

SWEEP = (1, 8, 32, 64)
H, I, E, TOPK = 2048, 1024, 64, 8
EXPERT_BYTES = 3 * H * I * 2          # fp16 bytes of one expert's weights
LAYERS = 8                             # resident weight sets used in rotation (8 x 805 MB)
METRIC, UNIT = "moe_layer_decode_expert_weight_GBps", "GB/s"
# The workload, in the words both arms print (the GPU arm and `--impl reference`).
CONFIG = {"workload": "configs[1]: OLMoE MoE layer decode sweep T=1,8,32,64 (fp16 on the GPU, the reference's "
                      "float32 expert loop on the host); a step = one layer pass at each T",
          "tokens": list(SWEEP), "hidden": H, "expert_width": I, "experts": E, "top_k": TOPK,
          "l2": f"GPU arm: inputs larger than L2, passes rotate over {LAYERS} resident weight sets of 805 MB; "
                "host arm: one float32 weight set",
          "seeds": {"weights": "100 + weight set", "hidden": "T"}}


def ncu_traffic():
    """DRAM bytes per launch of the dominant kernel from the committed ncu capture (a number
    measured once under ncu; the file names the capture it came from), or None."""
    try:
        with open(os.path.join(ROOT, "profiles", "expert_ffn_decode_T64_fp16.json")) as f:
            rec = json.load(f)
        return float(rec["dram_bytes_per_launch"]), rec.get("source")
    except Exception:
        return None, None


def peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            p = json.load(f)
        return float(p["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


def tensor_peak():
    """Sustained dense bf16 rate of cuBLAS on this pool's B200 (TFLOP/s): the prefill layer runs
    for hundreds of microseconds back to back, so the sustained figure is its denominator."""
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            p = json.load(f)
        return float(p["bf16_tflops_sustained"]), "measured"
    except Exception:
        return 1400.0, "fallback"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons sampled every 50 ms from the start of the timed region
    to the end of the last device-timed leg (steps, per-T sweep, end to end, dominant kernel)."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.p = index, None

    def __enter__(self):
        try:
            self.p = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                       "-lms", "50", "-i", str(self.index)], stdout=subprocess.PIPE,
                                      stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.p = None
        return self

    def __exit__(self, *a):
        return False

    def stop(self):
        if self.p is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.p.terminate()
        try:
            out, _ = self.p.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.p.kill()
            out, _ = self.p.communicate()
        sm, mx, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in out.strip().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


# ------------------------------------------------------------------------------ CPU arm
def reference_math():
    """(route, experts, kind): the reference's own `switchyard.moe` when a copy of the reference
    sits in baseline/_ref (kind "reference"), else its restatement in oracle/ (kind "port")."""
    ref = os.path.join(ROOT, "baseline", "_ref")
    if os.path.exists(os.path.join(ref, "switchyard", "moe.py")):
        try:
            sys.path.insert(0, ref)
            from switchyard import moe
            return moe.route, moe.experts_reference, "reference"
        except Exception:
            pass
        finally:
            sys.path.remove(ref)
    from oracle import moe_oracle as mo
    return mo.route_reference, mo.experts_reference, "port"


def cpu_sweep_inputs():
    """float32 weights and hidden states of the sweep on the host: weight set 0 and the hidden
    states of the GPU arm (same seeds, same distributions; generated on the CPU)."""
    g = torch.Generator().manual_seed(100)
    router = torch.randn(E, H, generator=g) * 0.02
    gate_up = torch.empty(E, 2 * I, H)
    down = torch.empty(E, H, I)
    for e in range(E):
        gate_up[e] = torch.randn(2 * I, H, generator=g) * 0.02
        down[e] = torch.randn(H, I, generator=g) * 0.02
    hs = {T: torch.randn(T, H, generator=torch.Generator().manual_seed(T)) for T in SWEEP}
    return router, gate_up, down, hs


def cpu_sweep_once(route, experts, router, gate_up, down, hs):
    """One sweep of the float32 reference loop; returns (seconds, algorithmic fp16 bytes)."""
    total_bytes, t0 = 0, time.perf_counter()
    for T in SWEEP:
        idx, w = route(hs[T], router, TOPK, False)
        experts(hs[T], idx, w, gate_up, down)
        total_bytes += int(torch.unique(idx).numel()) * EXPERT_BYTES
    return time.perf_counter() - t0, total_bytes


def cpu_leg(sweeps, warmup=1):
    route, experts, kind = reference_math()
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    router, gate_up, down, hs = cpu_sweep_inputs()
    for _ in range(warmup):
        cpu_sweep_once(route, experts, router, gate_up, down, hs)
    times, nbytes = [], 0
    for _ in range(sweeps):
        dt, nbytes = cpu_sweep_once(route, experts, router, gate_up, down, hs)
        times.append(dt)
    return times, nbytes, torch.get_num_threads(), kind


def run_reference(args):
    """--impl reference: the reference's CPU implementation of the path (its float32 expert
    loop) on the host cores, one sweep per step."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    times, nbytes, threads, kind = cpu_leg(args.steps, args.warmup)
    total = sum(times)
    value = nbytes * len(times) / total / 1e9
    source = "switchyard.moe of the reference, imported unchanged" if kind == "reference" else "oracle/moe_oracle.py"
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": total / len(times) * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": CONFIG,
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": kind,
                         "sample": f"{len(times)} sweeps of T=1,8,32,64, float32 expert loop ({source}), torch CPU"},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------ GPU arm
def run_single_gpu(args):
    from switchyard_b200 import kernels, synthetic
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    kernels.ext()
    dtype = torch.float16
    layers = [synthetic.layer_weights(dev, dtype, seed=100 + l) for l in range(LAYERS)]
    hs = {T: synthetic.hidden_states(T, dev, dtype, seed=T) for T in SWEEP}
    mode = "gemv"

    # experts used per (T, layer): fixed by the seeds, needed for the byte count
    used = {}
    for T in SWEEP:
        for l, (router, _, _) in enumerate(layers):
            idx, _ = kernels.route(hs[T], router, TOPK, False)
            used[(T, l)] = int(torch.unique(idx).numel())
    torch.cuda.synchronize()

    # warm-up of every (T, weight set) combination: library load, cuBLAS kernel choice, scratch
    stream = torch.cuda.Stream(dev)
    outs = {}
    with torch.cuda.stream(stream):
        for T in SWEEP:
            for router, gu, dn in layers:
                for _ in range(2):
                    kernels.moe_layer(hs[T], router, gu, dn, TOPK, False, mode)
        stream.synchronize()
    assert kernels.ext().device_status(dev) == 0

    # one CUDA graph per STEP: the four passes of a step back to back, as the layers of a
    # decode loop run (a pass starts while its predecessor drains); a step starting at weight set
    # 0 and one starting at set 4, replayed alternately, so that no pass finds its weights in L2
    step_graphs, step_bytes = [], []
    with torch.cuda.stream(stream):
        for first in range(0, LAYERS, len(SWEEP)):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream):
                for i, T in enumerate(SWEEP):
                    router, gu, dn = layers[(first + i) % LAYERS]
                    outs[("step", first, T)] = kernels.moe_layer(hs[T], router, gu, dn, TOPK, False, mode)
            step_graphs.append(g)
            step_bytes.append(sum(used[(T, (first + i) % LAYERS)] for i, T in enumerate(SWEEP)) * EXPERT_BYTES)
    torch.cuda.synchronize()

    # ---- the timed region: K steps, each one replay of a step graph
    with torch.cuda.stream(stream):
        for i in range(args.warmup):
            step_graphs[i % len(step_graphs)].replay()
        stream.synchronize()
        torch.cuda.synchronize()
        sampler = ClockSampler(dev.index).__enter__()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record(stream)
        for i in range(args.steps):
            step_graphs[i % len(step_graphs)].replay()
        t1.record(stream)
        stream.synchronize()
        torch.cuda.synchronize()
    total_ms = t0.elapsed_time(t1)
    total_bytes = sum(step_bytes[i % len(step_graphs)] for i in range(args.steps))
    value = total_bytes / (total_ms / 1e3) / 1e9

    # ---- per batch size: one graph per T holding that T's pass over each of the eight weight sets
    # back to back (what a decode loop's consecutive layers look like); K replays per T
    sweep = []
    with torch.cuda.stream(stream):
        for T in SWEEP:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream):
                for l, (router, gu, dn) in enumerate(layers):
                    outs[("sweep", T, l)] = kernels.moe_layer(hs[T], router, gu, dn, TOPK, False, mode)
            for _ in range(max(args.warmup // 2, 2)):
                g.replay()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(stream)
            for _ in range(args.steps):
                g.replay()
            b.record(stream)
            stream.synchronize()
            ms = a.elapsed_time(b)
            nbytes = sum(used[(T, l)] for l in range(LAYERS)) * EXPERT_BYTES * args.steps
            sweep.append({"tokens": T, "us_per_layer": ms / (args.steps * LAYERS) * 1e3,
                          "expert_weight_GBps": nbytes / (ms / 1e3) / 1e9,
                          "of_nominal_8TBps": nbytes / (ms / 1e3) / 1e9 / 8000.0,
                          "experts_used_mean": sum(used[(T, l)] for l in range(LAYERS)) / LAYERS})
            del g

    # ---- end to end through the public API with host buffers: kernels.GraphedLayer, the layer as
    # a decode loop holds it (launches captured once per batch size); every step copies its
    # input from pinned host memory and its output back
    host_in = {T: hs[T].cpu().pin_memory() for T in SWEEP}
    host_out = {T: torch.empty(T, H, dtype=dtype).pin_memory() for T in SWEEP}
    with torch.cuda.stream(stream):
        graphed = [kernels.GraphedLayer(router, gu, dn, TOPK, False, mode) for router, gu, dn in layers]

    pass_no = [0]

    def e2e_step():
        nbytes = 0
        for T in SWEEP:
            l = pass_no[0] % LAYERS
            pass_no[0] += 1
            graphed[l](host_in[T], out=host_out[T])
            nbytes += used[(T, l)] * EXPERT_BYTES
        torch.cuda.current_stream().synchronize()  # the results are on the host
        return nbytes

    with torch.cuda.stream(stream):
        # set-up, whatever --warmup is: a GraphedLayer captures a (batch size, host buffers) pair
        # the second time it sees it; every pair the steps will use is captured here
        for _ in range(3):
            for g in graphed:
                for T in SWEEP:
                    g(host_in[T], out=host_out[T])
        torch.cuda.current_stream().synchronize()
        for _ in range(args.warmup):
            e2e_step()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        e2e_bytes = sum(e2e_step() for _ in range(args.steps))
        e1.record(stream)
        torch.cuda.synchronize()
    e2e_ms = e0.elapsed_time(e1)
    io_bytes = sum(T * H * 2 for T in SWEEP)

    # ---- the dominant kernel alone: the fused expert launch of T=64 (both weight streams: the
    # launch the layer runs), one launch per weight set in rotation
    T = SWEEP[-1]
    ext = kernels.ext()
    kern_ms, kern_bytes = [], []
    with torch.cuda.stream(stream):
        sorted_in = []
        for l, (router, gu, dn) in enumerate(layers):
            idx, w, counts, offsets, token, wsorted, pos_of = kernels.route_and_sort(hs[T], router, TOPK, False)
            sorted_in.append((token, offsets, wsorted, pos_of))
        # One pair of events around a full rotation of back-to-back launches: with a single launch
        # between the events the host's launch latency (about 10 us) would be counted as kernel time.
        for rep in range(max(args.steps // 2, 4) + 2):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(stream)
            for l in range(LAYERS):
                token, offsets, wsorted, pos_of = sorted_in[l]
                ext.expert_ffn(hs[T], token, layers[l][1], layers[l][2], offsets, T * TOPK, wsorted, 0)
            b.record(stream)
            stream.synchronize()
            if rep >= 2:
                kern_ms.append(a.elapsed_time(b) / LAYERS)
                kern_bytes.append(sum(used[(T, l)] for l in range(LAYERS)) * EXPERT_BYTES / LAYERS)
    peak, peak_src = peaks()
    achieved = sum(kern_bytes) / (sum(kern_ms) / 1e3) / 1e9
    assert ext.device_status(dev) == 0
    clocks = sampler.stop()

    # ---- prefill: the same layer, compute-bound (bf16, Zipf-skewed routing), graph replays
    del step_graphs, graphed, outs, layers
    torch.cuda.empty_cache()
    prefill = prefill_leg(dev, stream, steps=max(args.steps // 2, 6))

    # ---- CPU baseline (bounded sample of the same sweep)
    cpu_times, cpu_bytes, threads, cpu_kind = cpu_leg(sweeps=20, warmup=1)
    cpu_value = cpu_bytes * len(cpu_times) / sum(cpu_times) / 1e9
    traffic, traffic_src = ncu_traffic()

    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": total_ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f16", "data": "synthetic",
        "config": CONFIG,
        "arm": {"mode": mode, "path": "router GEMM (library) -> route + sort (one launch) -> expert FFN (tcgen05 weight "
                                      "stream, both projections in one launch) -> combine",
                "timing": "CUDA events on the launch stream around K replays of CUDA graphs holding one step "
                          "(the four layer passes back to back); `sweep`: per T, replays of one graph holding "
                          "that T's pass over each of the eight weight sets"},
        "sweep": sweep,
        "vs_nominal_8TBps": value / 8000.0,
        "clocks": clocks,
        "e2e": {"value": e2e_bytes / (e2e_ms / 1e3) / 1e9, "unit": UNIT, "h2d_bytes_per_step": io_bytes,
                "d2h_bytes_per_step": io_bytes, "ms_per_step": e2e_ms / args.steps,
                "api": "switchyard_b200.kernels.GraphedLayer (moe_layer captured per batch size), host buffers pinned, H2D and D2H every step"},
        # this library's kernels in the timed region, per layer pass: route + sort, expert FFN, and the
        # combine where it is not folded into the expert launch; the library's router GEMM is not counted
        "gpu_launches": args.steps * sum(2 + (T * TOPK < kernels.FUSED_COMBINE_MIN_ROWS) for T in SWEEP),
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "traffic": traffic, "traffic_source": traffic_src, "peak_source": peak_src,
                     "kernel": "gemm_umma_kernel<half, streaming shape>: gate/up + down projections (sy_expert_ffn)",
                     "workload": "T=64, one layer's experts in one launch, weight sets in rotation",
                     "bytes_per_launch": statistics.mean(kern_bytes), "us_per_launch": statistics.mean(kern_ms) * 1e3,
                     "vs_nominal_8TBps": achieved / 8000.0},
        "prefill": prefill,
        "cpu_baseline": {"value": cpu_value, "unit": UNIT, "cores": threads, "kind": cpu_kind,
                         "sample": f"{len(cpu_times)} sweeps of T=1,8,32,64, float32 expert loop, torch CPU",
                         "ms_per_sweep": statistics.median(cpu_times) * 1e3},
    }
    print(json.dumps(line), flush=True)


def prefill_leg(dev, stream, steps):
    """configs[3] at one GPU: the layer in bf16 at 4096 and 8192 tokens, Zipf-skewed routing
    (busiest expert about four times the mean), whole layer (router GEMM to combine) replayed from
    CUDA graphs over three weight sets. FLOPs = rows x 12 582 912 (both projections)."""
    from switchyard_b200 import kernels, synthetic
    dtype, n_sets = torch.bfloat16, 3
    layers = [synthetic.layer_weights(dev, dtype, seed=200 + l) for l in range(n_sets)]
    bias = synthetic.zipf_bias().to(dev).to(dtype)
    peak, peak_src = tensor_peak()
    out = []
    with torch.cuda.stream(stream):
        for T in (4096, 8192):
            h = synthetic.hidden_states(T, dev, dtype, seed=T)

            def run(l):
                srt = kernels.route_and_sort(h, layers[l][0], TOPK, False, bias)
                return kernels._sorted_experts(h, srt, layers[l][1], layers[l][2], TOPK, "gemm")

            for l in range(n_sets):
                run(l)
            stream.synchronize()
            graphs, keep = [], []
            for l in range(n_sets):
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=stream):
                    keep.append(run(l))
                graphs.append(g)
            for i in range(3):
                graphs[i % n_sets].replay()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(stream)
            for i in range(steps):
                graphs[i % n_sets].replay()
            b.record(stream)
            stream.synchronize()
            ms = a.elapsed_time(b) / steps
            tflops = T * TOPK * 12582912 / (ms / 1e3) / 1e12
            out.append({"tokens": T, "dtype": "bf16", "routing": "zipf", "ms_per_layer": ms, "tflops": tflops,
                        "frac_of_sustained": tflops / peak, "peak_tflops": peak, "peak_source": peak_src,
                        "tile": "pair" if T * TOPK >= E * 768 else "single", "timing": f"{steps} graph replays"})
            del graphs, keep
    return out


def run_case(spec):
    """--case MODE:T[:bf16][:zipf]: three passes of one layer shape and nothing else. This is the
    small, self-ending program that ncu captures are taken from (two resident weight sets)."""
    from switchyard_b200 import kernels, synthetic
    parts = spec.split(":")
    mode, T = parts[0], int(parts[1])
    dtype = torch.bfloat16 if "bf16" in parts[2:] else torch.float16
    dev = torch.device("cuda:0")
    if mode == "ep":
        return run_case_ep(spec, T, dtype, dev)
    layers = [synthetic.layer_weights(dev, dtype, seed=100 + l) for l in range(2)]
    h = synthetic.hidden_states(T, dev, dtype, seed=T)
    bias = synthetic.zipf_bias().to(dev).to(dtype) if "zipf" in parts[2:] else None
    for i in range(3):
        router, gu, dn = layers[i % 2]
        if bias is None:
            out = kernels.moe_layer(h, router, gu, dn, TOPK, False, mode)
        else:
            logits = (torch.nn.functional.linear(h, router) + bias).contiguous()
            idx, w = kernels.ext().route(logits, TOPK, False)
            out = kernels.experts(h, idx, w, gu, dn, mode)
    torch.cuda.synchronize()
    print(json.dumps({"case": spec, "checksum": float(out.float().abs().sum()),
                      "device_status": kernels.ext().device_status(dev)}))


def run_case_ep(spec, T, dtype, dev):
    """--case ep:T: the one-process-per-GPU expert-parallel layer with a single rank (all 64
    experts local, every row "sent" to this GPU's own mailbox), three passes: the transport
    kernels (dispatch + build, signal + wait + combine) run on one GPU without a peer to wait for."""
    import torch.distributed as dist
    from switchyard_b200 import kernels, synthetic
    from switchyard_b200.ep_dist import DistributedExpertParallel
    torch.cuda.set_device(dev)
    dist.init_process_group("gloo", init_method="tcp://127.0.0.1:29599", rank=0, world_size=1)
    layers = [synthetic.layer_weights(dev, dtype, seed=100 + l) for l in range(2)]
    h = synthetic.hidden_states(T, dev, dtype, seed=T)
    ep = DistributedExpertParallel(64, TOPK, False, H, I, max_tokens=T, dtype=dtype, mode="auto", device=dev)
    for i in range(3):
        out = ep.layer(h, *layers[i % 2])
    torch.cuda.synchronize()
    same = bool(torch.equal(out, kernels.moe_layer(h, *layers[0], TOPK, False, ep.mode)))
    print(json.dumps({"case": spec, "checksum": float(out.float().abs().sum()), "equals_single_gpu_layer": same,
                      "device_status": kernels.ext().device_status(dev)}))
    ep.close()
    dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--case", default=None, help="MODE:T[:bf16][:zipf] (MODE gemv | gemm | ep) - run one small layer shape (for profiling)")
    ap.add_argument("--mode", default="auto", choices=["auto", "gemv", "gemm"],
                    help="kernel mode for --config ep256 / prefill (auto: by rows per expert)")
    ap.add_argument("--host", default="processes", choices=["processes", "threads"],
                    help="--config ep256 only: one process per GPU under torchrun (ep_dist, graph replays), or ONE process "
                         "driving --gpus N GPUs with a thread each (ep.ExpertParallel, the reference's shape; run without torchrun)")
    ap.add_argument("--placement", default="contiguous", choices=["contiguous", "balanced"],
                    help="expert placement for --config ep256 / prefill on several GPUs: contiguous blocks, or dealt out "
                         "by the measured per-expert load (switchyard_b200.placement.balanced)")
    ap.add_argument("--config", default="decode", choices=["decode", "ep256", "prefill", "model"],
                    help="decode = the bench line (configs[1]); ep256 / prefill / model = configs[2] / configs[3] / configs[4]")
    args = ap.parse_args()
    if args.case:
        return run_case(args.case)
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.impl == "reference":
        return run_reference(args)
    if not torch.cuda.is_available():
        sys.exit("bench.py needs a CUDA GPU (there is no CPU path); use --impl reference for the CPU baseline")
    if args.config != "decode":
        from switchyard_b200 import bench_ep
        if args.config == "ep256" and args.host == "threads":
            return bench_ep.run_threads(args)
        return bench_ep.run_model(args) if args.config == "model" else bench_ep.run_config(args)
    if args.gpus == 1 and int(os.environ.get("WORLD_SIZE", "1")) == 1:
        return run_single_gpu(args)
    from switchyard_b200 import bench_ep
    return bench_ep.run(args)


if __name__ == "__main__":
    main()
