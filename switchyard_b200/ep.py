"""Expert parallelism behind the reference's `ep.py` API, on device-driven transport.

The experts of every MoE layer are split contiguously over R ranks (rank r owns experts
[r*E/R, (r+1)*E/R)); attention stays data-parallel. Each rank routes and sorts its own tokens by
global expert id, so what it owes rank d is one contiguous run of sorted rows; rank d runs its
experts over what every rank sent it and the results land in the SENDER's buffer at the rows the
sender's sort gave them, so the sender's combine is the single-GPU combine. Per row the
arithmetic is that of one GPU and the combine adds in the same order: with an explicit kernel
mode the output is bit-identical to `kernels.moe_layer` on the rank's own tokens.

`ExpertParallel`, `CudaOps` and every public method and attribute keep the names and meanings of
switchyard/ep.py:66-343, so the reference's `serve.ParallelModel` and tests drive this class
unchanged. How a layer moves is new. There are two engines behind the three phases:

  * windows (CUDA ranks with `CudaOps`): every rank owns a window of device memory that all
    ranks address directly (peer access). After routing and sort a rank's layer is two launches
    on its own stream and no host read: `sy_ep_expert_ffn` first stores the rank's rows, weights
    and offsets into the owners' mailboxes and raises their arrival flags, waits for its own
    senders' flags on the device, runs the experts over the whole mailbox and stores each result
    row into the sender's `y`, then raises the senders' return flags; `sy_ep_combine` waits for
    those and sums. Ranks on different GPUs need neither events nor host barriers. Ranks that share a GPU (tests do that) must not wait
    for each other on the device, so there each phase is followed by an event and preceded by
    waits for the previous phase's events, the dispatch is a launch of its own (`sy_ep_dispatch`),
    and `layer_rank` keeps the reference's barriers; the kernels are the same, their flag waits
    then find the flags already raised.
    Windows have a fixed capacity (`max_tokens` per rank and layer, default 4096 or
    SWITCHYARD_EP_MAX_TOKENS); `layer()` / `layer_threaded()` grow them on demand, `layer_rank()`
    cannot (a rank does not know its peers' batch sizes) and raises: call `reserve(n)` first.
  * operations (any other `ops` object): the protocol spelled out on the host over the seven
    operations `route, sort, ffn, combine, gather_to, copy_to, host` that the caller injects.
    This package ships no CPU implementation of them; its tests inject the oracle's to run the
    host logic (segments, mailboxes, rebased offsets, capacity drop, failure handling) without a
    GPU. Constructing an ExpertParallel on CPU devices without `ops` raises.

`stats` is computed lazily: the window engine counts rows on the device and reads the counters
only when `stats` is looked at."""

import math
import os
import threading
from concurrent.futures import ThreadPoolExecutor

import torch

DEFAULT_MAX_TOKENS = 4096


class CudaOps:
    """This package's kernels as the seven operations the host protocol is written in, plus
    `route_sort`, which the window engine prefers (switchyard/ep.py:66-95 is the reference's
    class of the same name and duck type).
    mode: "gemv", "gemm" or "auto". logit_bias: optional [E] tensor added to the router logits
    in their dtype before routing (the benchmarks' synthetic routing skew)."""

    def __init__(self, mode="auto", logit_bias=None):
        from . import kernels as lib
        self.k = lib
        self.mode = mode
        self.logit_bias = logit_bias

    def _bias(self, like):
        b = self.logit_bias
        return None if b is None else b.to(device=like.device, dtype=like.dtype)

    def route_sort(self, hidden, router_weight, top_k, renormalise):
        """route + sort in as few launches as the batch size allows (one for decode sizes)."""
        return self.k.route_and_sort(hidden, router_weight, top_k, renormalise, bias=self._bias(hidden))

    def route(self, hidden, router_weight, top_k, renormalise):
        if self.logit_bias is None:
            return self.k.route(hidden, router_weight, top_k, renormalise)
        logits = torch.nn.functional.linear(hidden, router_weight) + self._bias(hidden)
        return self.k.ext().route(logits.contiguous(), top_k, renormalise)

    def sort(self, choices, weights, n_experts):
        return self.k.ext().sort_by_expert(choices, weights, n_experts)

    def ffn(self, rows_in, picks, offsets, counts, row_weights, gate_up, down, n_rows, host_counts=None):
        mode = self.mode
        if mode == "auto":  # per call, from the largest expert's rows (a host list if the caller has one)
            per_expert = host_counts if host_counts is not None else counts.tolist()
            mode = self.k.pick(max(per_expert, default=0))
        return self.k.ffn(rows_in, picks, offsets, counts, row_weights, gate_up, down, n_rows, mode, host_counts)

    def combine(self, results, row_of_choice, choices, n_tokens):
        return self.k.ext().combine(results, row_of_choice, choices, n_tokens)

    def gather_to(self, source, rows, destination):
        self.k.ext().gather_rows(source, rows, destination)

    def copy_to(self, destination, source):
        self.k.ext().copy_async(destination, source)

    def host(self, tensor):
        return tensor.tolist()


class _Scope:
    """Enters several context managers together (device + stream of a rank; nothing on the CPU)."""

    def __init__(self, *managers):
        self.managers = managers

    def __enter__(self):
        for m in self.managers:
            m.__enter__()
        return self

    def __exit__(self, *exc):
        for m in reversed(self.managers):
            m.__exit__(*exc)
        return False


class ExpertParallel:
    """Runs MoE layers whose experts are split over `devices` (one rank per device; ranks may
    share a device, which exercises the protocol on one GPU)."""

    def __init__(self, devices, num_experts, top_k, norm_topk_prob, ops=None):
        self.devices = list(map(torch.device, devices))
        self.R, self.E, self.k, self.norm = len(self.devices), num_experts, top_k, norm_topk_prob
        if self.E % self.R:
            raise AssertionError(f"{self.E} experts do not split evenly over {self.R} ranks")
        self.per = self.E // self.R
        self.cuda = all(d.type == "cuda" for d in self.devices)
        if ops is None:
            if self.devices[0].type != "cuda":
                raise RuntimeError("switchyard_b200 has no CPU implementation of the MoE operations: "
                                   "use CUDA devices, or pass an `ops` object (tests do)")
            ops = CudaOps()
        self.ops = ops
        self.peer = True
        self.windows = self.cuda and isinstance(ops, CudaOps)   # engine: device windows, or host protocol over ops
        self.shared_gpu = False
        if self.cuda:
            from . import kernels
            ids = [d.index if d.index is not None else torch.cuda.current_device() for d in self.devices]
            self.devices = [torch.device("cuda", i) for i in ids]
            self.shared_gpu = len(set(ids)) < self.R
            self.streams = [torch.cuda.Stream(device=d) for d in self.devices]
            self.mail = [[self.streams[d] for d in range(self.R)] for _ in range(self.R)]  # the reference's name; no own streams here
            uniq = sorted(set(ids))
            self.peer = all(kernels.ext().enable_peer_access(a, b) for a in uniq for b in uniq if a != b)
            if self.windows and not self.peer:
                raise RuntimeError("expert parallelism over device windows needs peer access between all GPUs")
        # What orders the phases of different ranks. Window engine on distinct GPUs: flags on the
        # device, nothing on the host. Everything else: an event per rank and phase (CUDA) and
        # the barrier between phases when ranks run in threads.
        self.host_ordered = not (self.windows and not self.shared_gpu)
        self.max_tokens = int(os.environ.get("SWITCHYARD_EP_MAX_TOKENS", DEFAULT_MAX_TOKENS))
        self._chan = None           # per rank: ep_window.Channel, once the first layer has shown H and dtype
        self._win = None            # per rank: (window tensor, zeroed counters, act scratch or None)
        self._win_key = None
        self._lock = threading.Lock()
        self._counted = {"dispatched_rows": 0, "local_rows": 0, "dropped_rows": 0, "routed_rows": 0}
        self._drop_counts = [None] * self.R   # per rank: device int64 [1], rows the capacity limit zeroed
        # capacity_factor: None routes every (token, expert) choice. A number c gives every
        # expert room for ceil(c * rows / E) rows of each rank's batch; later rows of an expert
        # (token order) get weight 0 (switchyard/ep.py:127-132).
        # trace: None, or a list that receives (rank, per-expert counts) per layer and rank.
        self.capacity_factor, self.trace = None, None
        self.barrier, self._pool = threading.Barrier(self.R), None

    def owner(self, expert):
        """The rank that holds `expert` (contiguous split)."""
        return int(expert) // self.per

    # ------------------------------------------------------------------ bookkeeping
    @property
    def stats(self):
        """Rows sent to other ranks, rows kept, rows whose weight the capacity limit zeroed, rows
        routed while a limit was set. Looking at it waits for the ranks' streams (device counters
        are read here, never inside a layer)."""
        with self._lock:
            self._fold_device_counters()
            return dict(self._counted)

    def _fold_device_counters(self):
        """Adds what the ranks' kernels have counted on the device since the last look."""
        def take(r, box):
            self.streams[r].synchronize()  # the counters are advanced by kernels on the rank's stream
            values = box.tolist()
            box.zero_()
            torch.cuda.current_stream(box.device).synchronize()
            return values

        if self._win is not None:
            for r in range(self.R):
                sent, kept = take(r, self._win[r]["stats"])
                self._counted["dispatched_rows"] += sent
                self._counted["local_rows"] += kept
        for r, t in enumerate(self._drop_counts):
            if t is not None:
                self._counted["dropped_rows"] += take(r, t)[0]

    def _count(self, key, n):
        with self._lock:
            self._counted[key] += n

    def new_state(self):
        """A layer's shared state: what each rank keeps (`st`), what it was sent (`inbox[d][r]`,
        host protocol only) and the events that order the phases (`back`)."""
        ranks = range(self.R)
        return {"st": [None for _ in ranks], "inbox": [[None for _ in ranks] for _ in ranks],
                "back": [[None, None, None] for _ in ranks]}

    def _rank(self, r):
        if not self.cuda:
            return _Scope()
        return _Scope(torch.cuda.device(self.devices[r]), torch.cuda.stream(self.streams[r]))

    def _mark(self, sh, phase, r):
        """Rank r has enqueued its part of `phase`."""
        if self.cuda and self.host_ordered:
            ev = torch.cuda.Event()
            ev.record(self.streams[r])
            sh["back"][r][phase] = ev

    def _after(self, sh, phase, r):
        """Rank r's stream waits for every rank's part of `phase`."""
        if self.cuda and self.host_ordered:
            for other in range(self.R):
                ev = sh["back"][other][phase]
                if ev is not None and other != r:
                    self.streams[r].wait_event(ev)

    # ------------------------------------------------------------------ windows
    def reserve(self, max_tokens):
        """Room for `max_tokens` tokens per rank and layer. Waits for all ranks' work and
        reallocates the windows on next use; call it between layers, from one thread."""
        if max_tokens <= self.max_tokens:
            return
        with self._lock:
            self.max_tokens = 1 << (int(max_tokens) - 1).bit_length()  # grow in powers of two
            if self._win is not None:
                for d in self.devices:
                    torch.cuda.synchronize(d)
                self._fold_device_counters()
                self._win = self._chan = self._win_key = None

    def _channels(self, H, dtype):
        """The ranks' channels, building every rank's window on first use (or after reserve)."""
        key = (H, dtype, self.max_tokens)
        if self._win_key == key:
            return self._chan
        from . import _lib, ep_window, kernels
        with self._lock:
            if self._win_key == key:
                return self._chan
            if self._win_key is not None and self._win_key[:2] != key[:2]:
                raise RuntimeError("ExpertParallel: hidden size or dtype changed between layers")
            lib = kernels.ext().lib
            elem = torch.empty(0, dtype=dtype).element_size()
            cap = self.max_tokens * self.k          # a sender's whole batch may go to one rank
            lay = ep_window.window_layout(self.R, self.per, cap, cap, H, elem)
            wins = []
            for r, dev in enumerate(self.devices):
                t = torch.zeros(lay["total"], dtype=torch.uint8, device=dev)
                wins.append({"mem": t, "ffn": torch.zeros(self.E + 1, dtype=torch.int32, device=dev), "act": None,
                             "stats": t[lay["stats"]:lay["stats"] + 16].view(torch.int64),
                             "y": t[lay["y"]:lay["y"] + cap * H * elem].view(dtype).view(cap, H)})
            for dev in set(self.devices):
                torch.cuda.synchronize(dev)  # zero-filled before any peer writes a flag
            bases = [w["mem"].data_ptr() for w in wins]
            code = _lib.SY_DTYPE_F16 if dtype == torch.float16 else _lib.SY_DTYPE_BF16
            self._chan = [ep_window.Channel(lib, r, self.R, self.per, self.k, H, 0, cap, cap, elem, code, bases,
                                            ffn_scratch=wins[r]["ffn"].data_ptr()) for r in range(self.R)]
            self._win, self._win_key = wins, key
        return self._chan

    # ------------------------------------------------------------------ phase 1
    def phase_send(self, sh, r, h, router):
        """Rank r routes and sorts its tokens by global expert and hands every rank its run of
        sorted rows (with their router weights and the run's per-expert offsets)."""
        # The layer may not read h before the caller's stream has produced it: take the caller's
        # stream before the rank's own stream becomes current (switchyard/ep.py:177-183).
        callers_stream = torch.cuda.current_stream(self.devices[r]) if self.cuda else None
        with self._rank(r):
            if self.cuda:
                self.streams[r].wait_stream(callers_stream)
            srt = self._route_sort(h, router)
            idx, counts, offsets, wsorted = srt[0], srt[2], srt[3], srt[5]
            if self.capacity_factor is not None:
                wsorted = self._drop(r, offsets, counts, wsorted)
            if isinstance(self.trace, list):
                self.trace.append((r, counts.detach().clone()))
            keep = dict(idx=idx, counts=counts, offsets=offsets, token=srt[4], wsorted=wsorted, pos_of=srt[6], h=h)
            sh["st"][r] = keep
            if self.windows:
                self._send_windows(r, h, keep)
            else:
                self._send_ops(sh, r, h, keep)
            self._mark(sh, 0, r)

    def _route_sort(self, h, router):
        ops = self.ops
        if self.windows and hasattr(ops, "route_sort"):
            return ops.route_sort(h, router, self.k, self.norm)
        choices, weights = ops.route(h, router, self.k, self.norm)
        return [choices, weights, *ops.sort(choices, weights, self.E)]

    def _drop(self, r, offsets, counts, wsorted):
        """Weight 0 for the rows past each expert's capacity, ceil(c * rows / E) rows per expert
        in sorted (= token) order (switchyard/ep.py:226-237). Nothing is read back here."""
        M = wsorted.numel()
        if not M:
            return wsorted
        room = math.ceil(self.capacity_factor * M / self.E)
        first = torch.repeat_interleave(offsets[:-1].long(), counts.long(), output_size=M)
        within = torch.arange(M, device=wsorted.device) - first < room
        self._count("routed_rows", M)
        if self.cuda:
            if self._drop_counts[r] is None:
                self._drop_counts[r] = torch.zeros(1, dtype=torch.int64, device=wsorted.device)
            self._drop_counts[r] += (~within).sum()
        else:
            self._count("dropped_rows", int((~within).sum()))
        return wsorted * within.to(wsorted.dtype)

    def _send_windows(self, r, h, keep):
        N = h.shape[0]
        if N > self.max_tokens:
            raise RuntimeError(f"ExpertParallel: {N} tokens on rank {r} exceed max_tokens={self.max_tokens}; "
                               "call reserve() between layers (layer() and layer_threaded() do it themselves)")
        chan = self._channels(h.shape[1], h.dtype)[r]
        h = h.contiguous()
        keep["h"] = h
        if self.host_ordered:  # ranks share a GPU: the dispatch is a launch of its own, followed by an event
            chan.dispatch(h.data_ptr(), keep["token"].data_ptr(), keep["wsorted"].data_ptr(), keep["offsets"].data_ptr(),
                          N * self.k, torch.cuda.current_stream().cuda_stream)

    def _send_ops(self, sh, r, h, keep):
        """Host protocol: one read of the offsets, then per destination a mailbox on its device
        holding the run's rows, weights, rebased offsets and counts."""
        ops, per = self.ops, self.per
        bounds = ops.host(keep["offsets"])  # the host protocol's one device-to-host read
        keep["seg"] = [(bounds[d * per], bounds[(d + 1) * per]) for d in range(self.R)]
        keep["hc"] = [bounds[e + 1] - bounds[e] for e in range(self.E)]
        keep["y"] = torch.empty(keep["idx"].numel(), h.shape[1], dtype=h.dtype, device=h.device)
        for d, (lo, hi) in enumerate(keep["seg"]):
            if d == r or hi == lo:
                sh["inbox"][d][r] = None
                continue
            dev = self.devices[d]
            box = dict(x=torch.empty(hi - lo, h.shape[1], dtype=h.dtype, device=dev),
                       w=torch.empty(hi - lo, dtype=keep["wsorted"].dtype, device=dev),
                       offsets=torch.empty(per + 1, dtype=keep["offsets"].dtype, device=dev),
                       counts=torch.empty(per, dtype=keep["counts"].dtype, device=dev),
                       rows=hi - lo, hc=keep["hc"][d * per:(d + 1) * per])
            ops.gather_to(h, keep["token"][lo:hi], box["x"])
            ops.copy_to(box["w"], keep["wsorted"][lo:hi].contiguous())
            ops.copy_to(box["offsets"], (keep["offsets"][d * per:(d + 1) * per + 1] - lo).to(keep["offsets"].dtype))
            ops.copy_to(box["counts"], keep["counts"][d * per:(d + 1) * per].contiguous())
            if self.cuda:  # written by rank r's stream, read by rank d's: neither is the stream that allocated
                for t in (box["x"], box["w"], box["offsets"], box["counts"]):
                    t.record_stream(self.streams[r])
                    t.record_stream(self.streams[d])
            sh["inbox"][d][r] = box
            self._count("dispatched_rows", hi - lo)

    # ------------------------------------------------------------------ phase 2
    def phase_compute(self, sh, d, h, gate_up, down):
        """Rank d's experts over its own run and over every run it was sent; each result goes
        back to the rows of the rank that sent it."""
        with self._rank(d):
            self._after(sh, 0, d)
            if self.windows:
                self._compute_windows(sh, d, h, gate_up, down)
            else:
                self._compute_ops(sh, d, h, gate_up, down)
            self._mark(sh, 1, d)

    def _compute_windows(self, sh, d, h, gate_up, down):
        from . import kernels
        chan, win = self._chan[d], self._win[d]
        inter = gate_up.shape[1] // 2
        if win["act"] is None or win["act"].shape[1] != inter:
            win["act"] = torch.empty(self.R * chan.cap, inter, dtype=h.dtype, device=h.device)
            chan.act, chan.I = win["act"].data_ptr(), inter
        mode = self.ops.mode
        if mode == "auto":  # from this rank's own batch: ranks may choose differently (no bit-identity promise)
            mode = kernels.auto_mode(h.shape[0] * self.R * self.k, self.E)
        push = None
        if not self.host_ordered:  # distinct GPUs: the dispatch rides in the expert launch's prologue
            mine = sh["st"][d]
            push = (mine["h"].data_ptr(), mine["token"].data_ptr(), mine["wsorted"].data_ptr(), mine["offsets"].data_ptr(),
                    mine["h"].shape[0] * self.k)
        chan.experts(gate_up.data_ptr(), down.data_ptr(), chan.shape_code(mode, h.shape[0]),
                     torch.cuda.current_stream().cuda_stream, push)

    def _compute_ops(self, sh, d, h, gate_up, down):
        ops, per, mine = self.ops, self.per, sh["st"][d]
        lo, hi = mine["seg"][d]
        if hi > lo:  # the rank's own run: rows read in place through token[]
            offs = (mine["offsets"][d * per:(d + 1) * per + 1] - lo).to(mine["offsets"].dtype)
            mine["y"][lo:hi] = ops.ffn(h, mine["token"][lo:hi].contiguous(), offs, mine["counts"][d * per:(d + 1) * per],
                                       mine["wsorted"][lo:hi].contiguous(), gate_up, down, hi - lo,
                                       mine["hc"][d * per:(d + 1) * per])
            self._count("local_rows", hi - lo)
        for r in range(self.R):
            box = sh["inbox"][d][r]
            if box is None:
                continue
            box["y"] = ops.ffn(box["x"], None, box["offsets"], box["counts"], box["w"], gate_up, down, box["rows"], box["hc"])
            a, b = sh["st"][r]["seg"][d]
            ops.copy_to(sh["st"][r]["y"][a:b], box["y"])  # home, at the rows the sender's sort gave them

    # ------------------------------------------------------------------ phase 3
    def phase_combine(self, sh, r, n_tokens):
        mine = sh["st"][r]
        with self._rank(r):
            self._after(sh, 1, r)
            if self.windows:
                h = mine["h"]
                out = torch.empty(n_tokens, h.shape[1], dtype=h.dtype, device=h.device)
                self._chan[r].combine(mine["pos_of"].data_ptr(), mine["idx"].data_ptr(), n_tokens, out.data_ptr(),
                                      torch.cuda.current_stream().cuda_stream)
            else:
                out = self.ops.combine(mine["y"], mine["pos_of"], mine["idx"], n_tokens)
            self._mark(sh, 2, r)
        if self.cuda:  # hand the result to the caller's stream
            caller = torch.cuda.current_stream(self.devices[r])
            caller.wait_stream(self.streams[r])
            out.record_stream(caller)
        return out

    # ------------------------------------------------------------------ whole layers
    def layer(self, hs, routers, gate_ups, downs):
        """hs[r]: [N_r, H] hidden states of rank r's tokens; routers[r]: the layer's router (on
        every rank); gate_ups[r], downs[r]: rank r's experts. Returns the MoE output for every
        rank's tokens. All ranks driven from this thread (switchyard/ep.py:274-285)."""
        if self.windows:
            self.reserve(max(h.shape[0] for h in hs))
        state = self.new_state()
        for r, (h, router) in enumerate(zip(hs, routers)):
            self.phase_send(state, r, h, router)
        for r, (h, gate_up, down) in enumerate(zip(hs, gate_ups, downs)):
            self.phase_compute(state, r, h, gate_up, down)
        results = [self.phase_combine(state, r, h.shape[0]) for r, h in enumerate(hs)]
        self._keep = state  # what the enqueued kernels read stays referenced until the next layer
        return results

    def layer_rank(self, sh, r, h, router, gate_up, down):
        """Rank r's part of one layer, from rank r's thread (switchyard/ep.py:289-296). Ranks whose
        phases are ordered on the host meet at the barrier between phases; ranks on distinct GPUs
        over windows do not meet at all: their kernels wait for each other's flags."""
        meet = self.barrier.wait if self.host_ordered else (lambda: None)
        self.phase_send(sh, r, h, router)
        meet()
        self.phase_compute(sh, r, h, gate_up, down)
        meet()
        return self.phase_combine(sh, r, len(h))

    def run_ranks(self, fn):
        """fn(r) in one thread per rank (a persistent pool); results in rank order. A rank that
        raises breaks the barrier so that the others stop instead of waiting for it, and its
        exception (not their BrokenBarrierError) is what the caller sees (switchyard/ep.py:298-321)."""
        self._pool = self._pool or ThreadPoolExecutor(max_workers=self.R, thread_name_prefix="sy-rank")

        def one(rank):
            if self.cuda:
                torch.cuda.set_device(self.devices[rank])
            try:
                return fn(rank)
            except BaseException:
                self.barrier.abort()  # the others must not wait for a rank that is gone
                raise

        jobs = [self._pool.submit(one, rank) for rank in range(self.R)]
        failures = [j.exception() for j in jobs]  # returns once every rank has finished
        if self.barrier.broken:  # usable again for the next call
            self.barrier.reset()
        own = [f for f in failures if f is not None and not isinstance(f, threading.BrokenBarrierError)]
        if own:
            raise own[0]
        if any(f is not None for f in failures):
            raise next(f for f in failures if f is not None)
        return [j.result() for j in jobs]

    def layer_threaded(self, hs, routers, gate_ups, downs):
        """Same as layer(), every rank driven by its own thread."""
        if self.windows:
            self.reserve(max(h.shape[0] for h in hs))
        state = self.new_state()

        def rank_part(r):
            return self.layer_rank(state, r, hs[r], routers[r], gate_ups[r], downs[r])

        results = self.run_ranks(rank_part)
        self._keep = state
        return results

    def check(self):
        """Raises RuntimeError if a kernel of any rank gave up on a bounded wait (a peer that never
        arrived) since the last check. Waits for the ranks' streams."""
        if not self.cuda:
            return
        from . import kernels
        for r, dev in enumerate(self.devices):
            with self._rank(r):
                kernels.ext().check_device(dev)
