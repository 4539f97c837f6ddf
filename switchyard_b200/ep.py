"""Expert parallelism behind the reference's `ep.py` API.

Every MoE layer's experts are split contiguously over R ranks (rank r owns experts
[r*E/R, (r+1)*E/R)); attention stays data-parallel, so every rank routes and sorts its own
tokens, ships each destination its contiguous segment of sorted rows straight into that
GPU's memory, runs its own experts over every segment it holds, returns each result segment
to the sender's rows, and combines locally. A row's arithmetic is the same as on one GPU and
the combine adds in the same order, so the output is bit-identical to the one-GPU layer run
with the same kernel mode.

Public names, signatures and attributes follow switchyard/ep.py:66-343 (`CudaOps`,
`ExpertParallel` with `phase_send / phase_compute / phase_combine / layer / layer_rank /
run_ranks / layer_threaded / new_state / owner`, and the attributes `stats`, `trace`,
`capacity_factor`, `peer`, `barrier`, `streams`, `mail`), so the reference's `serve.py` and
tests drive it unchanged. What is different underneath:

  * the operations are this package's sm_100a kernels; there is no built-in CPU
    implementation. The protocol itself only talks to an `ops` object with seven methods
    (route, sort, ffn, combine, gather_to, copy_to, host), so tests inject a CPU
    implementation of those to exercise the host logic without a GPU; constructing an
    ExpertParallel on CPU devices WITHOUT passing `ops` raises;
  * what a rank sends to a peer lands in a mailbox on the peer that is allocated once per
    (sender, receiver) pair and reused by every layer (grown when a segment is larger), instead
    of four fresh allocations on the peer per pair per layer. A mailbox is rewritten only
    after the sender has waited for the receiver's results of the previous use, which is
    already part of the protocol (the `back` events).
"""

import math
import threading
from concurrent.futures import ThreadPoolExecutor

import torch


class CudaOps:
    """The seven protocol operations on this package's kernels (switchyard/ep.py:66-95).
    mode: "gemv", "gemm" or "auto" (per segment, by its largest expert's row count)."""

    def __init__(self, mode="auto"):
        from . import kernels
        self.k, self.mode = kernels, mode

    def route(self, h, router, k, norm):
        return self.k.route(h, router, k, norm)

    def sort(self, idx, w, E):
        return self.k.ext().sort_by_expert(idx, w, E)

    def ffn(self, x, a_rows, offsets, counts, wsorted, gate_up, down, rows, host_counts=None):
        mode = self.mode
        if mode == "auto":
            hc = host_counts if host_counts is not None else counts.tolist()
            mode = self.k.pick(max(hc, default=0))
        return self.k.ffn(x, a_rows, offsets, counts, wsorted, gate_up, down, rows, mode, host_counts)

    def combine(self, y, pos_of, idx, N):
        return self.k.ext().combine(y, pos_of, idx, N)

    def gather_to(self, src, index, dst):
        self.k.ext().gather_rows(src, index, dst)

    def copy_to(self, dst, src):
        self.k.ext().copy_async(dst, src)

    def host(self, t):
        return t.tolist()


class _Null:
    def __enter__(self):
        return self

    def __exit__(self, *a):
        return False


class _Mailbox:
    """Buffers on the receiver's device that one sender writes: rows, their router weights,
    the rebased per-expert offsets and the per-expert counts of the segment."""

    __slots__ = ("x", "w", "offsets", "counts", "cap")

    def __init__(self):
        self.x = self.w = self.offsets = self.counts = None
        self.cap = 0

    def fit(self, rows, H, per, dtype, device):
        if self.x is None or rows > self.cap or self.x.shape[1] != H or self.x.dtype != dtype:
            self.cap = max(rows, 2 * self.cap, 64)
            self.x = torch.empty(self.cap, H, dtype=dtype, device=device)
            self.w = torch.empty(self.cap, dtype=dtype, device=device)
            self.offsets = torch.empty(per + 1, dtype=torch.int32, device=device)
            self.counts = torch.empty(per, dtype=torch.int32, device=device)
        return self.x[:rows], self.w[:rows], self.offsets, self.counts


class ExpertParallel:
    """Runs MoE layers whose experts are split over `devices` (one rank per device; ranks may
    share a device, which exercises the protocol on one GPU)."""

    def __init__(self, devices, num_experts, top_k, norm_topk_prob, ops=None):
        self.devices = [torch.device(d) for d in devices]
        self.R = len(self.devices)
        assert num_experts % self.R == 0, "experts must split evenly over the ranks"
        self.E, self.per = num_experts, num_experts // self.R
        self.k, self.norm = top_k, norm_topk_prob
        self.cuda = self.devices[0].type == "cuda"
        if ops is None:
            if not self.cuda:
                raise RuntimeError("switchyard_b200 has no CPU implementation of the MoE operations: "
                                   "use CUDA devices, or pass an `ops` object (tests do)")
            ops = CudaOps()
        self.ops = ops
        self.peer = True
        if self.cuda:
            from . import kernels
            self.streams = [torch.cuda.Stream(d) for d in self.devices]
            # mail[r][d]: kept for API compatibility (the reference allocates what rank r sends
            # to rank d on this stream's pool); here it is the stream the pair's mailbox is
            # allocated on, once.
            self.mail = [[torch.cuda.Stream(d) for d in self.devices] for _ in self.devices]
            ids = sorted({d.index if d.index is not None else torch.cuda.current_device() for d in self.devices})
            self.peer = all(kernels.ext().enable_peer_access(a, b) for a in ids for b in ids if a != b)
        self._boxes = [[_Mailbox() for _ in range(self.R)] for _ in range(self.R)]  # [sender][receiver]
        self.stats = {"dispatched_rows": 0, "local_rows": 0, "dropped_rows": 0, "routed_rows": 0}
        # capacity_factor: None routes every (token, expert) choice. A number c gives every
        # expert room for ceil(c * rows / E) rows of each rank's batch; later rows of an expert
        # (token order) get weight 0 (switchyard/ep.py:127-132).
        self.capacity_factor = None
        # trace: None, or a list that receives (rank, per-expert counts) per layer and rank.
        self.trace = None
        self._pool = None
        self._stats_lock = threading.Lock()
        self.barrier = threading.Barrier(self.R)

    def owner(self, expert):
        return expert // self.per

    # ---- CPU/CUDA helpers
    def _on(self, r):
        if not self.cuda:
            return _Null()
        return _Both(torch.cuda.device(self.devices[r]), torch.cuda.stream(self.streams[r]))

    def _event(self, r):
        if not self.cuda:
            return None
        e = torch.cuda.Event()
        e.record(self.streams[r])
        return e

    def _wait(self, r, event):
        if event is not None:
            self.streams[r].wait_event(event)

    def _count(self, key, n):
        with self._stats_lock:
            self.stats[key] = self.stats.get(key, 0) + n

    def new_state(self):
        R = self.R
        return dict(st=[None] * R, inbox=[[None] * R for _ in range(R)], back=[[] for _ in range(R)])

    # ---- phase 1: route, sort, send
    def phase_send(self, sh, r, h, router):
        """Route rank r's tokens, sort them by global expert, and write every other rank its
        segment (rows, weights, rebased offsets, counts) into the pair's mailbox."""
        ops, R, per = self.ops, self.R, self.per
        # the caller's stream, taken before the MoE stream becomes current: the layer must
        # not read h before the caller's work that produced it (switchyard/ep.py:177-183)
        caller = torch.cuda.current_stream(self.devices[r]) if self.cuda else None
        with self._on(r):
            if caller is not None:
                self.streams[r].wait_stream(caller)
            idx, w = ops.route(h, router, self.k, self.norm)
            counts, offsets, token, wsorted, pos_of = ops.sort(idx, w, self.E)
            if self.capacity_factor is not None:
                wsorted = self._drop(offsets, counts, wsorted)
            if self.trace is not None:
                self.trace.append((r, counts.clone()))
            y = torch.empty(idx.numel(), h.shape[1], dtype=h.dtype, device=h.device)
            off = ops.host(offsets)  # the one host read of the layer
            hc = [off[e + 1] - off[e] for e in range(self.E)]
            seg = [(off[d * per], off[(d + 1) * per]) for d in range(R)]
            sh["st"][r] = dict(idx=idx, offsets=offsets, counts=counts, token=token, wsorted=wsorted,
                               pos_of=pos_of, y=y, seg=seg, hc=hc)
            sh["back"][r] = []
            for d in range(R):
                a, b = seg[d]
                if d == r or b == a:
                    sh["inbox"][d][r] = None
                    continue
                dev = self.devices[d]
                if self.cuda:
                    with torch.cuda.stream(self.mail[r][d]):
                        x, wts, offs, cnt = self._boxes[r][d].fit(b - a, h.shape[1], per, h.dtype, dev)
                else:
                    x, wts, offs, cnt = self._boxes[r][d].fit(b - a, h.shape[1], per, h.dtype, dev)
                lo = offsets[d * per:(d + 1) * per + 1]
                ops.gather_to(h, token[a:b], x)  # straight into rank d's memory
                ops.copy_to(offs, (lo - a).to(lo.dtype).contiguous())
                ops.copy_to(wts, wsorted[a:b].contiguous())
                ops.copy_to(cnt, counts[d * per:(d + 1) * per].contiguous())
                sh["inbox"][d][r] = dict(x=x, offsets=offs, counts=cnt, w=wts, rows=b - a,
                                         hc=hc[d * per:(d + 1) * per], done=self._event(r))
                self._count("dispatched_rows", b - a)

    def _drop(self, offsets, counts, wsorted):
        """Zero the weights of the rows past each expert's capacity (switchyard/ep.py:226-237)."""
        M = wsorted.shape[0]
        if M == 0:
            return wsorted
        cap = math.ceil(self.capacity_factor * M / self.E)
        start = offsets[:-1].long().repeat_interleave(counts.long(), output_size=M)
        keep = (torch.arange(M, device=wsorted.device) - start) < cap
        self._count("dropped_rows", M - int(keep.sum()))
        self._count("routed_rows", M)
        return wsorted * keep.to(wsorted.dtype)

    # ---- phase 2: experts over the local segment and every received one
    def phase_compute(self, sh, d, h, gate_up, down):
        ops, st, per = self.ops, sh["st"], self.per
        with self._on(d):
            a, b = st[d]["seg"][d]
            if b > a:
                lo = st[d]["offsets"][d * per:(d + 1) * per + 1]
                offs = (lo - a).to(lo.dtype).contiguous()
                cnt = st[d]["counts"][d * per:(d + 1) * per]
                hc = st[d]["hc"][d * per:(d + 1) * per]
                st[d]["y"][a:b] = ops.ffn(h, st[d]["token"][a:b].contiguous(), offs, cnt,
                                          st[d]["wsorted"][a:b].contiguous(), gate_up, down, b - a, hc)
                self._count("local_rows", b - a)
            for r in range(self.R):
                m = sh["inbox"][d][r]
                if m is None:
                    continue
                self._wait(d, m["done"])
                yr = ops.ffn(m["x"], None, m["offsets"], m["counts"], m["w"], gate_up, down, m["rows"], m["hc"])
                a2, b2 = st[r]["seg"][d]
                ops.copy_to(st[r]["y"][a2:b2], yr)  # results home, into the sender's memory
                m["keep"] = yr
                sh["back"][r].append(self._event(d))

    # ---- phase 3: combine at home
    def phase_combine(self, sh, r, n_tokens):
        st = sh["st"][r]
        with self._on(r):
            for e in sh["back"][r]:
                self._wait(r, e)
            out = self.ops.combine(st["y"], st["pos_of"], st["idx"], n_tokens)
        if self.cuda:
            torch.cuda.current_stream(self.devices[r]).wait_stream(self.streams[r])
        return out

    def layer(self, hs, routers, gate_ups, downs):
        """hs[r]: [N_r, H] hidden states of rank r's tokens; routers[r]: the layer's router (on
        every rank); gate_ups[r], downs[r]: rank r's experts. Returns the MoE output for every
        rank's tokens. All ranks driven from this thread (switchyard/ep.py:274-285)."""
        sh = self.new_state()
        for r in range(self.R):
            self.phase_send(sh, r, hs[r], routers[r])
        for d in range(self.R):
            self.phase_compute(sh, d, hs[d], gate_ups[d], downs[d])
        outs = [self.phase_combine(sh, r, hs[r].shape[0]) for r in range(self.R)]
        self._keep = sh  # buffers stay referenced until the next layer
        return outs

    # ---- one thread per rank
    def layer_rank(self, sh, r, h, router, gate_up, down):
        """Rank r's part of one layer, from rank r's thread; the barriers order the phases
        across ranks (switchyard/ep.py:289-296)."""
        self.phase_send(sh, r, h, router)
        self.barrier.wait()
        self.phase_compute(sh, r, h, gate_up, down)
        self.barrier.wait()
        return self.phase_combine(sh, r, h.shape[0])

    def run_ranks(self, fn):
        """fn(r) in one thread per rank (a persistent pool); results in rank order. A rank that
        raises breaks the barrier so the others stop instead of waiting for it, and its
        exception (not their BrokenBarrierError) is re-raised (switchyard/ep.py:298-321)."""
        if self._pool is None:
            self._pool = ThreadPoolExecutor(self.R, thread_name_prefix="switchyard-rank")

        def guarded(r):
            try:
                if self.cuda:
                    torch.cuda.set_device(self.devices[r])
                return fn(r)
            except BaseException:
                self.barrier.abort()
                raise

        futures = [self._pool.submit(guarded, r) for r in range(self.R)]
        errors = [f.exception() for f in futures]  # waits for every rank
        if self.barrier.broken:
            self.barrier.reset()
        real = [e for e in errors if e is not None and not isinstance(e, threading.BrokenBarrierError)]
        if real or any(e is not None for e in errors):
            raise (real or [e for e in errors if e is not None])[0]
        return [f.result() for f in futures]

    def layer_threaded(self, hs, routers, gate_ups, downs):
        """Same as layer(), every rank driven by its own thread."""
        sh = self.new_state()
        outs = self.run_ranks(lambda r: self.layer_rank(sh, r, hs[r], routers[r], gate_ups[r], downs[r]))
        self._keep = sh
        return outs


class _Both:
    def __init__(self, a, b):
        self.a, self.b = a, b

    def __enter__(self):
        self.a.__enter__()
        self.b.__enter__()
        return self

    def __exit__(self, *e):
        self.b.__exit__(*e)
        self.a.__exit__(*e)
        return False
