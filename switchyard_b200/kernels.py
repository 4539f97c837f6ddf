"""The MoE layer's kernels behind the reference's `kernels.py` API.

Same module-level names, argument order, defaults and return values as the reference
(switchyard/kernels.py:12-93), so code written against it (its `ep.CudaOps`, its benches, the
`moe=` hook of its `Model`) runs unchanged. Underneath, `ext()` is not a JIT-built torch
extension but a ctypes binding of this package's C-ABI library of hand-written sm_100a
kernels; this module allocates outputs with torch, checks shapes and dtypes, looks up the
current stream and raises RuntimeError on any failure. There is no CPU path and no other
backend: without the built library every call raises.

Differences a caller can observe:
  * fp16 and bf16 are both accepted (the reference is fp16 only);
  * `grouped_gemm` ignores `tile_offsets` / `total_tiles`: tiles are scheduled on the device
    from `offsets`, so the "gemm" mode never reads anything back to the host;
  * there is no cuBLAS mode; "cublas" is accepted as an alias of "gemm";
  * `experts(mode="auto")` chooses from the token count, not from a device-to-host read of
    the largest expert's row count, so the layer never synchronises;
  * `route_fused` computes the router logits inside the routing launch instead of calling the
    library GEMM. It is not what `moe_layer` uses unless SWITCHYARD_FUSED_ROUTER=1 (or
    `route_and_sort(..., fused=True)`): measured on a B200 the library GEMM followed by the
    one-launch route + sort is faster (10 us against 14-17 us up to 64 tokens), and the fused
    logits, the same dot products summed in another order, can differ from the library's in the
    last bit, so that a token whose k-th and (k+1)-th logits are that close may pick the other
    expert.
"""

import os

import ctypes

import torch
import torch.nn.functional as F

from . import _lib

_EXT = None


def _dtype_code(t, what):
    if t.dtype == torch.float16:
        return _lib.SY_DTYPE_F16
    if t.dtype == torch.bfloat16:
        return _lib.SY_DTYPE_BF16
    raise RuntimeError(f"{what}: fp16 or bf16 expected, got {t.dtype}")


def _check(t, name):
    if not (t.is_cuda and t.is_contiguous()):
        raise RuntimeError(f"{name} must be a contiguous CUDA tensor")
    return t


def _ptr(t):
    return t.data_ptr() if t is not None else None


class _Device:
    """Makes `dev` the current CUDA device for the call when it is not already."""

    __slots__ = ("dev", "prev")

    def __init__(self, dev):
        self.dev = dev.index if dev.index is not None else torch.cuda.current_device()
        self.prev = -1

    def __enter__(self):
        cur = torch.cuda.current_device()
        if cur != self.dev:
            self.prev = cur
            torch.cuda.set_device(self.dev)
        return torch.cuda.current_stream(self.dev).cuda_stream

    def __exit__(self, *a):
        if self.prev >= 0:
            torch.cuda.set_device(self.prev)
        return False


class Scratch:
    """Zeroed int32 device memory that the fused launches count in (per-expert readiness, the
    fused combine's arrivals, the fused routing's ticket). Every launch leaves it zero, so it is
    allocated once and grown on demand. Launches that share one Scratch must not overlap on the
    GPU: eager calls use one per (device, stream); an object that replays its launches from a
    CUDA graph on whatever stream is current (GraphedLayer) owns its own."""

    def __init__(self, device):
        self.device = device
        self.main = torch.zeros(1024, dtype=torch.int32, device=device)
        self.ticket = torch.zeros(1, dtype=torch.int32, device=device)

    def ints(self, n):
        if self.main.numel() < n:
            self.main = torch.zeros(max(n, 2 * self.main.numel()), dtype=torch.int32, device=self.device)
        return self.main


class Ext:
    """The eight operations of the reference's extension module
    (switchyard/csrc/moe_kernels.cu:491-500), on torch tensors, plus this library's fused ones."""

    def __init__(self):
        self.lib = _lib.load()
        self._scratch = {}  # (device index, stream handle) -> Scratch of eager calls

    def scratch(self, device, stream):
        index = device.index if device.index is not None else torch.cuda.current_device()
        s = self._scratch.get((index, stream))
        if s is None:
            s = self._scratch[(index, stream)] = Scratch(torch.device("cuda", index))
        return s

    def expert_ffn(self, x, a_rows, gate_up, down, offsets, rows, wsorted, compute_shape, scratch=None):
        """Both projections of the expert FFN in one launch (sy_expert_ffn): returns y [rows, H]."""
        _check(x, "x"), _check(gate_up, "gate_up"), _check(down, "down"), _check(offsets, "offsets")
        _check(wsorted, "wsorted")
        code = _dtype_code(x, "expert_ffn")
        E, I2, H = gate_up.shape
        if down.shape != (E, H, I2 // 2) or x.shape[1] != H or gate_up.dtype != x.dtype or down.dtype != x.dtype:
            raise RuntimeError("expert_ffn: shapes or dtypes do not match")
        if offsets.dtype != torch.int32 or offsets.numel() != E + 1:
            raise RuntimeError("expert_ffn: offsets must be int32 [E+1]")
        if a_rows is not None:
            _check(a_rows, "a_rows")
        y = torch.empty(rows, H, dtype=x.dtype, device=x.device)
        if rows == 0:
            return y
        act = torch.empty(rows, I2 // 2, dtype=x.dtype, device=x.device)
        with _Device(x.device) as stream:
            ints = (scratch or self.scratch(x.device, stream)).ints(E + 1)
            _lib.check(self.lib.sy_expert_ffn(_ptr(x), _ptr(a_rows), _ptr(gate_up), _ptr(down), _ptr(offsets),
                                              offsets.data_ptr() + 4, E, 1, int(rows), H, I2 // 2, _ptr(wsorted),
                                              _ptr(act), _ptr(y), None, _ptr(ints), code, int(compute_shape), stream),
                       "expert_ffn")
        return y

    def expert_ffn_combine(self, x, token, gate_up, down, offsets, wsorted, pos_of, top_k, scratch=None):
        """The expert FFN in its streaming shape with the combine folded into the down projection's
        epilogue (sy_expert_ffn_combine): one launch from sorted rows to the layer's output.
        Returns out [N, H], bit-identical to expert_ffn followed by combine."""
        for t, name in ((x, "x"), (token, "token"), (gate_up, "gate_up"), (down, "down"), (offsets, "offsets"),
                        (wsorted, "wsorted"), (pos_of, "pos_of")):
            _check(t, name)
        code = _dtype_code(x, "expert_ffn_combine")
        E, I2, H = gate_up.shape
        N, rows = x.shape[0], token.numel()
        if down.shape != (E, H, I2 // 2) or x.shape[1] != H or gate_up.dtype != x.dtype or down.dtype != x.dtype:
            raise RuntimeError("expert_ffn_combine: shapes or dtypes do not match")
        if rows != N * top_k or pos_of.numel() != rows or offsets.numel() != E + 1:
            raise RuntimeError("expert_ffn_combine: rows must be tokens * top_k")
        out = torch.empty(N, H, dtype=x.dtype, device=x.device)
        if rows == 0:
            return out
        both = torch.empty(rows, I2 // 2 + H, dtype=x.dtype, device=x.device)  # act | y: one allocation
        act, y = both.view(-1)[:rows * (I2 // 2)], both.view(-1)[rows * (I2 // 2):]
        need = self.lib.sy_expert_ffn_combine_scratch_bytes(E, N, H) // 4
        with _Device(x.device) as stream:
            ints = (scratch or self.scratch(x.device, stream)).ints(need)
            _lib.check(self.lib.sy_expert_ffn_combine(_ptr(x), _ptr(token), _ptr(gate_up), _ptr(down), _ptr(offsets), E,
                                                      rows, H, I2 // 2, _ptr(wsorted), _ptr(act), _ptr(y), _ptr(pos_of),
                                                      int(top_k), N, _ptr(out), _ptr(ints), code, stream),
                       "expert_ffn_combine")
        return out

    def route_fused(self, h, router, k, norm, bias=None, logits=False, scratch=None):
        """Router GEMM + route + sort_by_expert in one launch (sy_route_fused), for decode-sized
        batches: returns [idx, w, counts, offsets, token, wsorted, pos_of] (+ the logits the routing
        was made from when logits=True)."""
        _check(h, "h"), _check(router, "router")
        code = _dtype_code(h, "route_fused")
        N, H = h.shape
        E = router.shape[0]
        if router.dtype != h.dtype or router.shape[1] != H:
            raise RuntimeError("route_fused: h and router do not match")
        if bias is not None:
            _check(bias, "bias")
            if bias.dtype != h.dtype or bias.numel() != E:
                raise RuntimeError("route_fused: bias must be [E] in h's dtype")
        dev, M = h.device, N * k
        ints = torch.empty(2 * E + 1 + 3 * M, dtype=torch.int32, device=dev)
        counts, offsets = ints[:E], ints[E:2 * E + 1]
        token, pos_of = ints[2 * E + 1:2 * E + 1 + M], ints[2 * E + 1 + M:2 * E + 1 + 2 * M]
        idx = ints[2 * E + 1 + 2 * M:].view(N, k)
        halves = torch.empty(2 * M, dtype=h.dtype, device=dev)
        w, wsorted = halves[:M].view(N, k), halves[M:]
        dump = torch.empty(N, E, dtype=h.dtype, device=dev) if logits else None
        with _Device(dev) as stream:
            ticket = (scratch or self.scratch(dev, stream)).ticket
            _lib.check(self.lib.sy_route_fused(_ptr(h), _ptr(router), _ptr(bias), N, E, H, int(k), int(bool(norm)), code,
                                               _ptr(dump), _ptr(idx), _ptr(w), _ptr(counts), _ptr(offsets), _ptr(token),
                                               _ptr(wsorted), _ptr(pos_of), _ptr(ticket), stream), "route_fused")
        res = [idx, w, counts, offsets, token, wsorted, pos_of]
        return res + [dump] if logits else res

    def route(self, logits, k, norm):
        _check(logits, "logits")
        N, E = logits.shape
        code = _dtype_code(logits, "route")
        idx = torch.empty(N, k, dtype=torch.int32, device=logits.device)
        w = torch.empty(N, k, dtype=logits.dtype, device=logits.device)
        with _Device(logits.device) as stream:
            _lib.check(self.lib.sy_route(_ptr(logits), N, E, int(k), int(bool(norm)), code, _ptr(idx), _ptr(w), stream),
                       "route")
        return [idx, w]

    def sort_by_expert(self, idx, w, E):
        _check(idx, "idx"), _check(w, "w")
        if idx.dtype != torch.int32:
            raise RuntimeError("sort_by_expert: idx must be int32")
        M = idx.numel()
        k = idx.shape[1] if idx.dim() == 2 else 1
        code = _dtype_code(w, "sort_by_expert")
        dev = idx.device
        ints = torch.empty(2 * E + 1 + 2 * M, dtype=torch.int32, device=dev)
        counts, offsets = ints[:E], ints[E:2 * E + 1]
        token, pos_of = ints[2 * E + 1:2 * E + 1 + M], ints[2 * E + 1 + M:]
        wsorted = torch.empty(M, dtype=w.dtype, device=dev)
        need = self.lib.sy_sort_scratch_bytes(M, int(E))
        scratch = torch.empty(need, dtype=torch.uint8, device=dev) if need else None
        with _Device(dev) as stream:
            _lib.check(self.lib.sy_sort_by_expert(_ptr(idx), _ptr(w), M, k, int(E), code, _ptr(counts), _ptr(offsets),
                                                  _ptr(token), _ptr(wsorted), _ptr(pos_of), _ptr(scratch), need, stream),
                       "sort_by_expert")
        return [counts, offsets, token, wsorted, pos_of]

    def route_sort(self, logits, k, norm, scratch=None):
        """route + sort_by_expert in one launch (decode-sized batches): returns
        [idx, w, counts, offsets, token, wsorted, pos_of], the same tensors the two calls give."""
        _check(logits, "logits")
        N, E = logits.shape
        code = _dtype_code(logits, "route_sort")
        dev, M = logits.device, N * k
        ints = torch.empty(2 * E + 1 + 3 * M, dtype=torch.int32, device=dev)
        counts, offsets = ints[:E], ints[E:2 * E + 1]
        token, pos_of = ints[2 * E + 1:2 * E + 1 + M], ints[2 * E + 1 + M:2 * E + 1 + 2 * M]
        idx = ints[2 * E + 1 + 2 * M:].view(N, k)
        halves = torch.empty(2 * M, dtype=logits.dtype, device=dev)
        w, wsorted = halves[:M].view(N, k), halves[M:]
        with _Device(dev) as stream:
            ticket = (scratch or self.scratch(dev, stream)).ticket
            _lib.check(self.lib.sy_route_sort(_ptr(logits), N, E, int(k), int(bool(norm)), code, _ptr(idx), _ptr(w),
                                              _ptr(counts), _ptr(offsets), _ptr(token), _ptr(wsorted), _ptr(pos_of),
                                              _ptr(ticket), stream), "route_sort")
        return [idx, w, counts, offsets, token, wsorted, pos_of]

    def _grouped(self, fn, name, A, a_rows, B, offsets, rows, swiglu, scale):
        _check(A, "A"), _check(B, "B"), _check(offsets, "offsets")
        code = _dtype_code(A, name)
        if B.dtype != A.dtype:
            raise RuntimeError(f"{name}: A and B must have the same dtype")
        E, Nfull, K = B.shape
        if A.shape[1] != K:
            raise RuntimeError(f"{name}: K must match (A has {A.shape[1]}, B has {K})")
        if offsets.dtype != torch.int32 or offsets.numel() != E + 1:
            raise RuntimeError(f"{name}: offsets must be int32 [E+1]")
        if a_rows is not None:
            _check(a_rows, "a_rows")
            if a_rows.dtype != torch.int32:
                raise RuntimeError(f"{name}: a_rows must be int32")
        if scale is not None:
            _check(scale, "scale")
        Nout = Nfull // 2 if swiglu else Nfull
        C = torch.empty(rows, Nout, dtype=A.dtype, device=A.device)
        if rows == 0:
            return C
        with _Device(A.device) as stream:
            _lib.check(fn(_ptr(A), _ptr(a_rows), _ptr(B), _ptr(offsets), E, int(rows), Nout, K, int(bool(swiglu)),
                          _ptr(scale), _ptr(C), code, stream), name)
        return C

    def grouped_gemm(self, A, a_rows, B, offsets, tile_offsets, total_tiles, rows, swiglu, scale):
        return self._grouped(self.lib.sy_grouped_gemm, "grouped_gemm", A, a_rows, B, offsets, rows, swiglu, scale)

    def grouped_gemv(self, A, a_rows, B, offsets, rows, swiglu, scale):
        return self._grouped(self.lib.sy_grouped_gemv, "grouped_gemv", A, a_rows, B, offsets, rows, swiglu, scale)

    def combine(self, y, pos_of, idx, n_tokens, residual=None):
        """residual [n_tokens, H] (optional, y's dtype): returns residual + combine(...) from the same
        launch, with the bits of the separate 16-bit addition."""
        _check(y, "y"), _check(pos_of, "pos_of"), _check(idx, "idx")
        code = _dtype_code(y, "combine")
        H, k = y.shape[1], idx.shape[1]
        out = torch.empty(n_tokens, H, dtype=y.dtype, device=y.device)
        if residual is not None:
            _check(residual, "residual")
            if residual.shape != out.shape or residual.dtype != y.dtype:
                raise RuntimeError("combine: residual must be [n_tokens, hidden] in y's dtype")
        if n_tokens == 0:
            return out
        with _Device(y.device) as stream:
            if residual is None:
                rc = self.lib.sy_combine(_ptr(y), _ptr(pos_of), _ptr(idx), int(n_tokens), k, H, _ptr(out), code, stream)
            else:
                rc = self.lib.sy_combine_add(_ptr(y), _ptr(pos_of), _ptr(idx), int(n_tokens), k, H, _ptr(residual),
                                             _ptr(out), code, stream)
            _lib.check(rc, "combine")
        return out

    def gather_rows(self, src, index, dst):
        _check(src, "src"), _check(index, "index"), _check(dst, "dst")
        n, H = index.numel(), src.shape[1]
        row_bytes = H * src.element_size()
        if row_bytes % 16 or dst.shape[0] != n or dst.shape[1] != H or dst.dtype != src.dtype:
            raise RuntimeError("gather_rows: shapes")
        if n == 0:
            return
        with _Device(src.device) as stream:  # the kernel runs where the rows are read
            _lib.check(self.lib.sy_gather_rows(_ptr(src), _ptr(index), n, row_bytes, _ptr(dst), stream), "gather_rows")

    def copy_async(self, dst, src):
        nbytes = src.numel() * src.element_size()
        if not (dst.is_contiguous() and src.is_contiguous()) or dst.numel() * dst.element_size() != nbytes:
            raise RuntimeError("copy_async: shapes")
        if nbytes == 0:
            return
        with _Device(src.device) as stream:
            _lib.check(self.lib.sy_copy_async(_ptr(dst), _ptr(src), nbytes, stream), "copy_async")

    def enable_peer_access(self, device, peer):
        ok = ctypes.c_int(0)
        _lib.check(self.lib.sy_enable_peer_access(int(device), int(peer), ctypes.byref(ok)), "enable_peer_access")
        return bool(ok.value)

    def device_status(self, device=None):
        """Waits for the current stream and returns (and clears) the device's kernel status
        word: 0 unless a kernel gave up on a bounded wait or skipped a bad index."""
        dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        v = ctypes.c_int(0)
        with _Device(dev) as stream:
            rc = self.lib.sy_device_status(stream, ctypes.byref(v))
            if rc != _lib.SY_ERR_DEVICE:
                _lib.check(rc, "device_status")
        return v.value

    def check_device(self, device=None):
        """Raises RuntimeError if a kernel on `device` gave up on a bounded wait since the last
        check (its results are then garbage). Waits for the current stream; call it at the end of
        a request or a decode step, not per layer."""
        dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        with _Device(dev) as stream:
            _lib.check(self.lib.sy_device_status(stream, None), "device_status")

    def set_wait_limit(self, seconds):
        """How long kernels wait for a flag or for one another before giving up (default 2 s)."""
        _lib.check(self.lib.sy_set_wait_limit_ns(int(seconds * 1e9)), "set_wait_limit_ns")


def ext():
    """The kernel library (loaded on first use). Raises RuntimeError if it was not built."""
    global _EXT
    if _EXT is None:
        _EXT = Ext()
    return _EXT


def tile_offsets(counts, block=64):
    """Cumulative row tiles per expert (switchyard/kernels.py:23-27). Kept for callers of the
    reference API; this library's grouped_gemm does not use it."""
    tiles = (counts + block - 1) // block
    off = torch.zeros(counts.numel() + 1, dtype=torch.int32, device=counts.device)
    off[1:] = torch.cumsum(tiles, 0)
    return off


def route(h, router, top_k, norm_topk_prob):
    """Router GEMM in h's dtype, then the routing kernel: (indices int32 [N,k], weights [N,k])
    (switchyard/kernels.py:30-32)."""
    return ext().route(F.linear(h, router).contiguous(), top_k, norm_topk_prob)


# Measured on a B200 with OLMoE's shapes: the streaming shape ("gemv", 64 token rows per tile)
# wins while few experts need a second row tile, the compute shape ("gemm", 128 token rows
# against 256 weight rows) beyond that. There is no third mode on this hardware.
GEMV_MAX_ROWS = 64
GEMM_MAX_ROWS = 1 << 30
# What "auto" uses instead of a device-to-host read of the counts: the mean rows per expert.
# Whole layer, 64 experts, top-8, graph replays, uniform / Zipf routing: at 384 tokens (48 rows per
# expert) gemv 161 / 177 us against gemm 177 / 182; at 512 tokens 209 / 197 against 182 / 188.
AUTO_GEMV_MAX_MEAN_ROWS = 48


def auto_mode(n_rows, n_experts):
    """The mode "auto" stands for, for n_rows sorted rows over n_experts experts."""
    return "gemv" if n_rows <= AUTO_GEMV_MAX_MEAN_ROWS * n_experts else "gemm"


def pick(max_rows):
    """Mode for a batch whose largest expert has `max_rows` rows (switchyard/kernels.py:41-45)."""
    return "gemv" if max_rows <= GEMV_MAX_ROWS else "gemm"


def ffn(x, a_rows, offsets, counts, wsorted, gate_up, down, rows, mode, host_counts=None, scratch=None):
    """The experts over rows already sorted by expert: row i is x[a_rows[i]] (or x[i] when
    a_rows is None); expert e owns rows offsets[e]:offsets[e+1]. Returns each row's expert
    output scaled by its router weight, [rows, H] (switchyard/kernels.py:48-73). `counts` and
    `host_counts` are accepted for compatibility; neither kernel needs them."""
    E = ext()
    if rows == 0:
        return torch.empty(0, down.shape[1], dtype=x.dtype, device=x.device)
    x = x.contiguous()
    # one launch for both projections (bit-identical to grouped_gemv / grouped_gemm called twice,
    # which remain available on ext() as in the reference)
    if mode == "gemv":
        return E.expert_ffn(x, a_rows, gate_up, down, offsets, rows, wsorted, 0, scratch)
    if mode in ("gemm", "cublas"):
        # Compute-bound batches: bring the rows into expert order first (one streaming copy),
        # so that both projections load their token tiles as contiguous TMA boxes. Gathering
        # through a_rows inside the kernel is correct too (grouped_gemm does it, as in the
        # reference) but cannot feed the tensor cores at this rate.
        if a_rows is not None:
            xs = torch.empty(rows, x.shape[1], dtype=x.dtype, device=x.device)
            E.gather_rows(x, a_rows, xs)
            x = xs
        return E.expert_ffn(x, None, gate_up, down, offsets, rows, wsorted, 1, scratch)
    raise RuntimeError(f"ffn: unknown mode {mode!r}")


def _sorted_experts(h, srt, gate_up, down, top_k, mode, scratch=None, residual=None):
    """From sorted choices (idx, w, counts, offsets, token, wsorted, pos_of) to the layer's output
    (plus the residual, when given)."""
    idx, _, counts, offsets, token, wsorted, pos_of = srt
    if mode == "auto":
        mode = auto_mode(idx.numel(), gate_up.shape[0])  # no device-to-host read
    if mode == "gemv" and 0 < top_k <= 8 and idx.numel() >= FUSED_COMBINE_MIN_ROWS:
        # streaming shape: the combine rides in the down projection's epilogue (one launch)
        out = ext().expert_ffn_combine(h.contiguous(), token, gate_up, down, offsets, wsorted, pos_of, top_k, scratch)
        return out if residual is None else residual + out
    y = ffn(h, token, offsets, counts, wsorted, gate_up, down, idx.numel(), mode, scratch=scratch)
    return ext().combine(y, pos_of, idx, h.shape[0], residual)


def experts(h, idx, w, gate_up, down, mode="auto"):
    """The experts of one MoE layer on this GPU for routing (idx, w) computed already: sort by
    expert, SwiGLU projection reading rows of h in place, down projection scaled by the router
    weights, combine (switchyard/kernels.py:76-88). idx int32 [N,k] of local expert ids."""
    idx = idx.contiguous()
    w = w.contiguous()
    srt = ext().sort_by_expert(idx, w, gate_up.shape[0])
    return _sorted_experts(h, [idx, w] + srt, gate_up, down, idx.shape[1], mode)


ROUTE_SORT_MAX_CHOICES = 8192  # sy_route_sort_max_choices(): what the one-launch route + sort handles
# Up to this many tokens routing and sort are ONE launch (blocks of sixteen tokens, the last block
# to finish sorts); beyond it the separate routing kernel and the multi-block sort take over.
ROUTE_SORT_MAX_TOKENS = 256
# route_fused (router GEMM inside the routing launch) is used up to this many tokens when asked for.
ROUTE_FUSED_MAX_TOKENS = 64
FUSED_ROUTER = os.environ.get("SWITCHYARD_FUSED_ROUTER") == "1"
# The streaming mode can fold the combine into the expert launch (expert_ffn_combine: one launch
# less). Measured on a B200 (OLMoE layer, graph replays) it does not pay: the expert launch gets
# 4-6 us longer at 64 tokens (per tile a fence, an atomic per row and the re-read of finished
# rows sit in the epilogue), while the separate combine kernel, overlapped by programmatic
# dependent launch, adds 2.8 us. So it is off unless a caller lowers this row count.
FUSED_COMBINE_MIN_ROWS = 1 << 30


def fused_routing_applies(n_tokens, n_experts, hidden, top_k):
    return (0 < n_tokens <= ROUTE_FUSED_MAX_TOKENS and n_tokens * top_k <= ROUTE_SORT_MAX_CHOICES and
            8 <= n_experts <= 128 and n_experts % 8 == 0 and hidden % 32 == 0 and 1 <= top_k <= 8)


def route_and_sort(h, router, top_k, norm_topk_prob, bias=None, scratch=None, fused=None):
    """Everything before the experts: [idx, w, counts, offsets, token, wsorted, pos_of] for h's
    tokens: the library GEMM for the logits (as in the reference, switchyard/kernels.py:30-32),
    then routing and sort in one launch for decode-sized batches, in two or three beyond.
    bias: optional [E] tensor in h's dtype added to the logits. fused=True (default: the
    SWITCHYARD_FUSED_ROUTER environment switch) computes the logits inside the routing launch
    where `route_fused` applies."""
    X = ext()
    N, E = h.shape[0], router.shape[0]
    if (FUSED_ROUTER if fused is None else fused) and fused_routing_applies(N, E, h.shape[1], top_k):
        return X.route_fused(h.contiguous(), router, top_k, norm_topk_prob, bias, scratch=scratch)
    logits = F.linear(h, router)
    if bias is not None:
        logits = logits + bias
    logits = logits.contiguous()
    if 0 < N <= ROUTE_SORT_MAX_TOKENS and N * top_k <= ROUTE_SORT_MAX_CHOICES and E <= 128:
        return X.route_sort(logits, top_k, norm_topk_prob, scratch)
    idx, w = X.route(logits, top_k, norm_topk_prob)
    return [idx, w] + X.sort_by_expert(idx, w, E)


def moe_layer(h, router, gate_up, down, top_k, norm_topk_prob, mode="auto", scratch=None, residual=None):
    """route + experts (switchyard/kernels.py:91-93): router GEMM, routing + sort (one launch for
    decode-sized batches), the expert FFN (one launch), combine. residual [N,H] (optional, beyond
    the reference's signature): returns residual + layer(h), the caller's `x + self.moe(i, h)`
    (switchyard/model.py:135) from the combine launch, same bits as the separate addition."""
    srt = route_and_sort(h, router, top_k, norm_topk_prob, scratch=scratch)
    return _sorted_experts(h, srt, gate_up, down, top_k, mode, scratch, residual)


def moe_layer_with_bias(h, router, gate_up, down, top_k, norm_topk_prob, mode, bias, scratch=None, residual=None):
    """moe_layer with a per-expert bias [E] (h's dtype) added to the router logits before routing:
    how the benchmarks apply their synthetic routing skew."""
    srt = route_and_sort(h, router, top_k, norm_topk_prob, bias, scratch)
    return _sorted_experts(h, srt, gate_up, down, top_k, mode, scratch, residual)


class GraphedLayer:
    """moe_layer for one layer's weights with the launches of every batch size captured once in a
    CUDA graph and replayed afterwards: what a decode loop does with its layers (the reference
    captures its decode step the same way). Call it with h [N,H], on the device or in pinned
    host memory; the result is a buffer owned by this object (valid until the next call with
    the same N), or is copied into `out` (device or pinned host memory) when given. Called with
    the same pair of pinned host buffers again, the two copies are part of the replayed graph.
    Everything is enqueued on the current stream; nothing synchronises. `check()` raises if one of the replayed
    kernels gave up on a bounded wait (call it when a request or a decode step ends)."""

    def __init__(self, router, gate_up, down, top_k, norm_topk_prob, mode="auto"):
        self.args = (router, gate_up, down, top_k, norm_topk_prob, mode)
        self.device = gate_up.device
        self.graphs = {}  # N -> (graph, static input, static output)
        self.staged = {}  # (N, pinned input address, pinned output address) -> graph with the two copies inside
        self._seen = set()  # buffer pairs seen once (a graph is captured when a pair comes back)
        self.scratch = Scratch(self.device)  # the captured launches' counters: not shared with anyone

    def _capture(self, N, dtype):
        router, gate_up, down, top_k, norm, mode = self.args
        x = torch.zeros(N, gate_up.shape[2], dtype=dtype, device=self.device)
        side = torch.cuda.Stream(self.device)
        side.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(side):
            for _ in range(2):  # first use loads the library, cuBLAS picks its kernel, the scratch grows
                moe_layer(x, router, gate_up, down, top_k, norm, mode, self.scratch)
            side.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=side):
                y = moe_layer(x, router, gate_up, down, top_k, norm, mode, self.scratch)
        torch.cuda.current_stream(self.device).wait_stream(side)
        self.graphs[N] = (g, x, y)
        return self.graphs[N]

    def _capture_staged(self, h, out):
        """The layer between two pinned host buffers as ONE graph: copy in, the layer's launches,
        copy out. A decode loop stages its activations in the same pinned buffers every step, so
        the copies become nodes of the graph instead of two more calls per step."""
        N = h.shape[0]
        _, x, _ = self.graphs.get(N) or self._capture(N, h.dtype)
        router, gate_up, down, top_k, norm, mode = self.args
        side = torch.cuda.Stream(self.device)
        side.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(side):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=side):
                x.copy_(h, non_blocking=True)
                y = moe_layer(x, router, gate_up, down, top_k, norm, mode, self.scratch)
                out.copy_(y, non_blocking=True)
        torch.cuda.current_stream(self.device).wait_stream(side)
        self.staged[(N, h.data_ptr(), out.data_ptr())] = (g, h, out, y)  # keeps the buffers alive
        return g

    def __call__(self, h, out=None):
        N = h.shape[0]
        if out is not None and not h.is_cuda and not out.is_cuda and h.is_pinned() and out.is_pinned():
            key = (N, h.data_ptr(), out.data_ptr())
            hit = self.staged.get(key)
            if hit is None and key in self._seen and len(self.staged) < 64:  # a pair that comes back: worth a graph
                hit = (self._capture_staged(h, out),)
            if hit is not None:
                hit[0].replay()
                return out
            self._seen.add(key)
        g, x, y = self.graphs.get(N) or self._capture(N, h.dtype)
        x.copy_(h, non_blocking=True)
        g.replay()
        if out is None:
            return y
        out.copy_(y, non_blocking=True)
        return out

    def check(self):
        ext().check_device(self.device)
