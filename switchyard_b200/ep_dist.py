"""Expert parallelism with one process per GPU (torchrun-style), over this library's
device-driven transport (csrc/ep.cu, host side in ep_window.py).

`ep.ExpertParallel` keeps the reference's shape: one process drives all GPUs, a thread per rank.
`DistributedExpertParallel` is the same transport for one process per GPU: every rank maps every
other rank's window (CUDA IPC), a layer is four launches on the rank's stream (five beyond 256
tokens, where routing and sort are separate), and the host never reads anything back:

    router GEMM, route + sort                     (local tokens, global expert ids)
    ep_expert_ffn                                 prologue: this rank's rows -> owners' mailboxes, their arrival
                                                  flags; waits for its own senders' flags on the device; both
                                                  projections; results stored straight into the senders' y;
                                                  raises the senders' return flags when done
    ep_combine                                    waits for all owners' return flags, sums in expert order

The arithmetic per row and the order of the combine are those of the single-GPU layer with the
same `mode`, so every rank's output is bit-identical to `kernels.moe_layer` on its own tokens
(mode "auto" is resolved from `max_tokens`, which all ranks share, so that it is one mode for the
whole group; it need not be the mode the single-GPU layer would pick for one rank's batch).

`placement`: optional permutation of the experts. Rank r then holds experts
placement[r*per:(r+1)*per] (the caller loads those weights) and the router's rows are permuted
the same way before routing, so the layer computes the same function up to the order in which a
token's expert outputs are added (switchyard/serve.py:14-33).

torch.distributed is used at set-up only (to exchange the 64-byte IPC handles) and never on the
data path."""

import ctypes

import torch
import torch.distributed as dist

from . import _lib, kernels
from .ep_window import Channel, window_layout  # noqa: F401  (window_layout is part of this module's API)


class CudaBackend:
    """What the protocol below needs from a device: the C-ABI library, the torch-level kernel
    wrappers, memory for the window and the scratch, the router GEMM and the current stream.
    Tests substitute an object with the same attributes that keeps windows in host shared memory,
    to run the host-side protocol (layout, pointer tables, call order) in CPU processes."""

    def __init__(self, device):
        self.device = torch.device(device if device is not None else f"cuda:{torch.cuda.current_device()}")
        torch.cuda.set_device(self.device)
        self.lib = _lib.load()
        self.ext = kernels.ext()

    def zeros(self, n, dtype):
        return torch.zeros(n, dtype=dtype, device=self.device)

    def empty(self, shape, dtype):
        return torch.empty(shape, dtype=dtype, device=self.device)

    def route_and_sort(self, h, router, k, norm, bias):
        return kernels.route_and_sort(h, router, k, norm, bias)

    def stream(self):
        return kernels._Device(self.device)

    def sync(self):
        torch.cuda.synchronize(self.device)


class DistributedExpertParallel:
    """One rank of an expert-parallel MoE layer; construct it on every rank of `group`
    (collective). max_tokens bounds the tokens any single rank passes to layer()."""

    def __init__(self, num_experts, top_k, norm_topk_prob, hidden, inter, max_tokens, dtype=torch.float16,
                 mode="gemv", device=None, group=None, logit_bias=None, backend=None, placement=None):
        self.group = group
        self.rank, self.R = dist.get_rank(group), dist.get_world_size(group)
        assert num_experts % self.R == 0, "experts must split evenly over the ranks"
        assert mode in ("gemv", "gemm", "auto"), "mode: gemv, gemm, or auto (from max_tokens)"
        self.E, self.per, self.k, self.norm = num_experts, num_experts // self.R, top_k, norm_topk_prob
        self.H, self.I, self.dtype = hidden, inter, dtype
        # one mode for the whole group: every rank brings up to max_tokens tokens
        self.mode = kernels.auto_mode(max_tokens * self.R * top_k, num_experts) if mode == "auto" else mode
        self.backend = backend if backend is not None else CudaBackend(device)
        self.device = self.backend.device
        self.max_tokens = max_tokens
        self.cap = max_tokens * top_k          # a sender's whole batch may go to one rank
        self.elem = torch.empty(0, dtype=dtype).element_size()
        self.bias = None if logit_bias is None else logit_bias.to(device=self.device, dtype=dtype)
        self.perm = None
        if placement is not None:
            assert sorted(int(e) for e in placement) == list(range(num_experts)), "placement must permute the experts"
            self.perm = torch.tensor([int(e) for e in placement], dtype=torch.int64, device=self.device)
            if self.bias is not None:
                self.bias = self.bias[self.perm].contiguous()
        self._routers = {}                     # id(router) -> (router, its rows in placement order)
        self.lib, self.ext = self.backend.lib, self.backend.ext
        lay = self.layout = window_layout(self.R, self.per, self.cap, self.cap, hidden, self.elem)

        self.window = self.backend.zeros(lay["total"], torch.uint8)
        self.backend.sync()
        handle = (ctypes.c_ubyte * 64)()
        offset = ctypes.c_uint64(0)
        _lib.check(self.lib.sy_ipc_export(self.window.data_ptr(), handle, ctypes.byref(offset)), "ipc_export", self.lib)
        mine = (bytes(handle), int(offset.value))
        everyone = [None] * self.R
        dist.all_gather_object(everyone, mine, group=group)
        bases, self._opened = [], []
        for r, (hbytes, off) in enumerate(everyone):
            if r == self.rank:
                bases.append(self.window.data_ptr())
                continue
            p = ctypes.c_void_p()
            buf = (ctypes.c_ubyte * 64).from_buffer_copy(hbytes)
            _lib.check(self.lib.sy_ipc_open(buf, off, ctypes.byref(p)), "ipc_open", self.lib)
            bases.append(p.value)
            self._opened.append((p.value, off))
        # local scratch of the compute phase
        self.act = self.backend.empty((self.R * self.cap, inter), dtype)
        self.ffn_scratch = self.backend.zeros(self.E + 1, torch.int32)
        code = _lib.SY_DTYPE_F16 if dtype == torch.float16 else _lib.SY_DTYPE_BF16
        self.chan = Channel(self.lib, self.rank, self.R, self.per, top_k, hidden, inter, self.cap, self.cap, self.elem,
                            code, bases, act=self.act.data_ptr(), ffn_scratch=self.ffn_scratch.data_ptr())
        self.stats_box = self.window[lay["stats"]:lay["stats"] + 16].view(torch.int64)
        dist.barrier(group=group)  # every window is mapped everywhere before the first layer

    def _placed(self, router):
        """The router's rows in placement order (cached per router tensor)."""
        if self.perm is None:
            return router
        hit = self._routers.get(id(router))
        if hit is None or hit[0] is not router:
            hit = self._routers[id(router)] = (router, router[self.perm].contiguous())
        return hit[1]

    def layer(self, h, router, gate_up, down, residual=None):
        """h [N,H] this rank's tokens (N <= max_tokens, may be 0); router [E,H] (replicated, rows
        in the model's expert order); gate_up [E/R,2I,H], down [E/R,H,I]: this rank's experts.
        Returns [N,H]; with residual [N,H] (contiguous, h's dtype) residual + layer(h), added in the
        combine launch with the bits of the separate 16-bit addition. Collective: every rank must
        call it once per layer, in the same order."""
        N = h.shape[0]
        if residual is not None and (residual.shape != h.shape or residual.dtype != h.dtype
                                     or not residual.is_contiguous()):
            raise RuntimeError("layer: residual must be contiguous, of h's shape and dtype")
        if N > self.max_tokens:
            raise RuntimeError(f"layer: {N} tokens exceed max_tokens={self.max_tokens}")
        h = h.contiguous()
        idx, _, _, offsets, token, wsorted, pos_of = self.backend.route_and_sort(h, self._placed(router), self.k, self.norm,
                                                                                 self.bias)
        with self.backend.stream() as stream:
            # the dispatch rides in the expert launch's prologue
            self.chan.experts(gate_up.data_ptr(), down.data_ptr(), self.chan.shape_code(self.mode, N), stream,
                              push=(h.data_ptr(), token.data_ptr(), wsorted.data_ptr(), offsets.data_ptr(), N * self.k))
            out = self.backend.empty((N, self.H), self.dtype)
            self.chan.combine(pos_of.data_ptr(), idx.data_ptr(), N, out.data_ptr(), stream,
                              residual.data_ptr() if residual is not None else None)
        return out

    def row_counts(self):
        """(rows this rank has sent to other ranks, rows it kept) since the last call; waits for
        the rank's stream."""
        self.backend.sync()
        sent, kept = self.stats_box.tolist()
        self.stats_box.zero_()
        self.backend.sync()
        return sent, kept

    def check(self):
        """Raises RuntimeError if one of this rank's kernels gave up on a bounded wait (a peer that
        never arrived) since the last check; waits for the rank's stream. Call it when a request
        or a decode step ends, and before trusting a layer's output after a peer may have failed."""
        with self.backend.stream() as stream:
            _lib.check(self.lib.sy_device_status(stream, None), "device_status", self.lib)

    def close(self):
        """Collective. Raises if a bounded wait expired since the last check()."""
        self.backend.sync()
        try:
            self.check()
        finally:
            dist.barrier(group=self.group)
            for p, off in self._opened:
                self.lib.sy_ipc_close(p, off)
            self._opened = []
