"""Expert parallelism with one process per GPU (torchrun-style), over this library's
device-driven transport (csrc/ep.cu).

`ep.ExpertParallel` mirrors the reference: one process drives all GPUs with a thread per rank,
events between streams and one host read per layer. `DistributedExpertParallel` is the form for
one process per GPU: every rank maps every other rank's window (CUDA IPC), a layer is six
launches on the rank's stream (five up to 16 tokens), and the host never reads anything back:

    router GEMM, route, sort                      (local tokens, global expert ids)
    ep_dispatch_build                             rows -> owners' mailboxes, arrival flags; the last block
                                                  waits for all senders and builds the row groups
    expert_ffn                                    both projections; results stored straight into the senders' y
    ep_combine                                    return flags, wait for all owners, sum in expert order

The arithmetic per row and the order of the combine are those of the single-GPU layer with the
same `mode`, so every rank's output is bit-identical to `kernels.moe_layer` on its own tokens.

torch.distributed is used at set-up only (to exchange the 64-byte IPC handles) and never on the
data path."""

import ctypes
import os

import torch
import torch.distributed as dist
import torch.nn.functional as F

from . import _lib, kernels

_ALIGN = 256


def _up(n, a=_ALIGN):
    return (n + a - 1) // a * a


def window_layout(n_ranks, experts_per_rank, capacity, y_rows, hidden, elem_bytes):
    """Byte offsets of the regions of a rank's window. Every rank uses the same layout, so a
    peer's region is its mapped base plus these offsets.
      arrive [R] int32   arrival flag per sender       ret [R] int32   return flag per owner
      done   [1] int32   dispatch's block counter      epoch [1] int32  this rank's layer counter
      meta   [R][per+3] int32
      w      [R][cap]    router weights per sender     x    [R][cap][H] rows per sender
      y      [y_rows][H] results for this rank's own sorted rows"""
    off, lay = 0, {}
    for name, nbytes in (("arrive", 4 * n_ranks), ("ret", 4 * n_ranks), ("done", 4), ("epoch", 4),
                         ("meta", 4 * n_ranks * (experts_per_rank + 3)),
                         ("w", n_ranks * capacity * elem_bytes),
                         ("x", n_ranks * capacity * hidden * elem_bytes),
                         ("y", y_rows * hidden * elem_bytes)):
        lay[name] = off
        off += _up(nbytes)
    lay["total"] = off
    return lay


def _ptr_array(values):
    arr = (ctypes.c_void_p * len(values))(*values)
    return arr


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

    def linear(self, h, router):
        return F.linear(h, router)

    def stream(self):
        return kernels._Device(self.device)

    def sync(self):
        torch.cuda.synchronize(self.device)


class DistributedExpertParallel:
    """One rank of an expert-parallel MoE layer; construct it on every rank of `group`
    (collective). max_tokens bounds the tokens any single rank passes to layer()."""

    def __init__(self, num_experts, top_k, norm_topk_prob, hidden, inter, max_tokens, dtype=torch.float16,
                 mode="gemv", device=None, group=None, logit_bias=None, backend=None, fused_transport=True):
        self.group = group
        self.rank, self.R = dist.get_rank(group), dist.get_world_size(group)
        assert num_experts % self.R == 0, "experts must split evenly over the ranks"
        assert mode in ("gemv", "gemm", "auto"), "mode: gemv, gemm, or auto (by this rank's token count)"
        self.E, self.per, self.k, self.norm = num_experts, num_experts // self.R, top_k, norm_topk_prob
        self.H, self.I, self.dtype, self.mode = hidden, inter, dtype, mode
        # False: the five transport steps as separate launches (dispatch, wait+build, signal, wait, combine)
        self.fused_transport = fused_transport and os.environ.get("SY_EP_SEPARATE_LAUNCHES") != "1"
        self.backend = backend if backend is not None else CudaBackend(device)
        self.device = self.backend.device
        self.max_tokens = max_tokens
        self.cap = max_tokens * top_k          # a sender's whole batch may go to one rank
        self.y_rows = max_tokens * top_k
        self.elem = torch.empty(0, dtype=dtype).element_size()
        self.bias = None if logit_bias is None else logit_bias.to(device=self.device, dtype=dtype)
        self.lib, self.ext = self.backend.lib, self.backend.ext
        lay = self.layout = window_layout(self.R, self.per, self.cap, self.y_rows, hidden, self.elem)

        self.window = self.backend.zeros(lay["total"], torch.uint8)
        self.backend.sync()
        handle = (ctypes.c_ubyte * 64)()
        offset = ctypes.c_uint64(0)
        _lib.check(self.lib.sy_ipc_export(self.window.data_ptr(), handle, ctypes.byref(offset)), "ipc_export")
        mine = (bytes(handle), int(offset.value))
        everyone = [None] * self.R
        dist.all_gather_object(everyone, mine, group=group)
        self.bases, self._opened = [], []
        for r, (hbytes, off) in enumerate(everyone):
            if r == self.rank:
                self.bases.append(self.window.data_ptr())
                continue
            p = ctypes.c_void_p()
            buf = (ctypes.c_ubyte * 64).from_buffer_copy(hbytes)
            _lib.check(self.lib.sy_ipc_open(buf, off, ctypes.byref(p)), "ipc_open")
            self.bases.append(p.value)
            self._opened.append((p.value, off))

        me, cap, H, eb = self.rank, self.cap, hidden, self.elem
        # where this rank's rows for receiver d go: slot `me` of d's mailbox
        self.x_dst = _ptr_array([b + lay["x"] + me * cap * H * eb for b in self.bases])
        self.w_dst = _ptr_array([b + lay["w"] + me * cap * eb for b in self.bases])
        self.meta_dst = _ptr_array([b + lay["meta"] + me * (self.per + 3) * 4 for b in self.bases])
        self.arrive_dst = _ptr_array([b + lay["arrive"] + me * 4 for b in self.bases])
        self.ret_dst = _ptr_array([b + lay["ret"] + me * 4 for b in self.bases])
        self.y_dst = _ptr_array([b + lay["y"] for b in self.bases])
        base = self.window.data_ptr()
        self.p_arrive, self.p_ret, self.p_done = base + lay["arrive"], base + lay["ret"], base + lay["done"]
        self.p_epoch = base + lay["epoch"]
        self.p_meta, self.p_w, self.p_x = base + lay["meta"], base + lay["w"], base + lay["x"]
        self.y = self.window[lay["y"]:lay["y"] + self.y_rows * H * eb].view(dtype).view(self.y_rows, H)
        # local scratch of the compute phase
        G = self.R * self.per
        self.groups = self.backend.zeros(2 * G, torch.int32)
        self.c_table = self.backend.zeros(G, torch.int64)
        self.act = self.backend.empty((self.R * cap, inter), dtype)
        self.ffn_scratch = self.backend.zeros(self.per + 1, torch.int32)
        dist.barrier(group=group)  # every window is mapped everywhere before the first layer

    def layer(self, h, router, gate_up, down):
        """h [N,H] this rank's tokens (N <= max_tokens, may be 0); router [E,H] (replicated);
        gate_up [E/R,2I,H], down [E/R,H,I]: this rank's experts. Returns [N,H]. Collective:
        every rank must call it once per layer, in the same order."""
        N = h.shape[0]
        if N > self.max_tokens:
            raise RuntimeError(f"layer: {N} tokens exceed max_tokens={self.max_tokens}")
        lib, ext, R, per, cap, H = self.lib, self.ext, self.R, self.per, self.cap, self.H
        epoch = self.p_epoch  # the layer counter lives on the device: nothing here changes per layer
        h = h.contiguous()
        logits = self.backend.linear(h, router)
        if self.bias is not None:
            logits = logits + self.bias
        if 0 < N <= kernels.ROUTE_SORT_MAX_TOKENS and N * self.k <= kernels.ROUTE_SORT_MAX_CHOICES and self.E <= 128:
            idx, w, counts, offsets, token, wsorted, pos_of = ext.route_sort(logits.contiguous(), self.k, self.norm)
        else:
            idx, w = ext.route(logits.contiguous(), self.k, self.norm)
            counts, offsets, token, wsorted, pos_of = ext.sort_by_expert(idx, w, self.E)
        M = N * self.k
        code = _lib.SY_DTYPE_F16 if self.dtype == torch.float16 else _lib.SY_DTYPE_BF16
        mode = self.mode
        if mode == "auto":  # every rank brings about as many rows as this one: rows per expert ~ tokens * ranks * k / E
            mode = kernels.auto_mode(N * self.R * self.k, self.E)
        shape = 1 if mode == "gemm" else 0
        with self.backend.stream() as stream:
            G = R * per
            begins, ends = self.groups.data_ptr(), self.groups.data_ptr() + 4 * G
            if not self.fused_transport:
                return self._layer_separate_launches(h, token, wsorted, offsets, pos_of, idx, N, M, gate_up, down, code,
                                                     shape, stream)
            # dispatch; its last block waits for every sender's rows and builds the row groups
            _lib.check(lib.sy_ep_dispatch_build(h.data_ptr(), token.data_ptr(), wsorted.data_ptr(), offsets.data_ptr(), M,
                                                per, R, H * self.elem, cap, self.x_dst, self.w_dst, self.meta_dst,
                                                self.arrive_dst, self.p_done, epoch, self.p_arrive, self.p_meta,
                                                self.y_dst, H * self.elem, begins, ends, self.c_table.data_ptr(), stream),
                       "ep_dispatch_build")
            _lib.check(lib.sy_expert_ffn(self.p_x, None, gate_up.data_ptr(), down.data_ptr(), begins, ends, G, R, R * cap,
                                         H, self.I, self.p_w, self.act.data_ptr(), None, self.c_table.data_ptr(),
                                         self.ffn_scratch.data_ptr(), code, shape, stream), "expert_ffn")
            # tell the senders their results are in place, wait for this rank's own, sum in expert order
            out = self.backend.empty((N, H), self.dtype)
            _lib.check(lib.sy_ep_combine(self.ret_dst, self.p_ret, R, epoch, self.y.data_ptr(), pos_of.data_ptr(),
                                         idx.data_ptr(), N, self.k, H, out.data_ptr(), code, stream), "ep_combine")
        return out

    def _layer_separate_launches(self, h, token, wsorted, offsets, pos_of, idx, N, M, gate_up, down, code, shape, stream):
        """The same layer with every transport step as its own launch."""
        lib, R, per, cap, H, epoch = self.lib, self.R, self.per, self.cap, self.H, self.p_epoch
        G = R * per
        begins, ends = self.groups.data_ptr(), self.groups.data_ptr() + 4 * G
        _lib.check(lib.sy_ep_dispatch(h.data_ptr(), token.data_ptr(), wsorted.data_ptr(), offsets.data_ptr(), M, per, R,
                                      H * self.elem, cap, self.x_dst, self.w_dst, self.meta_dst, self.arrive_dst,
                                      self.p_done, epoch, stream), "ep_dispatch")
        _lib.check(lib.sy_ep_wait_build(self.p_arrive, self.p_meta, per, R, cap, self.y_dst, H * self.elem, epoch, begins,
                                        ends, self.c_table.data_ptr(), stream), "ep_wait_build")
        _lib.check(lib.sy_expert_ffn(self.p_x, None, gate_up.data_ptr(), down.data_ptr(), begins, ends, G, R, R * cap, H,
                                     self.I, self.p_w, self.act.data_ptr(), None, self.c_table.data_ptr(),
                                     self.ffn_scratch.data_ptr(), code, shape, stream), "expert_ffn")
        _lib.check(lib.sy_ep_signal(self.ret_dst, R, epoch, stream), "ep_signal")
        _lib.check(lib.sy_ep_wait(self.p_ret, R, epoch, stream), "ep_wait")
        return self.ext.combine(self.y, pos_of, idx, N)

    def close(self):
        self.backend.sync()
        dist.barrier(group=self.group)
        for p, off in self._opened:
            self.lib.sy_ipc_close(p, off)
        self._opened = []
