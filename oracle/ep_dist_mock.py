"""A host-memory stand-in for the device side of switchyard_b200.ep_dist. TEST INFRASTRUCTURE ONLY.

`DistributedExpertParallel` talks to its device through a small backend object: the C-ABI entry
points of the transport (`sy_ep_dispatch`, `sy_ep_expert_ffn`, `sy_ep_combine`, `sy_ipc_*`), the
routing and sort step, and memory.
`MockBackend` provides the same names over HOST shared memory: a rank's window is a file in
/dev/shm that the other processes map (the stand-in for CUDA IPC), "kernels" are numpy / torch
code working on raw addresses, and flag waits are bounded polling loops. With it the product's
host-side protocol (window layout, pointer tables, argument order, epochs, buffer reuse) runs in
real separate processes over gloo, without a GPU.

The arithmetic follows the kernel rules of oracle/moe_oracle.py, one row at a time, so that a
row's result does not depend on how rows are grouped (the property the GPU kernels have)."""

import ctypes
import os
import tempfile
import time

import numpy as np
import torch

from . import moe_oracle as mo

WAIT_SECONDS = 30.0


def _view(addr, count, dtype):
    """numpy view of `count` items of `dtype` at raw address `addr`."""
    nbytes = count * np.dtype(dtype).itemsize
    buf = (ctypes.c_ubyte * nbytes).from_address(int(addr))
    return np.frombuffer(buf, dtype=dtype, count=count)


def _addr(p):
    return p.value if isinstance(p, ctypes.c_void_p) else (0 if p is None else int(p))


def _torch16(addr, rows, cols, dtype):
    a = _view(addr, rows * cols, np.int16)
    return torch.from_numpy(a).view(dtype).view(rows, cols)


def _row_linear(x_row, W):
    """One row through nn.Linear weights in float32: the same arithmetic whatever the batch."""
    return (W.float() @ x_row.float())


class _Lib:
    """The transport entry points, on host memory."""

    def __init__(self):
        self.maps = {}   # address -> tensor keeping a peer mapping alive
        self.error = b""

    def sy_last_error(self):
        return self.error

    # ---- the stand-in for CUDA IPC: a window is a file in /dev/shm
    def sy_ipc_export(self, ptr, handle, offset_ref):
        path = MockBackend.paths[_addr(ptr)].encode()
        assert len(path) < 64
        for i in range(64):
            handle[i] = path[i] if i < len(path) else 0
        offset_ref._obj.value = 0
        return 0

    def sy_ipc_open(self, handle, offset, out_ref):
        path = bytes(handle).split(b"\0")[0].decode()
        t = torch.from_file(path, shared=True, size=os.path.getsize(path), dtype=torch.uint8)
        self.maps[t.data_ptr()] = t
        out_ref._obj.value = t.data_ptr() + offset
        return 0

    def sy_ipc_close(self, ptr, offset):
        self.maps.pop(int(ptr) - offset, None)
        return 0

    # ---- transport
    def sy_ep_dispatch(self, h, token, wsorted, offsets, rows_bound, per, R, self_rank, row_bytes, cap, x_dst, w_dst,
                       meta_dst, flag_dst, counters, epoch_counter, stats, stream):
        off = _view(offsets, R * per + 1, np.int32)
        m = int(off[R * per])
        tok = _view(token, m, np.int32) if m else np.zeros(0, np.int32)
        wsrc = _view(wsorted, m, np.int16) if m else np.zeros(0, np.int16)
        ep = _view(epoch_counter, 1, np.int32)
        epoch = int(ep[0]) + 1
        for d in range(R):
            a, b = int(off[d * per]), int(off[(d + 1) * per])
            n = min(b - a, cap)
            meta = _view(meta_dst[d], per + 3, np.int32)
            meta[:per + 1] = off[d * per:(d + 1) * per + 1] - a
            meta[per + 1], meta[per + 2] = a, n
            if n:
                src_rows = tok[a:a + n]
                dst = _view(x_dst[d], n * row_bytes, np.uint8).reshape(n, row_bytes)
                hsrc = _view(h, (int(src_rows.max()) + 1) * row_bytes, np.uint8).reshape(-1, row_bytes)
                dst[:] = hsrc[src_rows]
                _view(w_dst[d], n, np.int16)[:] = wsrc[a:a + n]
            _view(flag_dst[d], 1, np.int32)[0] = epoch  # this receiver's rows are in place
        if _addr(stats):
            st = _view(stats, 2, np.int64)
            kept = int(off[(self_rank + 1) * per] - off[self_rank * per])
            st[0] += m - kept
            st[1] += kept
        ep[0] = epoch
        return 0

    def _wait(self, flags, n, epoch):
        f = _view(flags, n, np.int32)
        deadline = time.time() + WAIT_SECONDS
        while not (f >= epoch).all():
            if time.time() > deadline:
                self.error = b"mock: a flag never arrived"
                return False
            time.sleep(0.0005)
        return True

    def _groups(self, meta, per, R, cap, y_dst, out_row_bytes):
        """Row ranges and result addresses from the senders' metadata (what the expert kernel builds)."""
        m = _view(meta, R * (per + 3), np.int32).reshape(R, per + 3)
        b, e, c = np.zeros(R * per, np.int32), np.zeros(R * per, np.int32), np.zeros(R * per, np.uint64)
        for g in range(R * per):
            ex, s = divmod(g, R)
            lo, hi = int(m[s, ex]), min(int(m[s, ex + 1]), cap)
            b[g], e[g] = s * cap + lo, s * cap + max(hi, lo)
            c[g] = int(y_dst[s]) + (int(m[s, per + 1]) + lo) * out_row_bytes
        return b, e, c

    def _segments(self, A, B, b, e, per_expert, n_out, k_dim, swiglu, scale, C, table, dtype):
        dt = torch.float16 if dtype == 0 else torch.bfloat16
        n_full = 2 * n_out if swiglu else n_out
        for g in range(len(b)):
            lo, hi = int(b[g]), int(e[g])
            if hi <= lo:
                continue
            W = _torch16(_addr(B) + (g // per_expert) * n_full * k_dim * 2, n_full, k_dim, dt)
            x = _torch16(_addr(A) + lo * k_dim * 2, hi - lo, k_dim, dt)
            out_addr = int(table[g]) if table is not None else _addr(C) + lo * n_out * 2
            out = _torch16(out_addr, hi - lo, n_out, dt)
            sc = _torch16(_addr(scale) + lo * 2, hi - lo, 1, dt)[:, 0] if _addr(scale) else None
            for r in range(hi - lo):
                acc = _row_linear(x[r], W)[None]
                if swiglu:
                    out[r] = mo.epilogue_swiglu(acc[:, :n_out], acc[:, n_out:], dt)[0]
                elif sc is not None:
                    out[r] = mo.epilogue_scale(acc, sc[r:r + 1], dt)[0]
                else:
                    out[r] = acc.to(dt)[0]

    def sy_ep_expert_ffn(self, x_mail, w_mail, meta, arrive_flags, epoch_counter, R, per, cap, gate_up, down, hidden,
                         inter, act, y_dst, ret_flag_dst, scratch, dtype, compute_shape, push_h, push_token, push_wsorted,
                         push_offsets, push_rows, self_rank, x_dst, w_dst, meta_dst, flag_dst, push_counter, stats, stream):
        if _addr(push_counter):  # the dispatch in the same "launch"
            rc = self.sy_ep_dispatch(push_h, push_token, push_wsorted, push_offsets, push_rows, per, R, self_rank,
                                     hidden * 2, cap, x_dst, w_dst, meta_dst, flag_dst, push_counter, epoch_counter, stats,
                                     stream)
            if rc:
                return rc
        epoch = int(_view(epoch_counter, 1, np.int32)[0])
        if not self._wait(arrive_flags, R, epoch):
            return -3
        b, e, c = self._groups(meta, per, R, cap, y_dst, hidden * 2)
        self._segments(x_mail, gate_up, b, e, R, inter, hidden, 1, None, act, None, dtype)
        self._segments(act, down, b, e, R, hidden, inter, 0, w_mail, None, c, dtype)
        for s in range(R):
            _view(ret_flag_dst[s], 1, np.int32)[0] = epoch
        return 0

    def sy_ep_combine_add(self, ret_flags, R, epoch_counter, y, pos_of, idx, n_tokens, top_k, hidden, residual, out,
                          dtype, stream):
        rc = self.sy_ep_combine(ret_flags, R, epoch_counter, y, pos_of, idx, n_tokens, top_k, hidden, out, dtype, stream)
        if rc == 0 and n_tokens:
            dt = torch.float16 if dtype == 0 else torch.bfloat16
            o = _torch16(_addr(out), n_tokens, hidden, dt)
            o.copy_(_torch16(_addr(residual), n_tokens, hidden, dt) + o)  # the 16-bit addition done separately
        return rc

    def sy_ep_combine(self, ret_flags, R, epoch_counter, y, pos_of, idx, n_tokens, top_k, hidden, out, dtype, stream):
        if not self._wait(ret_flags, R, int(_view(epoch_counter, 1, np.int32)[0])):
            return -3
        if n_tokens == 0:
            return 0
        dt = torch.float16 if dtype == 0 else torch.bfloat16
        m = n_tokens * top_k
        pos = torch.from_numpy(_view(pos_of, m, np.int32).copy())
        ix = torch.from_numpy(_view(idx, m, np.int32).copy()).view(n_tokens, top_k)
        rows = int(pos.max()) + 1
        yy = _torch16(_addr(y), rows, hidden, dt)
        _torch16(_addr(out), n_tokens, hidden, dt).copy_(mo.combine_expert_order(yy, pos, ix, n_tokens))
        return 0

    def sy_device_status(self, stream, out):
        return 0


class _Ext:
    def route(self, logits, k, norm):
        idx, w = mo.route_kernel_rule(logits, k, norm)
        return [idx, w]

    def sort_by_expert(self, idx, w, E):
        return list(mo.sort_by_expert(idx, w, E))

    def route_sort(self, logits, k, norm):
        idx, w = mo.route_kernel_rule(logits, k, norm)
        return [idx, w] + list(mo.sort_by_expert(idx, w, logits.shape[1]))

    def combine(self, y, pos_of, idx, n_tokens):
        return mo.combine_expert_order(y, pos_of, idx, n_tokens)


class _NullStream:
    def __enter__(self):
        return None

    def __exit__(self, *a):
        return False


class MockBackend:
    paths = {}  # window address -> its /dev/shm path (this process)

    def __init__(self):
        self.device = torch.device("cpu")
        self.lib, self.ext = _Lib(), _Ext()
        self._files = []

    def zeros(self, n, dtype):
        item = torch.empty(0, dtype=dtype).element_size()
        fd, path = tempfile.mkstemp(prefix="sy_", dir="/dev/shm")
        os.close(fd)
        os.truncate(path, max(n * item, 1))
        t = torch.from_file(path, shared=True, size=max(n, 1), dtype=dtype)[:n]
        t.zero_()
        self._files.append(path)
        MockBackend.paths[t.data_ptr()] = path
        return t

    def empty(self, shape, dtype):
        return torch.zeros(shape, dtype=dtype)

    def linear(self, h, router):
        return torch.stack([_row_linear(r, router) for r in h]).to(h.dtype) if h.shape[0] else h.new_zeros(0, router.shape[0])

    def route_and_sort(self, h, router, k, norm, bias):
        logits = self.linear(h, router)
        if bias is not None:
            logits = logits + bias
        idx, w = mo.route_kernel_rule(logits, k, norm)
        return [idx, w] + list(mo.sort_by_expert(idx, w, router.shape[0]))

    def stream(self):
        return _NullStream()

    def sync(self):
        pass

    def cleanup(self):
        for p in self._files:
            try:
                os.unlink(p)
            except OSError:
                pass


def single_layer(h, router, gate_up, down, k, norm):
    """The one-process comparand with the same row-at-a-time arithmetic as the mock kernels."""
    be = MockBackend()
    logits = be.linear(h, router)
    idx, w = mo.route_kernel_rule(logits, k, norm)
    counts, offsets, token, wsorted, pos_of = mo.sort_by_expert(idx, w, gate_up.shape[0])
    M, I, H, dt = idx.numel(), gate_up.shape[1] // 2, down.shape[1], h.dtype
    y = torch.zeros(M, H, dtype=dt)
    off = offsets.tolist()
    for e in range(gate_up.shape[0]):
        for r in range(off[e], off[e + 1]):
            acc = _row_linear(h[token[r]], gate_up[e])[None]
            act = mo.epilogue_swiglu(acc[:, :I], acc[:, I:], dt)
            y[r] = mo.epilogue_scale(_row_linear(act[0], down[e])[None], wsorted[r:r + 1], dt)[0]
    return mo.combine_expert_order(y, pos_of, idx, h.shape[0])
