"""The device-driven expert-parallel transport as seen from the host: the layout of a rank's
window and `Channel`, one rank's three launches per layer over the windows of all ranks
(csrc/ep.cu, csrc/gemm.cu). Shared by `ep.ExpertParallel` (one process drives all GPUs; windows
reached by peer access) and `ep_dist.DistributedExpertParallel` (one process per GPU; windows
mapped by CUDA IPC). Nothing here reads anything back from the device.

Replaces, together with the kernels, the per-pair allocations, copies and events of
switchyard/ep.py:193-223, 239-262 and 264-272."""

import ctypes

from . import _lib

_ALIGN = 256


def _up(n, a=_ALIGN):
    return (n + a - 1) // a * a


def window_layout(n_ranks, experts_per_rank, capacity, y_rows, hidden, elem_bytes):
    """Byte offsets of the regions of a rank's window. Every rank uses the same layout, so a
    peer's region is its mapped base plus these offsets.
      arrive   [R] int32      arrival flag per sender        ret   [R] int32  return flag per owner
      epoch    [1] int32      this rank's layer counter      counters [R+1] int32  dispatch scratch
      stats    [2] int64      rows sent away / rows kept, accumulated
      meta     [R][per+3] int32  per sender: rebased offsets | first row | rows
      w        [R][cap]       router weights per sender      x     [R][cap][H] rows per sender
      y        [y_rows][H]    results for this rank's own sorted rows"""
    off, lay = 0, {}
    for name, nbytes in (("arrive", 4 * n_ranks), ("ret", 4 * n_ranks), ("epoch", 4), ("counters", 4 * (n_ranks + 1)),
                         ("stats", 16), ("meta", 4 * n_ranks * (experts_per_rank + 3)),
                         ("w", n_ranks * capacity * elem_bytes),
                         ("x", n_ranks * capacity * hidden * elem_bytes),
                         ("y", y_rows * hidden * elem_bytes)):
        lay[name] = off
        off += _up(nbytes)
    lay["total"] = off
    return lay


def _ptr_array(values):
    return (ctypes.c_void_p * len(values))(*values)


class Channel:
    """Rank `rank`'s end of the transport. `bases[i]` is the address, valid on this rank's
    device, of rank i's window (its own window for i == rank). `act` and `ffn_scratch` are
    addresses of local scratch: [n_ranks*capacity, inter] elements and experts_per_rank+1 zeroed
    int32. `lib` is the C-ABI library (or a stand-in with the same entry points)."""

    def __init__(self, lib, rank, n_ranks, experts_per_rank, top_k, hidden, inter, capacity, y_rows, elem_bytes,
                 dtype_code, bases, act=None, ffn_scratch=None):
        self.lib, self.rank, self.R, self.per, self.k = lib, rank, n_ranks, experts_per_rank, top_k
        self.H, self.I, self.cap, self.elem, self.code = hidden, inter, capacity, elem_bytes, dtype_code
        lay = self.layout = window_layout(n_ranks, experts_per_rank, capacity, y_rows, hidden, elem_bytes)
        row = hidden * elem_bytes
        # where this rank's rows for receiver d go: slot `rank` of d's mailbox
        self.x_dst = _ptr_array([b + lay["x"] + rank * capacity * row for b in bases])
        self.w_dst = _ptr_array([b + lay["w"] + rank * capacity * elem_bytes for b in bases])
        self.meta_dst = _ptr_array([b + lay["meta"] + rank * (experts_per_rank + 3) * 4 for b in bases])
        self.arrive_dst = _ptr_array([b + lay["arrive"] + rank * 4 for b in bases])
        self.ret_dst = _ptr_array([b + lay["ret"] + rank * 4 for b in bases])
        self.y_dst = _ptr_array([b + lay["y"] for b in bases])
        base = bases[rank]
        self.p_arrive, self.p_ret, self.p_epoch = base + lay["arrive"], base + lay["ret"], base + lay["epoch"]
        self.p_counters, self.p_stats = base + lay["counters"], base + lay["stats"]
        self.p_meta, self.p_w, self.p_x, self.p_y = base + lay["meta"], base + lay["w"], base + lay["x"], base + lay["y"]
        self.act, self.ffn_scratch = act, ffn_scratch

    # From this many rows per expert and sender the compute shape tiles every sender's rows of an
    # expert on their own (contiguous in the mailbox: TMA boxes) instead of gathering an expert's
    # rows from all senders into shared tiles; from PAIR_ROWS with CTA pairs.
    SPLIT_ROWS, PAIR_ROWS = 192, 768

    def shape_code(self, mode, n_tokens):
        """compute_shape of sy_ep_expert_ffn for a layer in which the ranks bring about n_tokens
        tokens each."""
        if mode == "gemv":
            return 0
        per_range = n_tokens * self.k / (self.per * self.R)
        return 4 if per_range >= self.PAIR_ROWS else 3 if per_range >= self.SPLIT_ROWS else 1

    def dispatch(self, h, token, wsorted, offsets, rows, stream):
        """Rows of h (picked through token[], sorted by global expert) into the owners' mailboxes."""
        _lib.check(self.lib.sy_ep_dispatch(h, token, wsorted, offsets, rows, self.per, self.R, self.rank,
                                           self.H * self.elem, self.cap, self.x_dst, self.w_dst, self.meta_dst,
                                           self.arrive_dst, self.p_counters, self.p_epoch, self.p_stats, stream),
                   "ep_dispatch", self.lib)

    def experts(self, gate_up, down, compute_shape, stream, push=None):
        """This rank's experts over everything in its mailbox; results go to the senders' y.
        push = (h, token, wsorted, offsets, rows): the layer's dispatch runs in this launch's
        prologue instead of a launch of its own (do not call dispatch() then)."""
        h, token, wsorted, offsets, rows = push if push is not None else (None, None, None, None, 0)
        _lib.check(self.lib.sy_ep_expert_ffn(self.p_x, self.p_w, self.p_meta, self.p_arrive, self.p_epoch, self.R,
                                             self.per, self.cap, gate_up, down, self.H, self.I, self.act, self.y_dst,
                                             self.ret_dst, self.ffn_scratch, self.code, compute_shape, h, token, wsorted,
                                             offsets, rows, self.rank, self.x_dst, self.w_dst, self.meta_dst,
                                             self.arrive_dst, self.p_counters if push is not None else None,
                                             self.p_stats, stream), "ep_expert_ffn", self.lib)

    def combine(self, pos_of, idx, n_tokens, out, stream, residual=None):
        """Waits for every owner's results, then sums each token's rows into out [n_tokens, H];
        residual (an address, optional): [n_tokens, H] added to the rounded sums in the same launch."""
        if residual is None:
            rc = self.lib.sy_ep_combine(self.p_ret, self.R, self.p_epoch, self.p_y, pos_of, idx, n_tokens, self.k,
                                        self.H, out, self.code, stream)
        else:
            rc = self.lib.sy_ep_combine_add(self.p_ret, self.R, self.p_epoch, self.p_y, pos_of, idx, n_tokens, self.k,
                                            self.H, residual, out, self.code, stream)
        _lib.check(rc, "ep_combine", self.lib)
