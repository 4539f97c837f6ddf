"""CPU oracle for the mixture-of-experts layer. TEST INFRASTRUCTURE ONLY.

This file restates, in plain PyTorch / numpy on the CPU, the algorithm of the reference
project's MoE layer (switchyard/moe.py and the arithmetic rules of
switchyard/csrc/moe_kernels.cu). It exists so that the CUDA kernels can be checked; nothing in
the product package imports it, and the product fails loudly without its CUDA library instead
of falling back to anything here. Only the tests, the smoke check and the CPU-baseline leg of
the benchmark may call it.

Parity status: pinned. `tests/golden/make_golden.py` imports the unmodified reference, runs it
on seeded inputs and stores its outputs; `tests/test_oracle.py` checks every function here
against those stored outputs and against the one literal known-answer vector the reference's
tests hold (tests/test_model.py:49-57).

Two families of functions:

* "reference math" (route_reference, plan, expert_mlp, experts_reference, run_sorted,
  combine_index_add, experts_grouped): what switchyard/moe.py computes, any dtype.
* "kernel rules" (route_kernel_rule, sort_by_expert, combine_expert_order,
  epilogue_swiglu, epilogue_scale): the exact tie-breaking, ordering and rounding points of
  the reference CUDA kernels, which define bit-exactness for indices, the sort permutation
  and the combine order.
"""

from __future__ import annotations

import math
from dataclasses import dataclass

import numpy as np
import torch
import torch.nn.functional as F


# --------------------------------------------------------------------------- reference math
def route_reference(h, router, top_k, norm_topk_prob):
    """switchyard/moe.py:17-25. h [N,H] -> (idx int64 [N,k], w [N,k] in h's dtype): softmax in
    float32 over all experts, then top-k, optional renormalisation."""
    logits = F.linear(h, router)
    probs = torch.softmax(logits, dim=-1, dtype=torch.float32)
    w, idx = torch.topk(probs, top_k, dim=-1)
    if norm_topk_prob:
        w = w / w.sum(dim=-1, keepdim=True)
    return idx, w.to(h.dtype)


def expert_mlp(x, gate_up, down):
    """switchyard/moe.py:28-31. SwiGLU expert: x [n,H], gate_up [2I,H] (gate rows first),
    down [H,I]."""
    gate, up = F.linear(x, gate_up).chunk(2, dim=-1)
    return F.linear(F.silu(gate) * up, down)


def experts_reference(h, idx, w, gate_up, down):
    """switchyard/moe.py:34-42. Loop over experts; contributions added in expert order."""
    out = torch.zeros_like(h)
    for e in range(gate_up.shape[0]):
        tok, slot = torch.where(idx == e)
        if tok.numel() == 0:
            continue
        y = expert_mlp(h[tok], gate_up[e], down[e]) * w[tok, slot, None]
        out.index_add_(0, tok, y.to(out.dtype))
    return out


@dataclass
class Plan:
    """switchyard/moe.py:45-53. Row i of the sorted batch is token[i]'s slot[i]-th choice;
    expert e owns rows offsets[e]:offsets[e+1]."""
    token: torch.Tensor
    slot: torch.Tensor
    weight: torch.Tensor
    counts: torch.Tensor
    offsets: torch.Tensor


def plan(idx, w, num_experts):
    """switchyard/moe.py:56-63. Stable sort of the flat choice list by expert."""
    N, k = idx.shape
    flat = idx.reshape(-1).long()
    order = torch.sort(flat, stable=True).indices
    counts = torch.bincount(flat, minlength=num_experts)
    offsets = torch.zeros(num_experts + 1, dtype=torch.int64)
    offsets[1:] = torch.cumsum(counts, 0)
    return Plan(order // k, order % k, w.reshape(-1)[order], counts, offsets)


def run_sorted(x_sorted, counts, gate_up, down):
    """switchyard/moe.py:66-74. Each expert's contiguous slice through that expert."""
    out = torch.empty_like(x_sorted)
    start = 0
    for e, n in enumerate(counts.tolist()):
        if n:
            out[start:start + n] = expert_mlp(x_sorted[start:start + n], gate_up[e], down[e])
        start += n
    return out


def combine_index_add(y_sorted, p, n_tokens):
    """switchyard/moe.py:77-82. Weighted sum back to token order with index_add_."""
    out = torch.zeros(n_tokens, y_sorted.shape[1], dtype=y_sorted.dtype)
    out.index_add_(0, p.token, y_sorted * p.weight[:, None])
    return out


def experts_grouped(h, idx, w, gate_up, down):
    """switchyard/moe.py:85-88."""
    p = plan(idx, w, gate_up.shape[0])
    y = run_sorted(h[p.token], p.counts, gate_up, down)
    return combine_index_add(y, p, h.shape[0])


def moe_layer_fp32(h, router, gate_up, down, top_k, norm_topk_prob):
    """The float32 layer used as the tolerance reference and as the CPU baseline:
    route_reference + experts_reference on float32 copies of the inputs."""
    h32, r32 = h.float(), router.float()
    idx, w = route_reference(h32, r32, top_k, norm_topk_prob)
    return experts_reference(h32, idx, w, gate_up.float(), down.float())


# --------------------------------------------------------------------------- kernel rules
def _butterfly_sum32(v):
    """Sum of 32 float32 lanes in the order of a xor-shuffle butterfly (offsets 16,8,4,2,1).
    v: [..., 32] float32. Every lane ends with the same value; lane 0's is returned."""
    v = v.astype(np.float32)
    for o in (16, 8, 4, 2, 1):
        v = (v + v[..., np.arange(32) ^ o]).astype(np.float32)
    return v[..., 0]


def route_kernel_rule(logits, top_k, norm_topk_prob):
    """The routing rule of the reference kernel (switchyard/csrc/moe_kernels.cu:23-71) on
    already computed router logits [N,E] (fp16 or bf16 tensor, E <= 128, k <= 8):
    float32 max, e = exp(v - max) in float32, top-k on e with ties going to the LOWER expert
    index, weights e / sum(e) (then / sum of the picked weights when norm), rounded to the
    logits' dtype. Slots are in descending probability order.
    Returns (idx int32 [N,k], w [N,k] in logits.dtype).

    Indices are the bit-exact contract. The weights agree with a GPU's expf to within one
    unit of the 16-bit result (libm's float32 exp and CUDA's expf may differ in the last bit).
    """
    dt = logits.dtype
    v = logits.float().numpy().astype(np.float32)
    N, E = v.shape
    lanes = 32
    per_lane = 1 if E <= 32 else (2 if E <= 64 else 4)
    mx = v.max(axis=1, keepdims=True) if N else v.reshape(0, 1)
    ev = np.exp((v - mx).astype(np.float32)).astype(np.float32)
    # per-lane partial sums (expert e lives in lane e % 32, register e // 32), then butterfly
    pad = np.zeros((N, lanes * per_lane), np.float32)
    pad[:, :E] = ev
    lane_sum = np.zeros((N, lanes), np.float32)
    for j in range(per_lane):
        lane_sum = (lane_sum + pad[:, j * lanes:(j + 1) * lanes]).astype(np.float32)
    total = _butterfly_sum32(lane_sum)
    # top-k: value descending, index ascending on ties == stable argsort of -ev
    order = np.argsort(-ev, axis=1, kind="stable")[:, :top_k]
    picked = (np.take_along_axis(ev, order, axis=1) / total[:, None]).astype(np.float32)
    if norm_topk_prob:
        s = np.zeros(N, np.float32)
        for r in range(top_k):
            s = (s + picked[:, r]).astype(np.float32)
        picked = (picked / s[:, None]).astype(np.float32)
    return torch.from_numpy(order.astype(np.int32)), torch.from_numpy(picked).to(dt)


def sort_by_expert(idx, w, num_experts):
    """The five arrays the reference's sort returns (switchyard/csrc/moe_kernels.cu:142-157;
    the same thing switchyard/ep.py:38-42 builds from moe.plan): counts [E] int32, offsets
    [E+1] int32 (exclusive prefix), token [M] int32 (= flat index // k), wsorted [M], pos_of
    [M] int32 (sorted row of flat choice i). Rows of one expert are in increasing flat index."""
    k = idx.shape[1] if idx.dim() == 2 else 1
    flat = idx.reshape(-1).long()
    M = flat.numel()
    order = torch.sort(flat, stable=True).indices
    counts = torch.bincount(flat, minlength=num_experts)[:num_experts]
    offsets = torch.zeros(num_experts + 1, dtype=torch.int64)
    offsets[1:] = torch.cumsum(counts, 0)
    pos_of = torch.empty(M, dtype=torch.int32)
    pos_of[order] = torch.arange(M, dtype=torch.int32)
    return counts.int(), offsets.int(), (order // max(k, 1)).int(), w.reshape(-1)[order], pos_of


def combine_expert_order(y, pos_of, idx, n_tokens):
    """The reference kernel's combine (switchyard/csrc/moe_kernels.cu:417-433): for every
    token, its k rows of y (already scaled by the router weight) are added in float32 in
    ascending expert id order, and the sum is rounded once to y's dtype. Equal expert ids keep
    slot order (insertion sort is stable)."""
    k = idx.shape[1]
    H = y.shape[1]
    out = torch.empty(n_tokens, H, dtype=y.dtype)
    if n_tokens == 0:
        return out
    order = torch.sort(idx.long(), dim=1, stable=True).indices          # [N,k]
    rows = pos_of.long().reshape(n_tokens, k).gather(1, order)           # [N,k]
    acc = torch.zeros(n_tokens, H, dtype=torch.float32)
    for j in range(k):
        acc = acc + y[rows[:, j]].float()
    return acc.to(y.dtype)


def epilogue_swiglu(acc_gate, acc_up, dtype):
    """Rounding points of the fused SwiGLU epilogue (switchyard/csrc/moe_kernels.cu:253-257,
    373-376): g = r(acc_gate), u = r(acc_up), s = r(g / (1 + exp(-g))), out = r(s * u), with
    r = round to the 16-bit dtype and the arithmetic in float32."""
    g = acc_gate.to(dtype).float()
    u = acc_up.to(dtype).float()
    s = (g / (1.0 + torch.exp(-g))).to(dtype).float()
    return (s * u).to(dtype)


def epilogue_scale(acc, scale, dtype):
    """Row-scale epilogue (switchyard/csrc/moe_kernels.cu:258, 377): r(r(acc) * scale[row])."""
    return (acc.to(dtype).float() * scale.float()[:, None]).to(dtype)


def ffn_sorted_kernel_rule(x, a_rows, offsets, wsorted, gate_up, down):
    """Expert FFN over sorted rows with the kernels' rounding points: float32 accumulation of
    each projection (here a float32 matmul, so the K-order differs from a GPU's and results
    agree to accumulation-order noise, not bit for bit), epilogue_swiglu, epilogue_scale.
    x [T,H] 16-bit, a_rows [M] or None, offsets [E+1], wsorted [M]; returns y [M,H]."""
    dt = x.dtype
    xs = x[a_rows.long()] if a_rows is not None else x
    M = xs.shape[0]
    Hout = down.shape[1]
    y = torch.empty(M, Hout, dtype=dt)
    off = offsets.tolist()
    for e in range(gate_up.shape[0]):
        a, b = off[e], off[e + 1]
        if b == a:
            continue
        acc = xs[a:b].float() @ gate_up[e].float().t()
        I = acc.shape[1] // 2
        act = epilogue_swiglu(acc[:, :I], acc[:, I:], dt)
        y[a:b] = epilogue_scale(act.float() @ down[e].float().t(), wsorted[a:b], dt)
    return y


def moe_layer_kernel_rule(h, router, gate_up, down, top_k, norm_topk_prob, logits=None):
    """The whole layer as the CUDA path computes it, on the CPU: logits in h's dtype, kernel
    routing rule, stable sort, FFN with kernel rounding points, expert-order combine."""
    if logits is None:
        logits = F.linear(h.float(), router.float()).to(h.dtype)
    idx, w = route_kernel_rule(logits, top_k, norm_topk_prob)
    counts, offsets, token, wsorted, pos_of = sort_by_expert(idx, w, gate_up.shape[0])
    y = ffn_sorted_kernel_rule(h, token, offsets, wsorted, gate_up, down)
    return combine_expert_order(y, pos_of, idx, h.shape[0])


def capacity_keep_mask(offsets, counts, M, num_experts, capacity_factor):
    """switchyard/ep.py:226-237. Rows past ceil(cf * M / E) within an expert (token order)
    are dropped: returns the boolean keep mask over sorted rows."""
    if M == 0:
        return torch.zeros(0, dtype=torch.bool)
    cap = math.ceil(capacity_factor * M / num_experts)
    start = offsets[:-1].long().repeat_interleave(counts.long(), output_size=M)
    return (torch.arange(M) - start) < cap
