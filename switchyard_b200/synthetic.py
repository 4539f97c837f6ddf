"""Seeded synthetic inputs with the shapes and value distributions of the benchmark
configurations: OLMoE-1B-7B's MoE layer (hidden 2048, 64 experts of width 1024, top-8, no
renormalisation), weights N(0, 0.02), hidden states N(0, 1), and an optional per-expert
Zipf(s=1.1) router bias that makes the busiest expert receive about 4x the mean rows (the skew
the reference measured on real text; the text and checkpoint themselves are not used)."""

import math

import torch

HIDDEN, INTER, EXPERTS, TOP_K = 2048, 1024, 64, 8
ZIPF_S = 1.1
ZIPF_ALPHA = 0.33       # scale of the log-Zipf bias, calibrated so that busiest / mean ~ 4
ZIPF_PERM_SEED = 1234


def layer_weights(device, dtype=torch.float16, seed=0, experts=EXPERTS, hidden=HIDDEN, inter=INTER, std=0.02):
    """router [E,H], gate_up [E,2I,H], down [E,H,I] ~ N(0, std), generated on `device`."""
    g = torch.Generator(device=device).manual_seed(seed)
    router = (torch.randn(experts, hidden, device=device, generator=g) * std).to(dtype)
    gate_up = torch.empty(experts, 2 * inter, hidden, device=device, dtype=dtype)
    down = torch.empty(experts, hidden, inter, device=device, dtype=dtype)
    for e in range(experts):  # expert by expert: no float32 copy of the whole stack
        gate_up[e] = (torch.randn(2 * inter, hidden, device=device, generator=g) * std).to(dtype)
        down[e] = (torch.randn(hidden, inter, device=device, generator=g) * std).to(dtype)
    return router, gate_up, down


def hidden_states(tokens, device, dtype=torch.float16, seed=1, hidden=HIDDEN):
    g = torch.Generator(device=device).manual_seed(seed)
    return torch.randn(tokens, hidden, device=device, generator=g).to(dtype)


def zipf_bias(experts=EXPERTS, alpha=ZIPF_ALPHA, s=ZIPF_S, seed=ZIPF_PERM_SEED):
    """b_e = alpha * log(E * p_e), p_e ~ rank_e^-s over a seeded permutation of the experts.
    Added to the router logits (identically on every rank)."""
    g = torch.Generator().manual_seed(seed)
    rank = torch.randperm(experts, generator=g).double() + 1.0
    p = rank.pow(-s)
    p = p / p.sum()
    return (alpha * torch.log(experts * p)).float()


def biased_ops(mode, bias):
    """The expert-parallel operations with `bias` (float [E]) added to the router logits in the
    logits' dtype before the routing: how the benchmark applies the Zipf skew on every rank
    identically."""
    from .ep import CudaOps
    return CudaOps(mode, logit_bias=bias)


def busiest_over_mean(idx, experts=EXPERTS):
    counts = torch.bincount(idx.flatten().long().cpu(), minlength=experts).double()
    return (counts.max() / counts.mean()).item()
