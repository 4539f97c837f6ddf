"""A caller for the MoE path: an OLMoE decoder host in plain PyTorch, one process per GPU.

The reference's `model.py` / `serve.py` own the hook this package plugs into; they run
unchanged on top of `switchyard_b200.ep.ExpertParallel` wherever a reference checkout is
present. This module is the same caller written for the one-process-per-GPU runtime
(`ep_dist.DistributedExpertParallel`), so that the full-model decode benchmark can run where no
reference checkout exists: attention is data-parallel (every rank serves its own requests with
its own KV cache), the experts of every layer are split over the ranks.

It computes what the reference's model computes (switchyard/model.py:14-162: OLMoE with
float32 RMSNorm, QK-norm, rotary embeddings on half-split heads, left-padded batches, greedy
decoding) and has the same MoE hook `moe(layer, h) -> [B*T, H]` between attention and the
residual add (its `self.moe(i, h)`), but is laid out for a decode loop on one large GPU: the
three input projections of a layer are one GEMM over a fused weight, rotary factors come from a
table built once, the KV cache of all layers is one allocation, and attention itself (off the
measured path) is torch.nn.functional.scaled_dot_product_attention.

A decode step has fixed shapes (one new token per request, attention over the whole cache with
a validity mask, positions kept on the device), so `DecodeGraph` captures it - all layers,
attention and expert-parallel MoE alike - in one CUDA graph and replays it per token."""

import math
from dataclasses import dataclass

import torch
import torch.nn.functional as F


@dataclass
class Config:
    """Same fields as the reference's config (switchyard/config.py:8-24)."""
    vocab: int = 50304
    hidden: int = 2048
    intermediate: int = 1024
    layers: int = 16
    heads: int = 16
    kv_heads: int = 16
    head_dim: int = 128
    experts: int = 64
    top_k: int = 8
    norm_topk_prob: bool = False
    rms_eps: float = 1e-5
    rope_theta: float = 10000.0
    clip_qkv: float | None = None
    tie_embeddings: bool = False
    max_positions: int = 4096


def random_weights(c, device, dtype, seed=0, experts=None, std=0.02):
    """Random-init weights in the layout of the reference's loader (switchyard/weights.py:46-68):
    N(0, std) matrices, norm weights 1. The same seed gives the same model on every rank; a rank
    keeps only `experts` (a range) of every layer's expert stacks."""
    experts = range(c.experts) if experts is None else experts
    g = torch.Generator(device=device).manual_seed(seed)

    def mat(*shape):
        return (torch.randn(*shape, device=device, generator=g) * std).to(dtype)

    ones = lambda n: torch.ones(n, device=device, dtype=dtype)
    w = {"embed": mat(c.vocab, c.hidden), "final_norm": ones(c.hidden)}
    w["lm_head"] = w["embed"] if c.tie_embeddings else mat(c.vocab, c.hidden)
    qd, kd = c.heads * c.head_dim, c.kv_heads * c.head_dim
    layers = []
    for _ in range(c.layers):
        L = {"attn_norm": ones(c.hidden), "mlp_norm": ones(c.hidden), "wq": mat(qd, c.hidden), "wk": mat(kd, c.hidden),
             "wv": mat(kd, c.hidden), "wo": mat(c.hidden, qd), "q_norm": ones(qd), "k_norm": ones(kd),
             "router": mat(c.experts, c.hidden)}
        gu = torch.empty(len(experts), 2 * c.intermediate, c.hidden, device=device, dtype=dtype)
        dn = torch.empty(len(experts), c.hidden, c.intermediate, device=device, dtype=dtype)
        for e in range(c.experts):  # every expert advances the generator; only this rank's are kept
            a, b = mat(2 * c.intermediate, c.hidden), mat(c.hidden, c.intermediate)
            if e in experts:
                gu[e - experts[0]], dn[e - experts[0]] = a, b
        L["gate_up"], L["down"] = gu, dn
        layers.append(L)
    w["layers"] = layers
    w["experts"] = list(experts)
    return w


def from_hf_state_dict(sd, c, dtype=torch.float32, device="cpu"):
    """The same layout from a Hugging Face OlmoeForCausalLM state dict (tests compare against it)."""
    t = lambda k: sd[k].to(device=device, dtype=dtype)
    w = {"embed": t("model.embed_tokens.weight"), "final_norm": t("model.norm.weight")}
    w["lm_head"] = w["embed"] if c.tie_embeddings or "lm_head.weight" not in sd else t("lm_head.weight")
    layers = []
    for i in range(c.layers):
        p = f"model.layers.{i}."
        L = {"attn_norm": t(p + "input_layernorm.weight"), "mlp_norm": t(p + "post_attention_layernorm.weight"),
             "wq": t(p + "self_attn.q_proj.weight"), "wk": t(p + "self_attn.k_proj.weight"),
             "wv": t(p + "self_attn.v_proj.weight"), "wo": t(p + "self_attn.o_proj.weight"),
             "q_norm": t(p + "self_attn.q_norm.weight"), "k_norm": t(p + "self_attn.k_norm.weight"),
             "router": t(p + "mlp.gate.weight")}
        e = p + "mlp.experts."
        if e + "gate_up_proj" in sd:  # stacked layout of recent transformers
            L["gate_up"], L["down"] = t(e + "gate_up_proj"), t(e + "down_proj")
        else:
            L["gate_up"] = torch.stack([torch.cat([t(f"{e}{j}.gate_proj.weight"), t(f"{e}{j}.up_proj.weight")])
                                        for j in range(c.experts)])
            L["down"] = torch.stack([t(f"{e}{j}.down_proj.weight") for j in range(c.experts)])
        layers.append(L)
    w["layers"] = layers
    w["experts"] = list(range(c.experts))
    return w


def scaled_norm(x, weight, eps):
    """RMS normalisation computed in float32, result in x's dtype, times the learned scale."""
    return weight * F.rms_norm(x.float(), (x.shape[-1],), eps=eps).to(x.dtype)


class RotaryTable:
    """cos / sin of every position below `max_positions` for one head, in the model's dtype
    (the angles are computed in float32 and rounded once). Only the first half of a head's
    dimensions is stored: dimension j and j + head_dim/2 share an angle."""

    def __init__(self, head_dim, theta, max_positions, dtype, device):
        half = torch.arange(0, head_dim, 2, dtype=torch.float32, device=device) / head_dim
        angles = torch.arange(max_positions, dtype=torch.float32, device=device)[:, None] * (1.0 / theta ** half)[None]
        self.cos, self.sin = angles.cos().to(dtype), angles.sin().to(dtype)

    def at(self, positions):
        """positions [B, T] -> (cos, sin), each [B, 1, T, head_dim/2] (broadcast over heads)."""
        flat = positions.reshape(-1)
        shape = (*positions.shape, -1)
        return self.cos[flat].view(shape)[:, None], self.sin[flat].view(shape)[:, None]


def rotate(x, cos, sin):
    """Rotary embedding of x [B, heads, T, head_dim]: the pair (x[j], x[j + head_dim/2]) is
    turned by its position's angle."""
    lo, hi = x.chunk(2, dim=-1)
    return torch.cat([lo * cos - hi * sin, hi * cos + lo * sin], dim=-1)


class Cache:
    """Keys and values of all layers in one allocation, [layers, 2, B, kv_heads, capacity,
    head_dim] (`k[i]`, `v[i]` are views); `valid` marks real tokens (batches are left-padded);
    `next_pos` is each request's next rotary position and `length` the number of cache slots in
    use, both on the device so that a decode step can be replayed from a CUDA graph."""

    def __init__(self, c, batch, capacity, dtype, device):
        self.store = torch.zeros(c.layers, 2, batch, c.kv_heads, capacity, c.head_dim, dtype=dtype, device=device)
        self.k, self.v = list(self.store[:, 0]), list(self.store[:, 1])
        self.valid = torch.zeros(batch, capacity, dtype=torch.bool, device=device)
        self.next_pos = torch.zeros(batch, dtype=torch.int64, device=device)
        self.length = torch.zeros((), dtype=torch.int64, device=device)
        self.capacity = capacity


class Decoder:
    """OLMoE decoder with an MoE hook. moe(i, h): h [B*T, H] -> [B*T, H]. With
    moe_adds_residual=True the hook is moe(i, h, x) and returns x + layer(h) itself (x [B*T, H]
    contiguous: `kernels.moe_layer(..., residual=x)` does the addition in its combine launch)."""

    def __init__(self, config, weights, moe, moe_adds_residual=False):
        self.c, self.w, self.moe, self.moe_adds_residual = config, weights, moe, moe_adds_residual
        c = config
        embed = weights["embed"]
        self.rope = RotaryTable(c.head_dim, c.rope_theta, c.max_positions, embed.dtype, embed.device)
        # one GEMM for the three input projections of a layer, one norm for q and k
        self.wqkv = [torch.cat([L["wq"], L["wk"], L["wv"]]) for L in weights["layers"]]
        self.qd, self.kd = c.heads * c.head_dim, c.kv_heads * c.head_dim

    def _qkv(self, i, x, cos, sin):
        """Normed, rotated queries and keys and the values of layer i for x [B, T, H], each
        [B, heads, T, head_dim]."""
        c, L = self.c, self.w["layers"][i]
        B, T, _ = x.shape
        q, k, v = F.linear(x, self.wqkv[i]).split([self.qd, self.kd, self.kd], dim=-1)
        q, k = scaled_norm(q, L["q_norm"], c.rms_eps), scaled_norm(k, L["k_norm"], c.rms_eps)
        if c.clip_qkv is not None:
            q, k, v = (t.clamp(-c.clip_qkv, c.clip_qkv) for t in (q, k, v))
        heads = lambda t, n: t.reshape(B, T, n, c.head_dim).transpose(1, 2)
        return rotate(heads(q, c.heads), cos, sin), rotate(heads(k, c.kv_heads), cos, sin), heads(v, c.kv_heads)

    def _after_moe(self, i, h, x):
        """x + moe layer i of h, for x [B, T, H] and h [B*T, H]."""
        if self.moe_adds_residual:
            return self.moe(i, h, x.reshape(h.shape).contiguous()).view(x.shape)
        return x + self.moe(i, h).view(x.shape)

    def _attend(self, L, q, k, v, mask):
        c = self.c
        B, _, T, _ = q.shape
        a = F.scaled_dot_product_attention(q, k, v, attn_mask=mask[:, None], enable_gqa=c.kv_heads != c.heads)
        return F.linear(a.transpose(1, 2).reshape(B, T, c.heads * c.head_dim), L["wo"])

    # ---- prefill / general forward (shapes depend on the call)
    @torch.no_grad()
    def forward(self, tokens, cache=None, valid=None):
        """tokens [B,T]; valid [B,T] marks real tokens (False = left padding). With a cache the
        tokens are appended after what it holds. Returns logits [B,T,vocab]."""
        c, W = self.c, self.w
        B, T = tokens.shape
        dev = tokens.device
        if valid is None:
            valid = torch.ones(B, T, dtype=torch.bool, device=dev)
        start = int(cache.length) if cache is not None else 0
        base = cache.next_pos if cache is not None else torch.zeros(B, dtype=torch.int64, device=dev)
        positions = (base[:, None] + torch.cumsum(valid.long(), 1) - 1).clamp(min=0)
        if cache is not None:
            cache.valid[:, start:start + T] = valid
            keys_valid = cache.valid[:, :start + T]
        else:
            keys_valid = valid
        causal = torch.ones(T, start + T, dtype=torch.bool, device=dev).tril(start)
        mask = causal[None] & keys_valid[:, None, :]
        diag = torch.zeros(T, start + T, dtype=torch.bool, device=dev)
        diag[torch.arange(T, device=dev), start + torch.arange(T, device=dev)] = True
        mask = mask | (~mask.any(-1, keepdim=True) & diag[None])  # a padding query attends to itself
        cos, sin = self.rope.at(positions)
        x = F.embedding(tokens, W["embed"])
        for i, L in enumerate(W["layers"]):
            q, k, v = self._qkv(i, scaled_norm(x, L["attn_norm"], c.rms_eps), cos, sin)
            if cache is not None:
                cache.k[i][:, :, start:start + T] = k
                cache.v[i][:, :, start:start + T] = v
                k, v = cache.k[i][:, :, :start + T], cache.v[i][:, :, :start + T]
            x = x + self._attend(L, q, k, v, mask)
            h = scaled_norm(x, L["mlp_norm"], c.rms_eps).reshape(B * T, -1)
            x = self._after_moe(i, h, x)
        if cache is not None:
            cache.length += T
            cache.next_pos += valid.long().sum(1)
        return F.linear(scaled_norm(x, W["final_norm"], c.rms_eps), W["lm_head"])

    # ---- one decode step with fixed shapes (CUDA-graph capturable)
    @torch.no_grad()
    def decode_step(self, tokens, cache):
        """tokens [B] (one new token per request). Attends over the whole cache under the
        validity mask; writes the new keys/values at slot cache.length. Returns logits [B,vocab]."""
        c, W = self.c, self.w
        B = tokens.shape[0]
        slot = cache.length
        onehot = torch.arange(cache.capacity, device=tokens.device) == slot          # [capacity]
        cache.valid.logical_or_(onehot[None])
        mask = cache.valid[:, None, :]                                                 # [B,1,capacity]
        cos, sin = self.rope.at(cache.next_pos[:, None])
        x = F.embedding(tokens[:, None], W["embed"])
        at = slot.view(1)  # device index: the step stays replayable
        for i, L in enumerate(W["layers"]):
            q, k, v = self._qkv(i, scaled_norm(x, L["attn_norm"], c.rms_eps), cos, sin)
            cache.k[i].index_copy_(2, at, k)
            cache.v[i].index_copy_(2, at, v)
            x = x + self._attend(L, q, cache.k[i], cache.v[i], mask)
            h = scaled_norm(x, L["mlp_norm"], c.rms_eps).reshape(B, -1)
            x = self._after_moe(i, h, x)
        cache.length += 1
        cache.next_pos += 1
        return F.linear(scaled_norm(x, W["final_norm"], c.rms_eps), W["lm_head"])[:, 0]

    @torch.no_grad()
    def generate(self, prompts, max_new_tokens, graph=False, marks=None, session=None):
        """Greedy decoding of a batch of token lists (left-padded internally); returns the new
        tokens per prompt. graph=True replays the decode step from a CUDA graph; pass a `Session`
        to keep the cache and the captured graph across calls of the same batch size. marks:
        optional list that receives ("prefill_done", t) and ("decode_done", t), time.perf_counter()
        values taken after the device has finished."""
        import time
        dev, dtype = self.w["embed"].device, self.w["embed"].dtype
        B, P = len(prompts), max(len(p) for p in prompts)
        tokens = torch.zeros(B, P, dtype=torch.int64, device=dev)
        valid = torch.zeros(B, P, dtype=torch.bool, device=dev)
        for b, p in enumerate(prompts):
            tokens[b, P - len(p):] = torch.tensor(p, device=dev)
            valid[b, P - len(p):] = True
        if session is None:
            session = Session(self, B, P + max_new_tokens)
        session.reset()
        cache = session.cache
        assert cache.k[0].shape[0] == B and cache.capacity >= P + max_new_tokens
        nxt = self.forward(tokens, cache, valid)[:, -1].argmax(-1)
        out = [nxt]
        if marks is not None:
            if dev.type == "cuda":
                torch.cuda.synchronize()
            marks.append(("prefill_done", time.perf_counter()))
        for _ in range(max_new_tokens - 1):
            logits = session.step(nxt) if graph and dev.type == "cuda" else self.decode_step(nxt, cache)
            nxt = logits.argmax(-1)
            out.append(nxt)
        result = torch.stack(out, 1).tolist()  # one transfer; also waits for the device
        if dev.type == "cuda":
            # a kernel of this request that gave up on a bounded wait (a peer that never arrived)
            # has left garbage behind: raise instead of returning its tokens
            from . import kernels
            kernels.ext().check_device(dev)
        if marks is not None:
            marks.append(("decode_done", time.perf_counter()))
        return result


class Session:
    """A KV cache of fixed batch and capacity plus the decode step captured over it in a CUDA
    graph (all layers: attention and MoE). Reused across generate() calls; every rank of an
    expert-parallel group must create, capture and replay in lockstep."""

    def __init__(self, decoder, batch, capacity):
        w = decoder.w["embed"]
        self.decoder = decoder
        self.cache = Cache(decoder.c, batch, capacity, w.dtype, w.device)
        self.tokens = torch.zeros(batch, dtype=torch.int64, device=w.device)
        self.graph, self.logits, self.warm = None, None, False

    def reset(self):
        c = self.cache
        c.valid.zero_()  # stale keys and values stay but are masked out
        c.next_pos.zero_()
        c.length.zero_()

    def step(self, tokens):
        self.tokens.copy_(tokens)
        if self.graph is None:
            if not self.warm:  # the first step runs eagerly (it warms every library up)
                self.warm = True
                return self.decoder.decode_step(self.tokens, self.cache)
            torch.cuda.synchronize()
            self.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph):
                self.logits = self.decoder.decode_step(self.tokens, self.cache)
        self.graph.replay()  # (capture does not execute: the replay is the step)
        return self.logits
