"""The decoder host on the GPU: the decode step replayed from a CUDA graph (all layers, attention
and this package's MoE layer in its hook) gives the bits of the same step run eagerly, and the
fp16 model stays close to the same model in float32 on the CPU with the oracle's MoE math."""

import pytest
import torch

import cases
from oracle import ep_oracle as eo

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def build(dtype, device, moe_of):
    from switchyard_b200 import olmoe
    c = olmoe.Config(vocab=211, hidden=256, intermediate=128, layers=3, heads=4, kv_heads=2, head_dim=64, experts=16,
                     top_k=4, max_positions=128)
    w = olmoe.random_weights(c, device, dtype, seed=3, std=0.06)
    return c, w, olmoe.Decoder(c, w, moe_of(c, w)), olmoe


def kernel_hook(c, w):
    from switchyard_b200 import kernels
    return lambda i, h: kernels.moe_layer(h, w["layers"][i]["router"], w["layers"][i]["gate_up"], w["layers"][i]["down"],
                                          c.top_k, c.norm_topk_prob, "gemv")


def test_graph_replay_equals_the_eager_decode_step():
    from switchyard_b200 import kernels
    c, w, dec, olmoe = build(torch.float16, DEV, kernel_hook)
    g = cases.gen(5)
    prompts = [torch.randint(3, c.vocab, (n,), generator=g).tolist() for n in (9, 14, 6)]
    eager = dec.generate(prompts, 12, graph=False)
    session = olmoe.Session(dec, 3, 14 + 12)
    for _ in range(2):  # the second call replays the graph captured by the first
        assert dec.generate(prompts, 12, graph=True, session=session) == eager
    assert session.graph is not None
    # step by step: logits of a replayed step are the eager step's logits, bit for bit
    a, b = olmoe.Session(dec, 3, 32), olmoe.Session(dec, 3, 32)
    toks = torch.randint(3, c.vocab, (3, 6), generator=g).to(DEV)
    dec.forward(toks, a.cache)
    dec.forward(toks, b.cache)
    nxt = torch.randint(3, c.vocab, (3,), generator=g).to(DEV)
    for _ in range(5):
        want = dec.decode_step(nxt.clone(), a.cache)
        got = b.step(nxt)
        assert torch.equal(got, want)
        nxt = want.argmax(-1)
    assert kernels.ext().device_status(DEV) == 0


def test_residual_added_in_the_combine_gives_the_same_logits():
    """Decoder(moe_adds_residual=True) hands x to the hook; moe_layer(residual=x) adds it in its
    combine launch with the bits of the separate addition, so the whole model's logits agree."""
    from switchyard_b200 import kernels
    c, w, dec, olmoe = build(torch.float16, DEV, kernel_hook)
    hook = lambda i, h, x: kernels.moe_layer(h, w["layers"][i]["router"], w["layers"][i]["gate_up"],
                                             w["layers"][i]["down"], c.top_k, c.norm_topk_prob, "gemv", residual=x)
    dec2 = olmoe.Decoder(c, w, hook, moe_adds_residual=True)
    toks = torch.randint(3, c.vocab, (3, 11), generator=cases.gen(8)).to(DEV)
    assert torch.equal(dec2.forward(toks), dec.forward(toks))
    prompts = [torch.randint(3, c.vocab, (n,), generator=cases.gen(9)).tolist() for n in (5, 8)]
    assert dec2.generate(prompts, 6, graph=False) == dec.generate(prompts, 6, graph=False)


def test_fp16_model_on_the_gpu_is_close_to_float32_on_the_cpu():
    c, w16, dec16, olmoe = build(torch.float16, DEV, kernel_hook)
    w32 = {k: (v.float().cpu() if torch.is_tensor(v) else v) for k, v in w16.items() if k != "layers"}
    w32["layers"] = [{k: v.float().cpu() for k, v in L.items()} for L in w16["layers"]]
    oracle_hook = lambda i, h: eo.single_device_layer(h, w32["layers"][i]["router"], w32["layers"][i]["gate_up"],
                                                      w32["layers"][i]["down"], c.top_k, c.norm_topk_prob)
    dec32 = olmoe.Decoder(c, w32, oracle_hook)
    t = torch.randint(3, c.vocab, (2, 17), generator=cases.gen(8))
    want = dec32.forward(t)
    got = dec16.forward(t.to(DEV)).float().cpu()
    rel = ((got - want).norm() / want.norm()).item()
    assert rel < 2e-2, rel
