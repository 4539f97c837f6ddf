"""The decoder host (switchyard_b200.olmoe) against Hugging Face transformers' OlmoeForCausalLM on
tiny random models, on the CPU with the oracle's MoE math as the hook: full forward, forward
with a cache, fixed-shape decode steps, left padding, greedy generation. (The reference pins
its own model the same way, tests/test_model.py:11-34,60-83.)"""

import pytest
import torch

from oracle import ep_oracle as eo

transformers = pytest.importorskip("transformers")


def tiny(experts=8, top_k=2, heads=4, kv_heads=4, layers=2, seed=0):
    from transformers import OlmoeConfig, OlmoeForCausalLM
    from switchyard_b200 import olmoe
    torch.manual_seed(seed)
    cfg = OlmoeConfig(vocab_size=131, hidden_size=64, intermediate_size=32, num_hidden_layers=layers,
                      num_attention_heads=heads, num_key_value_heads=kv_heads, num_experts=experts,
                      num_experts_per_tok=top_k, norm_topk_prob=False, max_position_embeddings=256,
                      eos_token_id=1, pad_token_id=0, bos_token_id=2)
    hf = OlmoeForCausalLM(cfg).eval()
    with torch.no_grad():
        for name, p in hf.named_parameters():
            if "norm" in name:
                p.copy_(1.0 + 0.1 * torch.randn_like(p))
            elif "gate.weight" in name:
                p.normal_(0, 1.0)
            else:
                p.normal_(0, 0.08)
    c = olmoe.Config(vocab=131, hidden=64, intermediate=32, layers=layers, heads=heads, kv_heads=kv_heads,
                     head_dim=64 // heads, experts=experts, top_k=top_k, rms_eps=cfg.rms_norm_eps,
                     rope_theta=getattr(cfg, "rope_theta", None) or (cfg.rope_parameters or {}).get("rope_theta", 10000.0),
                     max_positions=256)
    w = olmoe.from_hf_state_dict(hf.state_dict(), c)

    def moe(i, h):
        L = w["layers"][i]
        return eo.single_device_layer(h, L["router"], L["gate_up"], L["down"], c.top_k, c.norm_topk_prob)

    return hf, olmoe.Decoder(c, w, moe), olmoe


@pytest.mark.parametrize("kv_heads", [4, 2])
def test_logits_match_transformers(kv_heads):
    hf, dec, _ = tiny(kv_heads=kv_heads)
    g = torch.Generator().manual_seed(1)
    t = torch.randint(3, 131, (2, 11), generator=g)
    with torch.no_grad():
        want = hf(t).logits
    assert (dec.forward(t) - want).abs().max().item() < 1e-4


def test_cache_and_fixed_shape_decode_steps_match_the_full_forward():
    hf, dec, olmoe = tiny()
    g = torch.Generator().manual_seed(2)
    t = torch.randint(3, 131, (3, 9), generator=g)
    full = dec.forward(t)
    cache = olmoe.Cache(dec.c, 3, 16, torch.float32, "cpu")
    first = dec.forward(t[:, :5], cache)
    assert (first - full[:, :5]).abs().max().item() < 1e-5
    for j in range(5, 9):
        step = dec.decode_step(t[:, j], cache)
        assert (step - full[:, j]).abs().max().item() < 1e-5


def test_greedy_generation_matches_transformers_with_left_padding():
    hf, dec, _ = tiny(experts=16, top_k=4)
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(3, 131, (n,), generator=g).tolist() for n in (7, 12, 9)]
    got = dec.generate(prompts, 6)
    for p, mine in zip(prompts, got):
        with torch.no_grad():
            out = hf.generate(torch.tensor([p]), max_new_tokens=6, do_sample=False, min_new_tokens=6)
        assert out[0, len(p):].tolist() == mine


def test_random_weights_are_the_same_on_every_rank():
    from switchyard_b200 import olmoe
    c = olmoe.Config(vocab=50, hidden=32, intermediate=16, layers=2, heads=2, kv_heads=2, head_dim=16, experts=8, top_k=2)
    full = olmoe.random_weights(c, "cpu", torch.float32, seed=5)
    part = olmoe.random_weights(c, "cpu", torch.float32, seed=5, experts=range(4, 8))
    assert torch.equal(full["embed"], part["embed"]) and torch.equal(full["layers"][1]["wq"], part["layers"][1]["wq"])
    assert torch.equal(full["layers"][1]["gate_up"][4:], part["layers"][1]["gate_up"])
    assert torch.equal(full["layers"][0]["down"][4:], part["layers"][0]["down"])


def test_a_hook_that_adds_the_residual_itself_gives_the_same_model():
    hf, dec, olmoe = tiny()
    dec2 = olmoe.Decoder(dec.c, dec.w, lambda i, h, x: x + dec.moe(i, h), moe_adds_residual=True)
    t = torch.randint(3, 131, (2, 7), generator=torch.Generator().manual_seed(4))
    assert torch.equal(dec2.forward(t), dec.forward(t))
    cache, cache2 = (olmoe.Cache(dec.c, 2, 12, torch.float32, "cpu") for _ in range(2))
    dec.forward(t[:, :6], cache), dec2.forward(t[:, :6], cache2)
    assert torch.equal(dec2.decode_step(t[:, 6], cache2), dec.decode_step(t[:, 6], cache))
