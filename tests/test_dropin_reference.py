"""Drop-in check against the reference's own callers: its unmodified `serve.ParallelModel` and
`model.Model` (the owners of the `self.moe(layer, h)` hook) run on top of THIS package's
`ExpertParallel`, and generate exactly what the reference's single model generates. Runs on the
CPU with the protocol operations injected from the oracle; skipped where no reference checkout
sits next to the repository (set SWITCHYARD_REFERENCE to point at one)."""

import os
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = next((c for c in (os.environ.get("SWITCHYARD_REFERENCE"), os.path.join(os.path.dirname(ROOT), "reference"),
                        os.path.join(ROOT, "baseline", "_ref"))
            if c and os.path.exists(os.path.join(c, "switchyard", "serve.py"))), None)

pytestmark = pytest.mark.skipif(REF is None, reason="no reference checkout available")


@pytest.fixture(scope="module")
def ref():
    pytest.importorskip("transformers")
    sys.path.insert(0, REF)
    sys.path.insert(0, os.path.join(REF, "tests"))
    import switchyard.serve as serve
    import switchyard.model as model
    import switchyard.weights as weights
    import switchyard.config as config
    import tiny
    yield dict(serve=serve, model=model, weights=weights, config=config, tiny=tiny)
    sys.path.remove(REF)
    sys.path.remove(os.path.join(REF, "tests"))


def test_reference_serving_runs_unchanged_on_this_expert_parallel(ref, monkeypatch):
    from oracle.ep_oracle import TorchOps
    from switchyard_b200 import ep
    monkeypatch.setattr(ref["serve"], "ExpertParallel", ep.ExpertParallel)
    path, _ = ref["tiny"].checkpoint(experts=16, top_k=4)
    c = ref["config"].Config.load(path)
    one = ref["model"].Model(c, ref["weights"].load(path, c))
    two = ref["serve"].ParallelModel(path, ["cpu", "cpu"], dtype=torch.float32, ops=TorchOps())
    assert isinstance(two.ep, ep.ExpertParallel)
    prompts = ref["tiny"].prompts(5, seed=11)
    assert two.generate(prompts, 8) == one.generate(prompts, 8)
    toks = [torch.tensor([p[:7]]) for p in prompts[:2]]
    a, b = two.forward(toks, threaded=True), two.forward(toks, threaded=False)
    assert all(torch.equal(x, y) for x, y in zip(a, b))


def test_reference_model_hook_accepts_this_layer(ref):
    """Model(config, weights, moe=...) with a hook built from this package's API shape (here
    with the oracle's CPU math standing in for the kernels) equals the reference's own layer."""
    from oracle import ep_oracle as eo
    path, _ = ref["tiny"].checkpoint(experts=8, top_k=2)
    c = ref["config"].Config.load(path)
    w = ref["weights"].load(path, c)

    def moe(i, h):
        L = w["layers"][i]
        return eo.single_device_layer(h, L["router"], L["gate_up"], L["down"], c.top_k, c.norm_topk_prob)

    hooked, plain = ref["model"].Model(c, w, moe=moe), ref["model"].Model(c, w)
    t = torch.tensor([ref["tiny"].prompts(1, seed=3)[0][:9]])
    assert (hooked.forward(t) - plain.forward(t)).abs().max().item() < 1e-5
