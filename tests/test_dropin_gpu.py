"""Drop-in on the GPU with the reference's own, unmodified callers: its `model.Model` takes this
package's layer through the `moe=` hook (switchyard/model.py:39-42,135), and its
`serve.ParallelModel` runs on this package's `ExpertParallel` (switchyard/serve.py:13-110), the
cases of the reference's tests/test_ep_cuda.py:62-86. The reference is imported from a checkout:
SWITCHYARD_REFERENCE, `../reference`, or the copy that `python tests/fetch_reference.py` puts into
the git-ignored `baseline/_ref/` (which is how it reaches a machine without a checkout). Skipped
when there is none."""

import os
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

pytestmark = pytest.mark.gpu


def find_reference():
    for cand in (os.environ.get("SWITCHYARD_REFERENCE"), os.path.join(os.path.dirname(ROOT), "reference"),
                 os.path.join(ROOT, "baseline", "_ref")):
        if cand and os.path.exists(os.path.join(cand, "switchyard", "serve.py")):
            return cand
    return None


REF = find_reference()


def n_gpus():
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


@pytest.fixture(scope="module")
def ref():
    if REF is None:
        pytest.skip("no reference checkout available (python tests/fetch_reference.py <path>)")
    pytest.importorskip("transformers")
    sys.path.insert(0, REF)
    sys.path.insert(0, os.path.join(REF, "tests"))
    import switchyard.config as config
    import switchyard.model as model
    import switchyard.serve as serve
    import switchyard.weights as weights
    import tiny
    from switchyard_b200 import ep
    original = serve.ExpertParallel
    serve.ExpertParallel = ep.ExpertParallel  # the one line a maintainer changes: which ep module serve imports
    yield dict(serve=serve, model=model, weights=weights, config=config, tiny=tiny)
    serve.ExpertParallel = original
    sys.path.remove(REF)
    sys.path.remove(os.path.join(REF, "tests"))


@pytest.mark.parametrize("experts,top_k,norm", [(8, 2, False), (16, 4, True)])
def test_reference_model_runs_on_this_layer_through_its_hook(ref, experts, top_k, norm):
    """Model(config, weights, moe=<this package's moe_layer>) in fp16 on the GPU against the
    reference's own float32 model on the CPU; the yardstick is the reference's own fp16 GPU model
    (its PyTorch expert loop): the hooked model may be at most twice as far from float32."""
    from switchyard_b200 import kernels
    path, _ = ref["tiny"].checkpoint(experts=experts, top_k=top_k, norm_topk_prob=norm)
    c = ref["config"].Config.load(path)
    exact = ref["model"].Model(c, ref["weights"].load(path, c))
    w16 = ref["weights"].load(path, c, dtype=torch.float16, device=torch.device("cuda:0"))
    plain16 = ref["model"].Model(c, w16)

    def moe(i, h):
        L = w16["layers"][i]
        return kernels.moe_layer(h, L["router"], L["gate_up"], L["down"], c.top_k, c.norm_topk_prob)

    hooked = ref["model"].Model(c, w16, moe=moe)
    for seed, n in ((3, 9), (4, 23)):
        t = torch.tensor([ref["tiny"].prompts(1, seed=seed)[0][:n]])
        want = exact.forward(t)
        got = hooked.forward(t.cuda()).float().cpu()
        yard = plain16.forward(t.cuda()).float().cpu()
        err, err16 = (got - want).abs().max().item(), (yard - want).abs().max().item()
        assert err <= max(2 * err16, 2e-2), (err, err16)
    assert kernels.ext().device_status("cuda:0") == 0


def _threaded_generate_matches(ref, devices):
    path, _ = ref["tiny"].checkpoint(experts=16, top_k=4, layers=6)
    pm = ref["serve"].ParallelModel(path, devices, dtype=torch.float16)
    from switchyard_b200 import ep, kernels
    assert isinstance(pm.ep, ep.ExpertParallel) and pm.ep.windows
    ps = ref["tiny"].prompts(8, seed=5)
    pm.threaded = False
    want = pm.generate(ps, 24)
    pm.threaded = True
    for _ in range(3):
        assert pm.generate(ps, 24) == want
    pm.ep.check()
    total = pm.ep.stats
    assert total["dispatched_rows"] + total["local_rows"] > 0
    return pm


def test_reference_serving_threaded_equals_one_thread_on_one_gpu(ref):
    _threaded_generate_matches(ref, ["cuda:0", "cuda:0"])


@pytest.mark.skipif(n_gpus() < 2, reason="needs two GPUs")
def test_reference_serving_threaded_equals_one_thread_on_two_gpus(ref):
    pm = _threaded_generate_matches(ref, ["cuda:0", "cuda:1"])
    assert not pm.ep.host_ordered  # flags on the device: no events, no barriers
    assert pm.ep.stats["dispatched_rows"] > 0


def test_served_tokens_equal_the_single_model(ref):
    """Two ranks on one GPU generate what the reference's single fp16 model generates with this
    package's layer in its hook (same kernels, same mode: expert parallelism changes no bits)."""
    from switchyard_b200 import kernels
    from switchyard_b200.ep import CudaOps
    path, _ = ref["tiny"].checkpoint(experts=16, top_k=4)
    c = ref["config"].Config.load(path)
    w16 = ref["weights"].load(path, c, dtype=torch.float16, device=torch.device("cuda:0"))

    def moe(i, h):
        L = w16["layers"][i]
        return kernels.moe_layer(h, L["router"], L["gate_up"], L["down"], c.top_k, c.norm_topk_prob, "gemv")

    one = ref["model"].Model(c, w16, moe=moe)
    two = ref["serve"].ParallelModel(path, ["cuda:0", "cuda:0"], dtype=torch.float16, ops=CudaOps("gemv"))
    prompts = ref["tiny"].prompts(2, seed=11)
    # one request per rank, so that every rank's batch is what the single model sees for that request
    for p, got in zip(prompts, two.generate(prompts, 8)):
        assert got == one.generate([p], 8)[0]
