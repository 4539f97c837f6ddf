"""Generates the golden fixtures in this directory by running the UNMODIFIED reference
implementation (its `switchyard.moe` and `switchyard.ep` modules, imported from a checkout
given as argv[1]) on seeded CPU inputs. The fixtures are what the oracle and the CUDA kernels
are pinned against on machines where the reference checkout is not present.

    python tests/golden/make_golden.py /path/to/reference/checkout

Inputs are regenerated from seeds by `tests/cases.py`; a checksum of every regenerated input
is stored next to the outputs so that a change in the random stream is detected rather than
silently compared against.
"""

import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))          # tests/
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))  # repo root

import cases  # noqa: E402


def main(ref_root):
    sys.path.insert(0, ref_root)
    from switchyard import moe
    from switchyard.ep import ExpertParallel, TorchOps

    torch.set_num_threads(1)  # one thread: CPU float sums in a fixed order
    out = {}

    # ---- routing: reference softmax+topk on fixed fp16 logits (identity router keeps them)
    for name, (E, k, N) in cases.ROUTE_CASES.items():
        logits = cases.route_logits(E, N)
        out[f"route/{name}/logits_sum"] = cases.checksum(logits)
        for norm in (False, True):
            idx, w = moe.route(logits, torch.eye(E, dtype=logits.dtype), k, norm)
            out[f"route/{name}/norm{int(norm)}/idx"] = idx.numpy().astype(np.int32)
            out[f"route/{name}/norm{int(norm)}/w"] = w.numpy()

    # ---- sort: the reference's TorchOps.sort (moe.plan + pos_of)
    for name, (E, k, N, seed) in cases.SORT_CASES.items():
        idx, w = cases.sort_inputs(E, k, N, seed)
        out[f"sort/{name}/in_sum"] = cases.checksum(idx.float()) + cases.checksum(w)
        c, o, t, ws, p = TorchOps().sort(idx, w, E)
        pl = moe.plan(idx.long(), w, E)
        for key, val in dict(counts=c, offsets=o, token=t, wsorted=ws, pos_of=p, slot=pl.slot.int()).items():
            out[f"sort/{name}/{key}"] = val.numpy()

    # ---- experts: fp32 loop, grouped, and the 16-bit loop (tolerance baseline)
    for name, spec in cases.LAYER_CASES.items():
        h, router, gu, dn = cases.layer_inputs(**spec)
        k = spec["k"]
        out[f"layer/{name}/in_sum"] = sum(cases.checksum(t) for t in (h, router, gu, dn))
        ridx, rw = moe.route(h, router, k, False)
        want = moe.experts_reference(h.float(), ridx, rw.float(), gu.float(), dn.float())
        grouped = moe.experts_grouped(h.float(), ridx, rw.float(), gu.float(), dn.float())
        half = moe.experts_reference(h, ridx, rw, gu, dn)
        assert torch.equal(want, grouped)
        out[f"layer/{name}/ridx"] = ridx.numpy().astype(np.int32)
        out[f"layer/{name}/rw"] = cases.to_np(rw)
        out[f"layer/{name}/want_fp32"] = want.numpy()
        out[f"layer/{name}/loop16"] = cases.to_np(half)

    # ---- expert parallel on CPU ranks: outputs, stats and the inbox placement
    for name, (R, sizes) in cases.EP_CASES.items():
        router, gu, dn, hs = cases.ep_inputs(R, sizes)
        E, k = cases.EP_E, cases.EP_K
        per = E // R
        ep = ExpertParallel(["cpu"] * R, E, k, False)
        sh = ep.new_state()
        for r in range(R):
            ep.phase_send(sh, r, hs[r], router)
        for d in range(R):
            for r in range(R):
                m = sh["inbox"][d][r]
                if m is None:
                    continue
                pre = f"ep/{name}/inbox/{d}/{r}"
                out[pre + "/x"] = m["x"].numpy()
                out[pre + "/offsets"] = m["offsets"].numpy()
                out[pre + "/counts"] = m["counts"].numpy()
                out[pre + "/w"] = m["w"].numpy()
        for d in range(R):
            ep.phase_compute(sh, d, hs[d], gu[d * per:(d + 1) * per], dn[d * per:(d + 1) * per])
        for r in range(R):
            out[f"ep/{name}/out/{r}"] = ep.phase_combine(sh, r, hs[r].shape[0]).numpy()
            out[f"ep/{name}/seg/{r}"] = np.array(sh["st"][r]["seg"], dtype=np.int32)
        out[f"ep/{name}/dispatched_rows"] = np.int64(ep.stats["dispatched_rows"])
        out[f"ep/{name}/local_rows"] = np.int64(ep.stats["local_rows"])

    # ---- capacity drop
    for cf in cases.CAPACITY_FACTORS:
        router, gu, dn, hs = cases.capacity_inputs()
        E, k, R = cases.EP_E, cases.EP_K, 2
        per = E // R
        ep = ExpertParallel(["cpu"] * R, E, k, False)
        ep.capacity_factor = cf
        outs = ep.layer(hs, [router] * R, [gu[r * per:(r + 1) * per] for r in range(R)],
                        [dn[r * per:(r + 1) * per] for r in range(R)])
        for r, o in enumerate(outs):
            out[f"cap/{cf}/out/{r}"] = o.numpy()
        out[f"cap/{cf}/dropped"] = np.int64(ep.stats["dropped_rows"])
        out[f"cap/{cf}/routed"] = np.int64(ep.stats["routed_rows"])

    path = os.path.join(HERE, "reference_vectors.npz")
    np.savez_compressed(path, **out)
    print(f"wrote {path}: {len(out)} arrays, {os.path.getsize(path) / 1024:.0f} KiB")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: make_golden.py <reference checkout>")
    main(sys.argv[1])
