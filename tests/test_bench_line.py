"""The reference arm of bench.py (`--impl reference`: the reference's float32 expert loop on the
host cores) prints one JSON line with the contract's keys and the same `config` object as the
GPU arm, so that the two arms can be compared field by field."""

import io
import json
import os
import sys
from contextlib import redirect_stdout
from types import SimpleNamespace

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_prints_the_contract_line():
    sys.path.insert(0, ROOT)
    import bench
    out = io.StringIO()
    with redirect_stdout(out):
        bench.run_reference(SimpleNamespace(steps=1, warmup=0, gpus=1))
    line = json.loads(out.getvalue().strip().splitlines()[-1])
    for key in ("impl", "metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better",
                "scaling", "vs_baseline", "dtype", "data", "config", "cpu_baseline", "e2e"):
        assert key in line, key
    assert line["impl"] == "reference" and line["metric"] == bench.METRIC and line["unit"] == bench.UNIT
    assert line["config"] == bench.CONFIG  # the GPU arm prints this very object
    assert line["value"] > 0 and line["e2e"]["value"] == line["value"]
    assert line["e2e"]["h2d_bytes_per_step"] == 0 and line["e2e"]["d2h_bytes_per_step"] == 0
    assert line["cpu_baseline"]["kind"] in ("reference", "port") and line["cpu_baseline"]["cores"] >= 1
