"""The multi-GPU test cases guard themselves: every test that starts N > 1 ranks through `run(N, …)`
carries a skip mark for boxes with fewer than N GPUs (a rank that cannot get a device would leave
the others waiting for it), and every GPU test file is marked `gpu` as a whole."""

import ast
import os
import re

HERE = os.path.dirname(os.path.abspath(__file__))


def _tests(path):
    src = open(path).read()
    for node in ast.parse(src).body:
        if isinstance(node, ast.FunctionDef) and node.name.startswith("test"):
            yield node.name, [ast.get_source_segment(src, d) for d in node.decorator_list], ast.get_source_segment(src, node)


def test_every_multi_rank_case_is_skipped_without_its_gpus():
    checked = 0
    for name, decorators, body in _tests(os.path.join(HERE, "test_ep_dist_gpu.py")):
        worlds = [int(n) for n in re.findall(r"\brun\((\d+),", body)]
        if worlds and max(worlds) > 1:
            checked += 1
            assert any("skipif" in d and f"n_gpus() < {max(worlds)}" in d for d in decorators), name
    assert checked >= 6


def test_gpu_test_files_are_marked_as_a_whole():
    for f in sorted(os.listdir(HERE)):
        if f.endswith("_gpu.py"):
            assert re.search(r"^pytestmark = pytest\.mark\.gpu", open(os.path.join(HERE, f)).read(), re.M), f
