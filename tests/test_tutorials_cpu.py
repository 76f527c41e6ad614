"""The tutorial scripts under docs/tutorials run to completion on CPU (they assert their own
numerics)."""
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("name,marker", [
    ("quick_start", "quick start finished"),
    ("attention_single_gpu", "attention tutorial finished"),
    ("debug_print", "debugging tutorial finished"),
    ("mlp_multi_gpu", "multi-device tutorial finished"),
])
def test_tutorial_runs(name, marker):
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="", OMP_NUM_THREADS="2")
    res = subprocess.run([sys.executable, os.path.join(ROOT, "docs", "tutorials", f"{name}.py")],
                         capture_output=True, text=True, timeout=600, env=env, cwd=ROOT)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]
    assert marker in res.stdout


def test_api_page_is_up_to_date():
    """docs/python_api.md is generated from the docstrings (python docs/gen_api.py)."""
    import os
    import subprocess
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    res = subprocess.run([sys.executable, os.path.join(root, "docs", "gen_api.py"), "--check"],
                         capture_output=True, text=True)
    assert res.returncode == 0, "run `python docs/gen_api.py` and commit docs/python_api.md"
