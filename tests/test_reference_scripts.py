"""Drop-in check: the reference's OWN test scripts, unmodified, run against this library.

Each script does `import llaisys`; a two-line sitecustomize-style shim makes that name resolve to llaisys_b200.
Needs the reference tree, so it runs where that is mounted and is skipped elsewhere (the same cases are
restated in test_self_attention.py and test_tensor_runtime.py for machines without it)."""
import os
import subprocess
import sys
from pathlib import Path

import pytest

from tests import helpers

REFERENCE = helpers.reference_root()
ROOT = Path(__file__).resolve().parents[1]

SHIM = "import sys, llaisys_b200; sys.modules['llaisys'] = llaisys_b200; import runpy; " \
       "sys.argv = sys.argv[1:]; runpy.run_path(sys.argv[0], run_name='__main__')"

SCRIPTS = ["test/test_runtime.py", "test/test_tensor.py", "test/ops/add.py", "test/ops/self_attention.py",
           "test/ops/argmax.py", "test/ops/embedding.py", "test/ops/linear.py", "test/ops/rms_norm.py", "test/ops/rope.py",
           "test/ops/swiglu.py"]


def run_script(script: str, device: str):
    env = dict(os.environ, PYTHONPATH=f"{ROOT}:{REFERENCE / 'test'}")
    args = [sys.executable, "-c", SHIM, str(REFERENCE / script)]
    if "test_tensor" not in script:
        args += ["--device", device]
    return subprocess.run(args, env=env, capture_output=True, text=True, timeout=600)


@pytest.mark.skipif(REFERENCE is None, reason="reference tree not available (set LLAISYS_REFERENCE_ROOT)")
@pytest.mark.parametrize("script", SCRIPTS)
def test_reference_script_passes_on_cpu(script):
    res = run_script(script, "cpu")
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]
    assert "Test passed!" in res.stdout


@pytest.mark.skipif(REFERENCE is None, reason="reference tree not available (set LLAISYS_REFERENCE_ROOT)")
def test_reference_runtime_script_skips_nvidia_without_a_gpu():
    res = run_script("test/test_runtime.py", "nvidia")
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]
