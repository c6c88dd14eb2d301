"""The ggml-shaped callbacks (include/dc_ggml_compat.h) driven by a C++ host program the way ggml's executor
drives DenseCore's own callbacks (core/src/llm/matmul/graph_ops.cpp:212-227): fake custom-op nodes, four host
threads per call, results against the CPU oracle, and the fail-closed contract on bad nodes."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
pytestmark = pytest.mark.gpu


def test_ggml_shaped_callbacks_from_four_host_threads():
    exe = os.path.join(ROOT, "tests", "shims", "ggml_shims_test")
    if not os.path.exists(exe):
        from oracle import oracle as o
        o.build()
        subprocess.check_call(["make", "-C", os.path.dirname(exe), "ggml_shims_test"], stdout=subprocess.DEVNULL)
    r = subprocess.run([exe], capture_output=True, text=True, timeout=600)
    print(r.stdout)
    print(r.stderr[-2000:])
    assert r.returncode == 0 and "ALL PASS" in r.stdout, r.stdout + r.stderr[-2000:]
    assert "FAIL" not in r.stdout
