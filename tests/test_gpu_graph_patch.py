"""The reference engine's graph update path on the drop-in kernels: tests/graph_patch_test.cu captures the shim's
attn_partial / attn_combine in a CUDA graph, patches the two nodes with cudaGraphExecKernelNodeSetParams for shrinking
and growing contexts exactly as engine/engine.cu:533-552 does, and compares every replay with a direct launch."""
import os
import subprocess

import pytest

pytestmark = pytest.mark.gpu
BIN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_bin", "graph_patch_test")


def test_patched_graph_nodes_replay_like_direct_launches():
    if not os.path.exists(BIN):
        pytest.skip("tests/_bin/graph_patch_test is not built (python __graft_entry__.py builds it)")
    r = subprocess.run([BIN], capture_output=True, text=True, timeout=300)
    print(r.stdout)
    assert r.returncode == 0 and "PASS" in r.stdout, r.stdout + r.stderr
