"""The attention operators as the reference engine launches them (decode step `engine/engine.cu:427-432`, batched
prefill pass `:589-598`, partial buffers of the engine's size, the two-argument `pick_bpc`), on the same seeded inputs,
once with the reference's kernels and once with this package's kernels behind `include/attn_shim.cuh`. Both programs
are `tests/attn_ops_dump.cu`, built by `oracle/Makefile` (targets `ref`, `dropin`). Compared: the fp16 output and the
int8 activation form (`engine/attn.cu:340-357`) the dense projection consumes."""
import os
import subprocess

import numpy as np
import pytest

from conftest import ROOT

pytestmark = pytest.mark.gpu
REF = os.path.join(ROOT, "oracle", "_ref")


def frag_pos(c):
    """Position of channel c inside its 128-group in the int8 activation layout (engine/attn.cu:309-312)."""
    base, r = c & ~127, c & 127
    return base + 32 * ((r >> 2) & 3) + 8 * (r >> 5) + 4 * ((r >> 4) & 1) + (r & 3)


def read_dump(path):
    raw = np.fromfile(path, np.uint8)
    at, out = 0, []
    perm = frag_pos(np.arange(2048))
    while at < len(raw):
        ctx0, nb, bpc, nchunks = raw[at:at + 16].view(np.int32)
        at += 16
        rows = nb * 32
        O = raw[at:at + rows * 4096].view(np.float16).astype(np.float32).reshape(rows, 16, 128)
        at += rows * 4096
        q = raw[at:at + rows * 2048].view(np.int8).reshape(rows, 2048)[:, perm].reshape(rows, 16, 128)
        at += rows * 2048
        s = raw[at:at + rows * 64].view(np.float32).reshape(rows, 16)
        at += rows * 64
        sm = raw[at:at + rows * 64].view(np.int32).reshape(rows, 16)
        at += rows * 64
        out.append(dict(ctx0=int(ctx0), nb=int(nb), bpc=int(bpc), nchunks=int(nchunks), O=O, q=q, s=s, sum=sm))
    return out


def run(binary, tmp_path):
    out = str(tmp_path / (os.path.basename(binary) + ".bin"))
    p = subprocess.run([binary, out], capture_output=True, text=True, timeout=300)
    assert p.returncode == 0 and "DONE" in p.stdout, p.stdout[-2000:] + p.stderr[-2000:]
    return read_dump(out)


def test_engine_launch_shapes_match_the_reference_kernels(tmp_path):
    shim, ref = os.path.join(REF, "attn_ops_dump_shim"), os.path.join(REF, "attn_ops_dump_ref")
    if not (os.path.exists(shim) and os.path.exists(ref)):
        pytest.skip("oracle/_ref/attn_ops_dump_{shim,ref} not built (make -C oracle ref dropin REF=<reference checkout>)")
    mine, theirs = run(shim, tmp_path), run(ref, tmp_path)
    assert [(c["ctx0"], c["nb"]) for c in mine] == [(c["ctx0"], c["nb"]) for c in theirs] and len(mine) == 9
    for a, b in zip(mine, theirs):
        tag = f"ctx {a['ctx0']} nb {a['nb']}"
        rms = float(np.sqrt((b["O"].astype(np.float64) ** 2).mean()))
        # fp16 output: both kernels round P to fp16 and the output to fp16
        assert np.abs(a["O"] - b["O"]).max() <= 4e-3 * rms + 2.0 ** -10 * np.abs(b["O"]).max(), tag
        # int8 form, each build against its own fp16 output: code * scale is the output to half a code step
        for c in (a, b):
            deq = c["q"].astype(np.float32) * c["s"][:, :, None]
            assert np.abs(deq - c["O"]).max() <= 0.51 * c["s"].max() + 2.0 ** -10 * np.abs(c["O"]).max(), tag
            assert np.array_equal(c["q"].astype(np.int64).sum(-1), c["sum"]), tag
        # and between the builds
        assert np.allclose(a["s"], b["s"], rtol=5e-3), tag
        assert np.abs(a["q"].astype(np.int32) - b["q"].astype(np.int32)).max() <= 2, tag
        assert (a["q"] == b["q"]).mean() > 0.9, tag
