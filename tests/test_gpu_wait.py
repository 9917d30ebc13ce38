"""A wait that can never complete ends in an error code, not in a hang.

Every wait in this library's kernels has a time limit (two seconds in the real kernels), the mbarrier waits inside a
CTA as well as a CTA's wait for the other runs of a tile it shares; when one
runs out the role raises the CTA's abort flag, every other role leaves at its next poll, the kernel reports through the
device error word and returns. llattn_wait_selftest shows exactly that chain on a kernel of its own, with a
one-millisecond limit and barriers that nothing ever completes: no real kernel is made to fail, nothing faults, the
context stays usable, and an attention call afterwards is correct."""
import importlib

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


def test_wait_runs_out_with_an_error_code_and_the_context_stays_usable(pkg, orc):
    api = importlib.import_module(pkg.__name__ + ".api")
    api.lib()
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    waited = torch.zeros(6, dtype=torch.int64, device="cuda")
    api.wait_selftest(1_000_000, err, waited)
    torch.cuda.synchronize()
    assert int(err.item()) == 1 | 2 | 4 | 8 | 128              # every warp left through the error path
    w = waited.cpu().numpy()
    assert 0.9e6 <= w[0] <= 20e6                               # the short limit ran out where it should
    assert (w[1:5] >= 0.9e6).all() and (w[1:5] <= 50e6).all()  # the others were released by the abort flag, far below their 2 s
    assert 0.9e6 <= w[5] <= 20e6                               # the wait for a split tile's other runs, running out alone
    with pytest.raises(api.LlattnError):
        api.wait_selftest(0, err, waited)
    # the device is fine: a normal attention call on the same context of this process
    wl = pkg.workload
    Kc, Vc = wl.context_blocks(5, seq=3)
    Q, Kf, Vf = wl.query_blocks(1, seq=3)
    cache = np.zeros((4, 6, orc.REC_BYTES), np.uint8)
    orc.kv_commit(Kc, Vc, cache, 6, 0)
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    ctx = api.Context(0)
    plan = ctx.plan([api.Seq(cache=dev(cache), nblocks=5)])
    O = torch.zeros((32, 16, 128), dtype=torch.float32, device="cuda")
    ctx.attention(plan, dev(Q), dev(Kf), dev(Vf), O32=O)
    assert ctx.device_status() == 0
    O1, _ = orc.attention(Q, Kf, Vf, cache, 6, 5, dq_mode=1)
    assert np.abs(O.cpu().numpy() - O1).max() <= 2e-3 * np.sqrt((O1.astype(np.float64) ** 2).mean())
    plan.close(); ctx.close()
