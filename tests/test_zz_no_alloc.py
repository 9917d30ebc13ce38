"""The allocation-free attention entry point against the planned entry point, twice in a row.

Collected last on purpose (file name): a run that stops at the first failure has then already run every other test.
The entry point keeps its partial results in an array built into the library, for hosts that cannot allocate device
memory when they need attention (fixed and audited memory plans, plugins under another runtime's allocator,
no-allocation regions). The second call uses a shorter context and other inputs, so stale partials from the first call
would show. Tolerance: both paths run the same kernels but cut the context into runs at different places, so their
fp16 roundings differ; they are compared within the tolerances the other GPU tests use against the oracle for
contexts above 8 blocks (max-abs <= 5e-3 x output RMS, relative L2 <= 2.5e-4 each, so <= 3.6e-4 between two
independent results; LSE within 1e-3)."""
import importlib

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


def _case(wl, orc, nblocks, nq, seq):
    Kc, Vc = wl.context_blocks(nblocks, seq=seq)
    Q, Kf, Vf = wl.query_blocks(nq, seq=seq)
    maxb = nblocks + nq
    cache = np.zeros((4, maxb, orc.REC_BYTES), np.uint8)
    if nblocks:
        orc.kv_commit(Kc, Vc, cache, maxb, 0)
    if nblocks == 0:
        cache[:] = 0
    if nq > 1:
        orc.kv_commit(Kf, Vf, cache, maxb, nblocks)
    return Q, Kf, Vf, cache, maxb


def test_static_entry_point_matches_planned_path_twice(pkg, orc):
    api = importlib.import_module(pkg.__name__ + ".api")
    api.lib()
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    ctx = api.Context(0)
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    # the last two: 16 query blocks (the slot cap decides the split: 2 runs per tile) and an empty context
    for nblocks, nq, seq in [(150, 1, 301), (37, 3, 302), (40, 16, 303), (0, 1, 304)]:
        Q, Kf, Vf, cache, maxb = _case(pkg.workload, orc, nblocks, nq, seq)
        dQ, dK, dV, dC = dev(Q), dev(Kf), dev(Vf), dev(cache)
        rows = nq * 32
        # existing entry point
        plan = ctx.plan([api.Seq(cache=dC, nblocks=nblocks, nq=nq, q_first=0)])
        O_ref = torch.zeros((rows, 16, 128), dtype=torch.float32, device="cuda")
        L_ref = torch.zeros((rows, 16), dtype=torch.float32, device="cuda")
        q_ref = torch.zeros((rows, 2048), dtype=torch.int8, device="cuda")
        s_ref = torch.zeros((rows, 16), dtype=torch.float32, device="cuda")
        i_ref = torch.zeros((rows, 16), dtype=torch.int32, device="cuda")
        ctx.attention(plan, dQ, dK, dV, O32=O_ref, LSE=L_ref, q8=q_ref, s8=s_ref, sum8=i_ref)
        assert ctx.device_status() == 0
        # the allocation-free one
        O = torch.zeros_like(O_ref); L = torch.zeros_like(L_ref)
        O16 = torch.zeros((rows, 16, 128), dtype=torch.float16, device="cuda")
        q = torch.zeros_like(q_ref); s = torch.zeros_like(s_ref); isum = torch.zeros_like(i_ref)
        api.attention_static(dQ, dK, dV, dC, maxb, nblocks, O16=O16, O32=O, LSE=L, q8=q, s8=s, sum8=isum, err_word=err)
        torch.cuda.synchronize()
        assert int(err.item()) == 0
        a, b = O.cpu().numpy().astype(np.float64), O_ref.cpu().numpy().astype(np.float64)
        rms = np.sqrt((b ** 2).mean())
        assert np.abs(a - b).max() <= 5e-3 * rms, np.abs(a - b).max() / rms
        assert np.sqrt(((a - b) ** 2).sum() / (b ** 2).sum()) <= 3.6e-4
        assert np.abs(L.cpu().numpy() - L_ref.cpu().numpy()).max() <= 1e-3
        assert np.abs(O16.float().cpu().numpy() - O.cpu().numpy()).max() <= 2.0 ** -10 * np.abs(a).max() + 1e-7
        assert np.abs(q.cpu().numpy().astype(np.int32) - q_ref.cpu().numpy().astype(np.int32)).max() <= 1
        assert np.allclose(s.cpu().numpy(), s_ref.cpu().numpy(), rtol=2e-3)
        # and against the oracle, like every other attention test
        O1, L1 = orc.attention(Q, Kf, Vf, cache, maxb, nblocks, dq_mode=1)
        assert np.abs(a - O1).max() <= 5e-3 * rms and np.abs(L.cpu().numpy() - L1).max() <= 1e-3
        plan.close()
    ctx.close()


def test_static_entry_point_rejects_sizes_beyond_its_scratch(pkg):
    api = importlib.import_module(pkg.__name__ + ".api")
    api.lib()
    Q = torch.zeros((17, 32, 16, 128), dtype=torch.float16, device="cuda")
    KV = torch.zeros((17, 32, 4, 128), dtype=torch.float16, device="cuda")
    cache = torch.zeros((4, 32, 4736), dtype=torch.uint8, device="cuda")
    O = torch.zeros((17 * 32, 16, 128), dtype=torch.float16, device="cuda")
    with pytest.raises(api.LlattnError) as e:
        api.attention_static(Q, KV, KV, cache, 32, 4, O16=O)
    assert e.value.code == api.EINVAL and "16" in str(e.value)
