"""Re-planning without allocation and the fused tile merge.

The reference re-parameterises the 40 attention nodes of its captured step graph every time a block is committed
(engine/engine.cu:533-562). Here the kernel reads lengths and work items from the plan's device memory: a committed
block needs one llattn_plan_update (an asynchronous copy into the same device blob) and the captured graph is replayed
unchanged. One plan serves all layers of a step through llattn_io.cache_offset."""
import importlib

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

TOL_O, TOL_L2, TOL_LSE = 5e-3, 2.5e-4, 1e-3


@pytest.fixture(scope="module")
def api(pkg):
    m = importlib.import_module(pkg.__name__ + ".api")
    m.lib()
    return m


@pytest.fixture(scope="module")
def ctx(api):
    c = api.Context(0)
    yield c
    c.close()


def rel_l2(a, b):
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    return float(np.sqrt(((a - b) ** 2).sum() / (b ** 2).sum()))


def relmax(a, b):
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    return float(np.abs(a - b).max() / np.sqrt((b ** 2).mean()))


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def test_captured_step_survives_committed_blocks(api, ctx, orc, pkg):
    """A 6-layer step over two sequences, captured ONCE as a CUDA graph with a single plan; then blocks are committed
    (contexts grow by different amounts, one shrinks back as after a new prompt), the plan is updated on the stream
    and the same graph is replayed. Every replay is checked against the oracle."""
    L, wl = 6, pkg.workload
    maxb = 80
    lens = [[9, 33], [10, 34], [41, 34], [3, 70]]          # committed blocks of the two sequences, step after step
    top = [max(x[i] for x in lens) for i in range(2)]
    K = [[wl.context_blocks(top[s], seq=700 + s, layer=l) for s in range(2)] for l in range(L)]
    caches_np = np.zeros((L, 2, 4, maxb, orc.REC_BYTES), np.uint8)
    for l in range(L):
        for s in range(2):
            orc.kv_commit(K[l][s][0], K[l][s][1], caches_np[l, s], maxb, 0)     # every block that will ever be visible
    caches = dev(caches_np)
    layer_bytes = caches[0].numel()
    qkv = [[wl.query_blocks(1, seq=700 + s, layer=l) for s in range(2)] for l in range(L)]
    dQ = dev(np.stack([np.concatenate([qkv[l][s][0] for s in range(2)]) for l in range(L)]))
    dK = dev(np.stack([np.concatenate([qkv[l][s][1] for s in range(2)]) for l in range(L)]))
    dV = dev(np.stack([np.concatenate([qkv[l][s][2] for s in range(2)]) for l in range(L)]))
    O = torch.zeros((L, 64, 16, 128), dtype=torch.float32, device="cuda")
    LSE = torch.zeros((L, 64, 16), dtype=torch.float32, device="cuda")
    seqs = lambda n: [api.Seq(cache=caches[0, s], nblocks=n[s], nq=1, q_first=s) for s in range(2)]
    plan = ctx.plan(seqs(lens[0]))
    stream = torch.cuda.Stream()

    def step():
        for l in range(L):
            ctx.attention(plan, dQ[l], dK[l], dV[l], O32=O[l], LSE=LSE[l], stream=stream, cache_offset=l * layer_bytes)

    with torch.cuda.stream(stream):
        step()
        stream.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=stream):
            step()
    for k, n in enumerate(lens):
        with torch.cuda.stream(stream):
            if k:
                plan.update(seqs(n), stream=stream)           # no allocation, no device synchronisation
            O.zero_()
            g.replay()
            stream.synchronize()
        assert ctx.device_status(stream) == 0
        got, gl = O.cpu().numpy(), LSE.cpu().numpy()
        for l in range(L):
            for s in range(2):
                Q, Kf, Vf = qkv[l][s]
                O1, L1 = orc.attention(Q, Kf, Vf, caches_np[l, s], maxb, n[s], dq_mode=1)
                sl = slice(32 * s, 32 * s + 32)
                assert rel_l2(got[l, sl], O1) <= TOL_L2 and relmax(got[l, sl], O1) <= TOL_O, (k, l, s)
                assert np.abs(gl[l, sl] - L1).max() <= TOL_LSE, (k, l, s)
    # an update that does not fit what the plan was created for is refused, and the plan stays usable
    with pytest.raises(api.LlattnError):
        plan.update(seqs(lens[0])[:1], stream=stream)
    with pytest.raises(api.LlattnError):
        plan.update([api.Seq(cache=caches[0, s], nblocks=5, nq=2, q_first=2 * s) for s in range(2)], stream=stream)
    plan.close()


def test_fused_merge_is_deterministic_and_leaves_its_counters_clear(api, ctx, orc, pkg):
    """Tiles cut into many runs (a 200-block context cut into runs of 16 blocks: more than 10 per kv head): whichever CTA finishes
    last folds the tile, always in slot order, so repeated launches agree bit for bit; every output format comes from
    the same fp32 values; and the arrival counters are back at zero, or the second launch would never write."""
    n = 200
    wl = pkg.workload
    Kc, Vc = wl.context_blocks(n, seq=800)
    Q, Kf, Vf = wl.query_blocks(1, seq=800)
    cache = np.zeros((4, n + 1, orc.REC_BYTES), np.uint8)
    orc.kv_commit(Kc, Vc, cache, n + 1, 0)
    dC, dQ, dK, dV = dev(cache), dev(Q), dev(Kf), dev(Vf)
    plan = ctx.plan([api.Seq(cache=dC, nblocks=n)])
    assert plan.stats.nitems >= 40
    outs = []
    for rep in range(4):
        O = torch.full((32, 16, 128), float("nan"), dtype=torch.float32, device="cuda")
        O16 = torch.zeros((32, 16, 128), dtype=torch.float16, device="cuda")
        LSE = torch.zeros((32, 16), dtype=torch.float32, device="cuda")
        q8 = torch.zeros((32, 2048), dtype=torch.int8, device="cuda")
        s8 = torch.zeros((32, 16), dtype=torch.float32, device="cuda")
        sum8 = torch.zeros((32, 16), dtype=torch.int32, device="cuda")
        ctx.attention(plan, dQ, dK, dV, O32=O, O16=O16, LSE=LSE, q8=q8, s8=s8, sum8=sum8)
        assert ctx.device_status() == 0
        outs.append([x.cpu().numpy() for x in (O, O16, LSE, q8, s8, sum8)])
    for rep in range(1, 4):
        for a, b in zip(outs[0], outs[rep]):
            assert np.array_equal(a, b)
    O, O16, LSE, q8, s8, sum8 = outs[0]
    O1, L1 = orc.attention(Q, Kf, Vf, cache, n + 1, n, dq_mode=1)
    assert np.isfinite(O).all() and rel_l2(O, O1) <= TOL_L2 and relmax(O, O1) <= TOL_O and np.abs(LSE - L1).max() <= TOL_LSE
    assert np.array_equal(O16, O.astype(np.float16))
    w8, ws, wsum = orc.act_q8(O)
    assert np.array_equal(q8, w8) and np.array_equal(s8, ws) and np.array_equal(sum8, wsum)
    plan.close()
