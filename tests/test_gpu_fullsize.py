"""Parity at the full sizes of the benchmark configurations (B200).

Contexts of 8 K .. 32 K tokens are checked three ways: against the reference's own kernels compiled for sm_100a (when
oracle/_ref travelled), against the CPU oracle (fp64 attention over engine-style dequantised records), and through
properties that do not depend on size: the result must not depend on how the planner cuts the context into runs, and
the commit -> attend round trip of a prefill pass must equal attending the same records committed beforehand.
Tolerances of the default path (fp16 P) as in test_gpu_parity.py for long contexts: rel-L2 <= 2.5e-4, max-abs <= 5e-3 x
RMS for a decode step at 8 K and 32 K tokens (measured 1.7e-3 .. 4.1e-3 depending on where the planner cuts), <= 1e-2
for the 16-block prefill pass (measured 5.0e-3). The stated bar of 2e-3 x RMS is met at these sizes by the precise path
(tests/test_gpu_precise.py); tests/test_p_rounding_floor.py shows on the CPU that the default path's residual is the
fp16 rounding of P."""
import importlib

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

import refkernel  # noqa: E402


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


def device_case(api, pkg, nblocks, nq, seed):
    """Committed context built ON the GPU with the commit kernel (the way the engine does), seeded torch inputs."""
    wl = pkg.workload
    g = torch.Generator(device="cuda")
    g.manual_seed(seed)
    maxb = nblocks + nq
    K = torch.randn((nblocks, 32, 4, 128), generator=g, device="cuda")
    K[..., list(wl.OUTLIER_CHANNELS)] *= wl.OUTLIER_GAIN
    K = K.half()
    V = torch.randn((nblocks, 32, 4, 128), generator=g, device="cuda").half()
    cache = torch.zeros((4, maxb, 4736), dtype=torch.uint8, device="cuda")
    api.kv_commit(K, V, cache, maxb, 0)
    Q = torch.randn((nq, 32, 16, 128), generator=g, device="cuda").half()
    Kf = torch.randn((nq, 32, 4, 128), generator=g, device="cuda")
    Kf[..., list(wl.OUTLIER_CHANNELS)] *= wl.OUTLIER_GAIN
    Kf = Kf.half()
    Vf = torch.randn((nq, 32, 4, 128), generator=g, device="cuda").half()
    return Q, Kf, Vf, cache, maxb


def run(api, ctx, Q, Kf, Vf, cache, nblocks, nctas=0):
    nq = Q.shape[0]
    plan = ctx.plan([api.Seq(cache=cache, nblocks=nblocks, nq=nq, q_first=0)], nctas)
    O = torch.zeros((nq * 32, 16, 128), dtype=torch.float32, device="cuda")
    LSE = torch.zeros((nq * 32, 16), dtype=torch.float32, device="cuda")
    ctx.attention(plan, Q, Kf, Vf, O32=O, LSE=LSE)
    assert ctx.device_status() == 0
    stats = plan.stats
    plan.close()
    return O.cpu().numpy(), LSE.cpu().numpy(), stats


@pytest.mark.parametrize("nblocks", [256, 1024])
def test_decode_step_at_8k_and_32k(api, ctx, orc, pkg, nblocks):
    Q, Kf, Vf, cache, maxb = device_case(api, pkg, nblocks, 1, seed=nblocks)
    O, LSE, st = run(api, ctx, Q, Kf, Vf, cache, nblocks)
    assert st.nctas >= 48                                   # the context really is spread over the GPU
    hQ, hK, hV, hC = (x.cpu().numpy() for x in (Q, Kf, Vf, cache))
    O1, L1 = orc.attention(hQ, hK, hV, hC, maxb, nblocks, dq_mode=1)
    assert rel_l2(O, O1) <= 2.5e-4
    assert relmax(O, O1) <= 5e-3
    assert np.abs(LSE - L1).max() <= 1e-3
    # size-independent property: the answer does not depend on where the planner cuts the context
    for nctas in (4, 37):
        O2, L2, _ = run(api, ctx, Q, Kf, Vf, cache, nblocks, nctas)
        assert rel_l2(O2, O) <= 3.6e-4 and np.abs(L2 - LSE).max() <= 1e-3
    if refkernel.available():
        ref = refkernel.attention(Q, Kf, Vf, cache, maxb, nblocks).cpu().numpy().astype(np.float32)
        assert rel_l2(O, O1) <= rel_l2(ref, O1)             # closer to the oracle than the reference kernel is
        assert rel_l2(O, ref) <= 4e-4


def test_prefill_16_blocks_on_31744_tokens(api, ctx, orc, pkg):
    """The prefill workload at full size: 16 query blocks appended to 992 committed blocks, commit first, then block-causal attention
    (engine/engine.cu:591-598); the 16 new records are byte-compared with the oracle packer and the reference kernel."""
    ctx0, nq = 992, 16
    Q, Kf, Vf, cache, maxb = device_case(api, pkg, ctx0, nq, seed=4)
    api.kv_commit(Kf, Vf, cache, maxb, ctx0)
    torch.cuda.synchronize()
    hQ, hK, hV = (x.cpu().numpy() for x in (Q, Kf, Vf))
    want = np.zeros((4, nq, orc.REC_BYTES), np.uint8)
    orc.kv_commit(hK, hV, want, nq, 0)
    assert np.array_equal(cache[:, ctx0:ctx0 + nq].cpu().numpy(), want)
    O, LSE, st = run(api, ctx, Q, Kf, Vf, cache, ctx0)
    hC = cache.cpu().numpy()
    O1, L1 = orc.attention(hQ, hK, hV, hC, maxb, ctx0, dq_mode=1)
    assert rel_l2(O, O1) <= 2.5e-4 and relmax(O, O1) <= 1e-2 and np.abs(LSE - L1).max() <= 1e-3
    if refkernel.available():
        c2 = cache.clone()
        c2[:, ctx0:] = 0
        refkernel.kv_commit(Kf, Vf, c2, maxb, ctx0)
        torch.cuda.synchronize()
        assert torch.equal(c2, cache)
        ref = refkernel.attention(Q, Kf, Vf, cache, maxb, ctx0).cpu().numpy().astype(np.float32)
        assert rel_l2(O, ref) <= 4e-4


def test_ragged_batch_up_to_32k(api, ctx, orc, pkg):
    """The ragged serving batch in miniature: 12 sequences with seeded ragged lengths in [128, 32768] tokens in one call."""
    lens = [int(x) for x in pkg.workload.ragged_lengths(12, seed=11)]
    lens[0], lens[1] = 4, 1024                                # both ends of the range
    cases = [device_case(api, pkg, n, 1, seed=100 + i) for i, n in enumerate(lens)]
    seqs = [api.Seq(cache=c[3], nblocks=n, nq=1, q_first=i) for i, (c, n) in enumerate(zip(cases, lens))]
    plan = ctx.plan(seqs)
    Q = torch.cat([c[0] for c in cases]); Kf = torch.cat([c[1] for c in cases]); Vf = torch.cat([c[2] for c in cases])
    O = torch.zeros((len(lens) * 32, 16, 128), dtype=torch.float32, device="cuda")
    LSE = torch.zeros((len(lens) * 32, 16), dtype=torch.float32, device="cuda")
    ctx.attention(plan, Q, Kf, Vf, O32=O, LSE=LSE)
    assert ctx.device_status() == 0
    mean = plan.stats.total_units / plan.stats.nctas
    if plan.stats.nitems > plan.stats.nctas:                  # contiguous shares: near equal
        assert plan.stats.max_cta_units <= 1.02 * mean + 12
    else:                                                     # a run per CTA (chosen when the start-up of a second run costs more)
        assert plan.stats.max_cta_units <= 1.5 * mean + 12
    O, LSE = O.cpu().numpy(), LSE.cpu().numpy()
    for i, (c, n) in enumerate(zip(cases, lens)):
        sl = slice(i * 32, (i + 1) * 32)
        if refkernel.available():
            ref = refkernel.attention(c[0], c[1], c[2], c[3], c[4], n).cpu().numpy().astype(np.float32)
            assert rel_l2(O[sl], ref) <= 4e-4, (i, n)
        if i < 4:                                             # the oracle on a few of them (seconds each at 32 K)
            O1, L1 = orc.attention(*(x.cpu().numpy() for x in c[:4]), c[4], n, dq_mode=1)
            assert rel_l2(O[sl], O1) <= 2.5e-4 and np.abs(LSE[sl] - L1).max() <= 1e-3, (i, n)
    plan.close()
