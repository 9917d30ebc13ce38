"""The stated floating-point bar at the contexts where the default path misses it.

Bar: max-abs error <= 2e-3 x output RMS and log-sum-exp within 1e-3, against the fp64 oracle over engine-style
dequantised records (one fp16 FMA per value, engine/attn.cu:112-115).

The default path feeds the softmax probabilities to the P.V product as fp16, as the reference kernel does
(engine/attn.cu:261-263). Above about 4 K tokens a few output elements of rows that one key partly dominates then sit
at 2e-3 .. 1e-2 x RMS: that key's probability carries an fp16 rounding of relative size 2^-12 while the RMS over all
rows falls like 1/sqrt(keys) (tests/test_p_rounding_floor.py reproduces the size of that error on the CPU). With
LLATTN_IO_PRECISE_P every probability is carried as an fp16 value plus an fp16 remainder and the bar is met at every
context length; these tests assert exactly that, and keep the measured default-path figures in their output
(run with -s to see the table)."""
import importlib

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

import refkernel  # noqa: E402
from test_gpu_fullsize import device_case, rel_l2, relmax  # noqa: E402

BAR_O, BAR_LSE = 2e-3, 1e-3


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


def run(api, ctx, Q, Kf, Vf, cache, nblocks, precise, nctas=0):
    nq = Q.shape[0]
    plan = ctx.plan([api.Seq(cache=cache, nblocks=nblocks, nq=nq, q_first=0)], nctas)
    O = torch.zeros((nq * 32, 16, 128), dtype=torch.float32, device="cuda")
    LSE = torch.zeros((nq * 32, 16), dtype=torch.float32, device="cuda")
    ctx.attention(plan, Q, Kf, Vf, O32=O, LSE=LSE, precise=precise)
    assert ctx.device_status() == 0
    plan.close()
    return O.cpu().numpy(), LSE.cpu().numpy()


def report(name, O, LSE, O1, L1):
    rms = np.sqrt((O1.astype(np.float64) ** 2).mean())
    err = np.abs(O.astype(np.float64) - O1)
    line = (f"{name:<28} max-abs/rms {err.max() / rms:.2e}  rel-L2 {rel_l2(O, O1):.2e}  "
            f"elements over 2e-3 x rms {int((err > BAR_O * rms).sum())} of {err.size}")
    if LSE is not None:
        line += f"  lse {np.abs(LSE - L1).max():.1e}"
    print(line)
    return err.max() / rms


@pytest.mark.parametrize("nblocks,nq", [(256, 1), (512, 1), (1024, 1), (992, 16)])
def test_precise_path_meets_the_bar_at_long_contexts(api, ctx, orc, pkg, nblocks, nq):
    Q, Kf, Vf, cache, maxb = device_case(api, pkg, nblocks, nq, seed=7000 + nblocks + nq)
    if nq > 1:
        api.kv_commit(Kf, Vf, cache, maxb, nblocks)          # prefill order: commit first (engine/engine.cu:591)
        torch.cuda.synchronize()
    hQ, hK, hV, hC = (x.cpu().numpy() for x in (Q, Kf, Vf, cache))
    O1, L1 = orc.attention(hQ, hK, hV, hC, maxb, nblocks, dq_mode=1)
    print(f"\n{nblocks * 32} committed tokens, {nq} query block(s):")
    Od, Ld = run(api, ctx, Q, Kf, Vf, cache, nblocks, precise=False)
    Op, Lp = run(api, ctx, Q, Kf, Vf, cache, nblocks, precise=True)
    ed = report("default (fp16 P)", Od, Ld, O1, L1)
    ep = report("precise (fp16 P + remainder)", Op, Lp, O1, L1)
    if refkernel.available():
        ref = refkernel.attention(Q, Kf, Vf, cache, maxb, nblocks).cpu().numpy().astype(np.float32)
        report("reference kernel (fp16 out)", ref, None, O1, L1)
    assert ep <= BAR_O and np.abs(Lp - L1).max() <= BAR_LSE
    assert rel_l2(Op, O1) <= 1e-4
    assert ed <= 1e-2 and np.abs(Ld - L1).max() <= BAR_LSE    # the default path's enforced bound at these sizes
    # the precise result does not depend on where the planner cuts the context either
    O2, _ = run(api, ctx, Q, Kf, Vf, cache, nblocks, precise=True, nctas=37)
    assert relmax(O2, Op) <= 2 * BAR_O                       # two results, each within the bar of the oracle


@pytest.mark.parametrize("nblocks", [0, 3, 5, 33, 130])
def test_precise_path_on_short_and_ragged_tiles(api, ctx, orc, pkg, nblocks):
    """Tiles of 1 to 4 blocks and runs on few CTAs: the remainder columns of partial tiles and their PV chains."""
    wl = pkg.workload
    Kc, Vc = wl.context_blocks(nblocks, seq=500 + nblocks)
    Q, Kf, Vf = wl.query_blocks(1, seq=500 + nblocks)
    maxb = nblocks + 1
    cache = np.zeros((4, maxb, orc.REC_BYTES), np.uint8)
    if nblocks:
        orc.kv_commit(Kc, Vc, cache, maxb, 0)
    O1, L1 = orc.attention(Q, Kf, Vf, cache, maxb, nblocks, dq_mode=1)
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    for nctas in (0, 3):
        O, LSE = run(api, ctx, dev(Q), dev(Kf), dev(Vf), dev(cache), nblocks, precise=True, nctas=nctas)
        assert relmax(O, O1) <= BAR_O and np.abs(LSE - L1).max() <= BAR_LSE, (nblocks, nctas)


@pytest.mark.parametrize("pattern", ["rising", "alternating"])
def test_precise_path_when_the_reference_exponent_moves(api, ctx, orc, pkg, pattern):
    """Score levels that climb by many powers of two from block to block: the rare path rescales P and its remainders."""
    n = 37
    wl = pkg.workload
    Kc, Vc = wl.context_blocks(n, seq=901)
    Q, Kf, Vf = wl.query_blocks(1, seq=901)
    u = np.sign(np.random.default_rng(6).standard_normal(128)).astype(np.float32)
    j = np.arange(n, dtype=np.float32)
    g = {"rising": j * 0.5, "alternating": np.where((j // 2) % 2 == 0, 0.0, 6.0) * (1 + j / n)}[pattern]
    Kc = (Kc.astype(np.float32) * 0.25 + g[:, None, None, None] * u * 0.35).astype(np.float16)
    Q = (Q.astype(np.float32) * 0.25 + u * 1.0).astype(np.float16)
    Kf = (Kf.astype(np.float32) * 0.25).astype(np.float16)
    cache = np.zeros((4, n + 1, orc.REC_BYTES), np.uint8)
    orc.kv_commit(Kc, Vc, cache, n + 1, 0)
    O1, L1 = orc.attention(Q, Kf, Vf, cache, n + 1, n, dq_mode=1)
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    O, LSE = run(api, ctx, dev(Q), dev(Kf), dev(Vf), dev(cache), n, precise=True, nctas=2)
    assert np.isfinite(O).all()
    assert relmax(O, O1) <= BAR_O and np.abs(LSE - L1).max() <= 2 * BAR_LSE


@pytest.mark.parametrize("nblocks", [64, 256])
def test_kernel_error_is_the_emulated_fp16_rounding_of_p(api, ctx, orc, pkg, nblocks):
    """The kernel on one CTA (every kv head one run, like oracle/emulate_p.py) against the CPU emulation of its P
    rounding: their distances from the fp64 oracle agree to a few percent, in the worst element and in relative L2
    (single elements differ: ex2.approx and the exact exponential round a probability to different fp16 neighbours now
    and then) - so the default path's residual has the size of the fp16 rounding of P and no other source is needed."""
    import emulate_p
    wl = pkg.workload
    Kc, Vc = wl.context_blocks(nblocks, seq=77)
    Q, Kf, Vf = wl.query_blocks(1, seq=77)
    maxb = nblocks + 1
    cache = np.zeros((4, maxb, orc.REC_BYTES), np.uint8)
    orc.kv_commit(Kc, Vc, cache, maxb, 0)
    O1, _ = orc.attention(Q, Kf, Vf, cache, maxb, nblocks, dq_mode=1)
    rms = np.sqrt((O1.astype(np.float64) ** 2).mean())
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    for mode, precise in (("fp16", False), ("fp16x2", True)):
        Oe = emulate_p.attention_rounded_p(Q, Kf, Vf, cache, maxb, nblocks, mode)
        Ok, _ = run(api, ctx, dev(Q), dev(Kf), dev(Vf), dev(cache), nblocks, precise=precise, nctas=1)
        e_k, e_e = np.abs(Ok - O1).max() / rms, np.abs(Oe - O1).max() / rms
        l_k, l_e = rel_l2(Ok, O1), rel_l2(Oe, O1)
        print(f"{nblocks * 32} tokens, {mode}: max-abs/rms kernel {e_k:.3e} emulation {e_e:.3e}; rel-L2 kernel {l_k:.3e} emulation {l_e:.3e}")
        if not precise:
            assert abs(e_k - e_e) <= 0.15 * e_e and abs(l_k - l_e) <= 0.1 * l_e
        else:
            # one run of 257 units per kv head: the tensor core's own fp32 accumulation over a chain that long shows
            # (4e-4 x RMS here, 1.6e-3 for a 1025-unit run); in the planner's usual cuts it is below 1e-4
            assert e_k <= 1e-3 and e_e <= 5e-5
