"""Dense W4.A8 projection that consumes the attention output (llattn_dense_w4a8): oracle on CPU, kernel on the GPU.

Integer group products are exact and every float operation is the reference's, in its order (one product of the two
scales, one fused multiply-add per 128-group, one add into Y): the GPU tests ask for identical bits against the CPU
oracle and against the reference's own moe8::gemm compiled for sm_100a (when it travelled)."""
import importlib

import numpy as np
import pytest


def test_oracle_against_float64_restatement(orc, pkg):
    """The C oracle (tile and fragment layouts of engine/moe_i8.cu:55-60,127-160) against a numpy restatement that
    takes the weights in logical order and the activations out of fragment order."""
    wl = pkg.workload
    rows, K, nt = 256, 384, 7
    strips, codes, scale, zero = wl.dense_weights(rows, K, 1)
    q, s, qsum = wl.int8_activations(nt, K, 2)
    Y0 = np.random.default_rng(3).normal(size=(nt, rows)).astype(np.float32)
    Y = Y0.copy()
    orc.dense_w4a8(strips, q, s, qsum, Y)
    fp = np.array([orc.frag_pos(c) for c in range(128)])
    ql = q.reshape(nt, K // 128, 128)[:, :, fp].astype(np.int64)
    P = np.einsum("rgk,ngk->nrg", codes.reshape(rows, K // 128, 128).astype(np.int64), ql)
    v = P - zero.astype(np.int64)[None] * qsum[:, None, :]
    ref = Y0 + (scale.astype(np.float64)[None] * s[:, None, :] * v).sum(axis=2)
    assert np.abs(Y - ref).max() <= 2e-6 * np.abs(ref).max()


def test_meta_layout(pkg):
    """Scale pairs (rows g | g + 8) at 4 g and zero pairs at 32 + 2 g of every 48-byte meta (engine/moe_i8.cu:38-40)."""
    strips, codes, scale, zero = pkg.workload.dense_weights(32, 256, 5)
    ktot = 2
    for sidx in range(2):
        for kt in range(ktot):
            meta = strips[sidx, ktot * 1024 + kt * 48: ktot * 1024 + (kt + 1) * 48]
            for g in range(8):
                pair = meta[4 * g:4 * g + 4].view(np.uint16)
                assert pair[0] == scale[16 * sidx + g, kt].view(np.uint16) and pair[1] == scale[16 * sidx + g + 8, kt].view(np.uint16)
                assert meta[32 + 2 * g] == zero[16 * sidx + g, kt] and meta[33 + 2 * g] == zero[16 * sidx + g + 8, kt]


torch = pytest.importorskip("torch")


@pytest.fixture(scope="module")
def api(pkg):
    m = importlib.import_module(pkg.__name__ + ".api")
    m.lib()
    return m


def _dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


@pytest.mark.gpu
@pytest.mark.parametrize("ntokens,rows,K", [(32, 2048, 2048), (64, 2048, 2048), (100, 256, 512), (1, 128, 128), (192, 2048, 2048)])
def test_dense_bit_exact_vs_oracle(api, orc, pkg, ntokens, rows, K):
    wl = pkg.workload
    strips, _, _, _ = wl.dense_weights(rows, K, 11)
    q, s, qsum = wl.int8_activations(ntokens, K, 12)
    Y0 = np.random.default_rng(13).normal(size=(ntokens, rows)).astype(np.float32)
    want = Y0.copy()
    orc.dense_w4a8(strips, q, s, qsum, want)
    Y = _dev(Y0)
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    api.dense_w4a8(_dev(strips), _dev(q), _dev(s), _dev(qsum), Y, err_word=err)
    torch.cuda.synchronize()
    assert int(err.item()) == 0
    got = Y.cpu().numpy()
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), float(np.abs(got - want).max())


@pytest.mark.gpu
def test_dense_bit_exact_vs_reference_kernel(api, pkg):
    import refkernel
    if not refkernel.gemm_available():
        pytest.skip("reference GEMM library did not travel")
    wl = pkg.workload
    ntokens, rows, K = 96, 2048, 2048
    strips, _, _, _ = wl.dense_weights(rows, K, 21)
    q, s, qsum = wl.int8_activations(ntokens, K, 22)
    Y0 = np.random.default_rng(23).normal(size=(ntokens, rows)).astype(np.float32)
    dW, dq, ds, dsum = _dev(strips), _dev(q), _dev(s), _dev(qsum)
    Yr, Yn = _dev(Y0), _dev(Y0)
    refkernel.dense_w4a8(dW, dq, ds, dsum, Yr)
    api.dense_w4a8(dW, dq, ds, dsum, Yn)
    torch.cuda.synchronize()
    a, b = Yr.cpu().numpy(), Yn.cpu().numpy()
    assert np.array_equal(a.view(np.uint32), b.view(np.uint32)), float(np.abs(a - b).max())


@pytest.mark.gpu
def test_dense_consumes_the_attention_epilogue(api, orc, pkg):
    """Attention -> int8 Act (merge kernel) -> projection, against the oracle chain on the kernel's own fp32 output."""
    wl = pkg.workload
    Kc, Vc = wl.context_blocks(6, seq=400)
    Q, Kf, Vf = wl.query_blocks(1, seq=400)
    cache = np.zeros((4, 7, orc.REC_BYTES), np.uint8)
    orc.kv_commit(Kc, Vc, cache, 7, 0)
    ctx = api.Context(0)
    dc = _dev(cache)
    plan = ctx.plan([api.Seq(cache=dc, nblocks=6, nq=1, q_first=0)])
    q8 = torch.zeros((32, 2048), dtype=torch.int8, device="cuda")
    s8 = torch.zeros((32, 16), dtype=torch.float32, device="cuda")
    sum8 = torch.zeros((32, 16), dtype=torch.int32, device="cuda")
    ctx.attention(plan, _dev(Q), _dev(Kf), _dev(Vf), q8=q8, s8=s8, sum8=sum8)
    assert ctx.device_status() == 0
    strips, _, _, _ = wl.dense_weights(2048, 2048, 31)
    h0 = np.random.default_rng(32).normal(size=(32, 2048)).astype(np.float32)
    h = _dev(h0)
    api.dense_w4a8(_dev(strips), q8, s8, sum8, h)
    torch.cuda.synchronize()
    want = h0.copy()
    orc.dense_w4a8(strips, q8.cpu().numpy(), s8.cpu().numpy(), sum8.cpu().numpy(), want)
    assert np.array_equal(h.cpu().numpy().view(np.uint32), want.view(np.uint32))
    plan.close(); ctx.close()


@pytest.mark.gpu
def test_dense_argument_errors(api):
    t = torch.zeros(16, dtype=torch.uint8, device="cuda")
    with pytest.raises(api.LlattnError) as e:
        api.lib().llattn_dense_w4a8  # symbol exists
        api._check(api.lib().llattn_dense_w4a8(t.data_ptr(), t.data_ptr(), t.data_ptr(), t.data_ptr(), t.data_ptr(), 32, 100, 128, None, None))
    assert e.value.code == api.EINVAL
