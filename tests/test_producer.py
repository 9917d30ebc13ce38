"""The producer of the attention inputs (q/k RMSNorm + partial RoPE, engine/ops.cu:429-453).

CPU: the oracle restatement against an independent numpy form. GPU: the kernel against the reference's own kernel
compiled for sm_100a (bit-exact: same arithmetic in the same order) and against the oracle. Tolerance against the
oracle: the oracle works in double, the kernel in fp32 with CUDA's rsqrtf and sincosf, so an output may differ by an
fp16 ulp, and where sincosf's last-bit error crosses a bf16 rounding boundary of cos or sin by 2^-8 of the rotated
pair's magnitude; at least 99.5 % of the outputs must be within one fp16 ulp."""
import importlib

import numpy as np
import pytest


def inputs(T, seed, ctx_tokens=32768):
    g = np.random.default_rng(seed)
    qkv = g.standard_normal((T, 3072)).astype(np.float32) * g.uniform(0.2, 3.0, (T, 1)).astype(np.float32)
    pos = (ctx_tokens - T + np.arange(T)).astype(np.int32)
    gq = g.uniform(0.5, 1.5, 128).astype(np.float32)
    gk = g.uniform(0.5, 1.5, 128).astype(np.float32)
    return qkv, pos, gq, gk, np.float32(1e-6)


def numpy_form(qkv, pos, gq, gk, eps, inv_freq):
    T = qkv.shape[0]
    x = qkv.astype(np.float64).reshape(T, 24, 128)
    r = 1.0 / np.sqrt((x ** 2).mean(-1, keepdims=True) + float(eps))
    g = np.concatenate([np.tile(gq, (16, 1)), np.tile(gk, (4, 1))]).astype(np.float64)
    n = x[:, :20] * r[:, :20] * g[None]
    ang = (pos.astype(np.float32)[:, None] * inv_freq[None, :]).astype(np.float32).astype(np.float64)

    def bf16(a):
        u = a.astype(np.float32).view(np.uint32)
        u = (u + 0x7fff + ((u >> 16) & 1)) & np.uint32(0xffff0000)
        return u.view(np.float32).astype(np.float64)
    cs, sn = bf16(np.cos(ang))[:, None, :], bf16(np.sin(ang))[:, None, :]
    out = n.copy()
    out[..., 0:32] = n[..., 0:32] * cs - n[..., 32:64] * sn
    out[..., 32:64] = n[..., 32:64] * cs + n[..., 0:32] * sn
    return out[:, :16].astype(np.float16), out[:, 16:20].astype(np.float16), x[:, 20:].astype(np.float16)


def test_oracle_producer_matches_numpy_form(orc, pkg):
    api = importlib.import_module(pkg.__name__ + ".api")
    qkv, pos, gq, gk, eps = inputs(40, 1)
    f = api.inv_freq()
    assert f.shape == (32,) and f[0] == 1.0 and abs(float(f[31]) - 3e6 ** (-62 / 64)) < 1e-9
    q, k, v = orc.qk_norm_rope(qkv, pos, gq, gk, eps, f)
    q2, k2, v2 = numpy_form(qkv, pos, gq, gk, eps, f)
    assert np.array_equal(v.view(np.uint16), v2.view(np.uint16))
    for a, b in ((q, q2), (k, k2)):
        d = np.abs(a.astype(np.float32) - b.astype(np.float32))
        assert (d <= np.spacing(np.abs(b)).astype(np.float32)).mean() > 0.999 and d.max() < 2e-2


@pytest.mark.gpu
@pytest.mark.parametrize("T,ctx_tokens", [(32, 32768), (512, 32256), (1, 64), (2048, 131072)])
def test_producer_kernel(orc, pkg, T, ctx_tokens):
    torch = pytest.importorskip("torch")
    import refkernel
    api = importlib.import_module(pkg.__name__ + ".api")
    api.lib()
    qkv, pos, gq, gk, eps = inputs(T, T, ctx_tokens)
    f = api.inv_freq()
    d = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    dq = torch.zeros((T, 16, 128), dtype=torch.float16, device="cuda")
    dk = torch.zeros((T, 4, 128), dtype=torch.float16, device="cuda")
    dv = torch.zeros((T, 4, 128), dtype=torch.float16, device="cuda")
    args = (d(qkv), d(pos), d(gq), d(gk), float(eps), d(f))
    api.qk_norm_rope(*args, dq, dk, dv)
    torch.cuda.synchronize()
    if refkernel.ops_available():
        rq, rk, rv = torch.zeros_like(dq), torch.zeros_like(dk), torch.zeros_like(dv)
        refkernel.qk_norm_rope(*args, rq, rk, rv)
        torch.cuda.synchronize()
        assert torch.equal(rq.view(torch.int16), dq.view(torch.int16))
        assert torch.equal(rk.view(torch.int16), dk.view(torch.int16))
        assert torch.equal(rv.view(torch.int16), dv.view(torch.int16))
    oq, ok, ov = orc.qk_norm_rope(qkv, pos, gq, gk, eps, f)
    assert np.array_equal(dv.cpu().numpy().view(np.uint16), ov.view(np.uint16))
    for got, want in ((dq.cpu().numpy(), oq), (dk.cpu().numpy(), ok)):
        g32, w32 = got.astype(np.float32), want.astype(np.float32)
        diff = np.abs(g32 - w32)
        ulp = np.spacing(np.abs(want)).astype(np.float32)
        assert (diff <= ulp).mean() >= 0.995
        pair = np.abs(w32[..., 0:32]) + np.abs(w32[..., 32:64])                 # magnitude of a rotated pair
        bound = np.concatenate([pair, pair, np.zeros_like(pair), np.zeros_like(pair)], -1) * 2.0 ** -7 + 2 * ulp
        assert (diff <= bound).all()


@pytest.mark.gpu
@pytest.mark.parametrize("nb,paged", [(1, False), (16, False), (5, True)])
def test_producer_fused_with_commit(orc, pkg, nb, paged):
    """A prefill pass's blocks from fp32 qkv to fp16 Q/K/V AND to their 4736-byte records in one kernel
    (engine/engine.cu:589-591 runs ops::qk_norm_rope, then attn::kv_commit on its output): Q/K/V are bit-identical to the
    separate producer, the records byte-equal to committing that output afterwards - with this library's commit kernel,
    with the oracle packer and, when it travelled, with the reference's own two kernels."""
    torch = pytest.importorskip("torch")
    import refkernel
    api = importlib.import_module(pkg.__name__ + ".api")
    api.lib()
    T = 32 * nb
    qkv, pos, gq, gk, eps = inputs(T, 100 + nb, 32768)
    f = api.inv_freq()
    d = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    args = (d(qkv), d(pos), d(gq), d(gk), float(eps), d(f))
    mk = lambda: (torch.zeros((T, 16, 128), dtype=torch.float16, device="cuda"), torch.zeros((T, 4, 128), dtype=torch.float16, device="cuda"),
                  torch.zeros((T, 4, 128), dtype=torch.float16, device="cuda"))
    q0, k0, v0 = mk()
    api.qk_norm_rope(*args, q0, k0, v0)
    q1, k1, v1 = mk()
    maxb, blk = nb + 7, 3
    if paged:
        npages = 4 * nb + 11
        pages = torch.from_numpy(np.random.default_rng(nb).permutation(npages)[:4 * nb].astype(np.int32).reshape(nb, 4)).cuda()
        want = torch.full((npages, 4736), 0x5A, dtype=torch.uint8, device="cuda")
        got = want.clone()
        api.kv_commit_paged(k0.view(nb, 32, 4, 128), v0.view(nb, 32, 4, 128), want, pages)
        api.qkv_prepare_commit(*args, q1, k1, v1, got, pages=pages)
    else:
        want = torch.full((4, maxb, 4736), 0x5A, dtype=torch.uint8, device="cuda")
        got = want.clone()
        api.kv_commit(k0.view(nb, 32, 4, 128), v0.view(nb, 32, 4, 128), want, maxb, blk)
        api.qkv_prepare_commit(*args, q1, k1, v1, got, max_blocks=maxb, blk=blk)
    torch.cuda.synchronize()
    for a, b in ((q0, q1), (k0, k1), (v0, v1)):
        assert torch.equal(a.view(torch.int16), b.view(torch.int16))
    assert torch.equal(got, want)
    if not paged:
        rec = np.full((4, maxb, orc.REC_BYTES), 0x5A, np.uint8)
        orc.kv_commit(k0.cpu().numpy().reshape(nb, 32, 4, 128), v0.cpu().numpy().reshape(nb, 32, 4, 128), rec, maxb, blk)
        assert np.array_equal(got.cpu().numpy(), rec)
        if refkernel.ops_available() and refkernel.available():
            rq, rk, rv = mk()
            refkernel.qk_norm_rope(*args, rq, rk, rv)
            ref = torch.full((4, maxb, 4736), 0x5A, dtype=torch.uint8, device="cuda")
            refkernel.kv_commit(rk.view(nb, 32, 4, 128), rv.view(nb, 32, 4, 128), ref, maxb, blk)
            torch.cuda.synchronize()
            assert torch.equal(ref, got)
    with pytest.raises(ValueError):
        api.qkv_prepare_commit(args[0][:T - 1], *args[1:], q1, k1, v1, got, max_blocks=maxb, blk=blk)
