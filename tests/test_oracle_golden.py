"""The CPU oracle against the golden fixtures made from the reference's own fake_quant, and against itself
(C restatement vs the independent numpy restatement)."""
import os

import numpy as np
import pytest


def _load(golden_dir, name):
    return np.load(os.path.join(golden_dir, name))


@pytest.mark.parametrize("case", ["edge", "seeded"])
def test_packer_matches_reference_fake_quant_bitwise(orc, pkg, golden_dir, case):
    g = _load(golden_dir, "fakequant_cases.npz")
    if case == "edge":
        K, V = g["edge_K"], g["edge_V"]
    else:
        nb, seq, layer = (int(x) for x in g["seeded_args"])
        K, V = pkg.workload.context_blocks(nb, seq=seq, layer=layer)
    nb = K.shape[0]
    cache = np.zeros((4, nb + 1, orc.REC_BYTES), np.uint8)
    orc.kv_commit(K, V, cache, nb + 1, 0)
    # records dequantised the way fake_quant returns values (fp32 q*s + mn) must equal its output bit for bit
    Kd, Vd = orc.dequant_records_np(cache[:, :nb], mode=2)            # [4][nb][32][128]
    Kq, Vq = g[f"{case}_Kq"], g[f"{case}_Vq"]                          # [nb][32][4][128]
    assert np.array_equal(Kd.transpose(1, 2, 0, 3).view(np.uint32), Kq.view(np.uint32))
    assert np.array_equal(Vd.transpose(1, 2, 0, 3).view(np.uint32), Vq.view(np.uint32))
    # the scalar C dequantiser (mode 2) agrees with the numpy one
    for h, b in [(0, 0), (3, nb - 1)]:
        Kc, Vc = orc.dequant_record(cache[h, b], mode=2)
        assert np.array_equal(Kc.astype(np.float32), Kd[h, b]) and np.array_equal(Vc.astype(np.float32), Vd[h, b])


def test_c_packer_equals_numpy_packer(orc, pkg, golden_dir):
    g = _load(golden_dir, "fakequant_cases.npz")
    for K, V in [(g["edge_K"], g["edge_V"]), pkg.workload.context_blocks(5, seq=9, layer=4)]:
        nb = K.shape[0]
        cache = np.zeros((4, nb + 2, orc.REC_BYTES), np.uint8)
        orc.kv_commit(K, V, cache, nb + 2, 1)
        assert np.array_equal(cache[:, 1:nb + 1], orc.pack_records_np(K, V))
        assert not cache[:, 0].any() and not cache[:, nb + 1].any()


def test_fake_quant_restated_in_c_and_numpy(orc, golden_dir):
    g = _load(golden_dir, "fakequant_cases.npz")
    V = g["edge_V"].astype(np.float32)
    ref = g["edge_Vq"]
    assert np.array_equal(orc.fake_quant_np(V, 128).view(np.uint32), ref.view(np.uint32))
    assert np.array_equal(orc.fake_quant_c(V.reshape(-1, 128), 128).reshape(ref.shape).view(np.uint32), ref.view(np.uint32))


def test_record_layout_constants(orc):
    assert orc.REC_BYTES == 32 * 64 + 128 * 4 + 32 * 64 + 32 * 4 == 4736
    assert (orc.KOFF_META, orc.VOFF, orc.VOFF_META) == (2048, 2560, 4608)
    # fragment order is a permutation of each 128-group that keeps runs of 4
    pos = [orc.frag_pos(c) for c in range(256)]
    assert sorted(pos) == list(range(256))
    assert all(pos[c + 1] == pos[c] + 1 for c in range(0, 256, 4) for c in (c, c + 1, c + 2))
    assert orc.frag_pos(4) == 32 and orc.frag_pos(16) == 4 and orc.frag_pos(32) == 8


def test_attention_oracle_matches_reference_simquant_sdpa(orc, pkg, golden_dir):
    g = _load(golden_dir, "simquant_attn.npz")
    nb, seq, layer = (int(x) for x in g["args"])
    Kc, Vc = pkg.workload.context_blocks(nb, seq=seq, layer=layer)
    Q, Kf, Vf = pkg.workload.query_blocks(1, seq=seq, layer=layer)
    rms = float(np.sqrt((g["O"].astype(np.float64) ** 2).mean()))
    # numpy simulated-quantisation attention vs torch SDPA over the reference's fake_quant output
    O, LSE = orc.simquant_attention_np(Q[0], Kf[0], Vf[0], Kc, Vc)
    assert np.abs(O - g["O"]).max() <= 2e-5 * rms and np.abs(LSE - g["LSE"]).max() <= 2e-5
    # C oracle over packed records: fp32 flavour and fp64 flavour with exact dequantisation
    cache = np.zeros((4, nb + 1, orc.REC_BYTES), np.uint8)
    orc.kv_commit(Kc, Vc, cache, nb + 1, 0)
    O32, L32 = orc.attention(Q, Kf, Vf, cache, nb + 1, nb, dq_mode=2, acc_f32=True)
    O64, L64 = orc.attention(Q, Kf, Vf, cache, nb + 1, nb, dq_mode=0)
    for Ox, Lx in ((O32, L32), (O64, L64)):
        assert np.abs(Ox - g["O"]).max() <= 2e-5 * rms and np.abs(Lx - g["LSE"]).max() <= 2e-5


def test_attention_oracle_prefill_visibility_and_pages(orc, pkg):
    """Block j of a batched pass sees nblocks + j records plus its own fresh block (engine/attn.cu:150-158)."""
    wl = pkg.workload
    ctx0, nq = 3, 3
    Kc, Vc = wl.context_blocks(ctx0, seq=11)
    Q, Kf, Vf = wl.query_blocks(nq, seq=11)
    maxb = ctx0 + nq
    cache = np.zeros((4, maxb, orc.REC_BYTES), np.uint8)
    orc.kv_commit(Kc, Vc, cache, maxb, 0)
    orc.kv_commit(Kf, Vf, cache, maxb, ctx0)                  # commit-then-attend order of the prefill pass
    O, LSE = orc.attention(Q, Kf, Vf, cache, maxb, ctx0)
    for j in range(nq):
        Oj, Lj = orc.attention(Q[j:j + 1], Kf[j:j + 1], Vf[j:j + 1], cache, maxb, ctx0 + j)
        assert np.array_equal(O[j * 32:(j + 1) * 32], Oj) and np.array_equal(LSE[j * 32:(j + 1) * 32], Lj)
    # a shuffled record pool addressed through a page table gives the same answer
    g = np.random.default_rng(0)
    perm = g.permutation(4 * maxb).astype(np.int32).reshape(4, maxb)
    pool = np.zeros((4 * maxb, orc.REC_BYTES), np.uint8)
    pool[perm.reshape(-1)] = cache.reshape(-1, orc.REC_BYTES)
    Op, Lp = orc.attention(Q, Kf, Vf, pool, maxb, ctx0, pages=perm)
    assert np.array_equal(Op, O) and np.array_equal(Lp, LSE)


def test_empty_context(orc, pkg):
    Q, Kf, Vf = pkg.workload.query_blocks(1, seq=2)
    cache = np.zeros((4, 1, orc.REC_BYTES), np.uint8)
    O, LSE = orc.attention(Q, Kf, Vf, cache, 1, 0)
    O2, L2 = orc.simquant_attention_np(Q[0], Kf[0], Vf[0], Kf[:0], Vf[:0])
    assert np.abs(O - O2).max() < 1e-5 and np.abs(LSE - L2).max() < 1e-5


def test_act_q8_epilogue(orc):
    g = np.random.default_rng(5)
    O = g.standard_normal((3, 16, 128)).astype(np.float32)
    O[1, 2] = 0
    q8, s8, sum8 = orc.act_q8(O)
    inv = np.argsort([orc.frag_pos(c) for c in range(2048)])    # logical index at each stored position
    for r in range(3):
        logical = np.empty(2048, np.int8)
        logical[inv] = q8[r]                                     # stored[pos(c)] = q(c)
        logical = np.array([q8[r, orc.frag_pos(c)] for c in range(2048)], np.int8).reshape(16, 128)
        sc = np.maximum(np.abs(O[r]).max(-1) / np.float32(127), np.float32(1e-30))
        assert np.array_equal(s8[r], sc)
        assert np.array_equal(logical, np.clip(np.rint(O[r] / sc[:, None]), -127, 127).astype(np.int8))
        assert np.array_equal(sum8[r], logical.astype(np.int32).sum(-1))
