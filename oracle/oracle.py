"""Python face of the CPU oracle. TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke check and by the
bench's CPU-baseline legs; never by the product path.

Two things live here:
  * a ctypes binding of liboracle.so (oracle.c: packer, dequantiser, fp64/fp32 attention, int8 epilogue,
    simulated quantiser), and
  * an independent numpy restatement of the packer and of the simulated-quantisation attention, used to
    cross-check the C code and for the larger cases where vectorised numpy is quicker than scalar C.

Reference lines followed: engine/attn.cu:369-418 (packer), engine/tests/test_attn.cu:42-95 (dequantise +
fp64 attention), quant/s06_arbitrate.py:78-89 (fake_quant), quant/student_case.py:49-74 (block attention over
fake-quantised context).
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
D, BLK, NKV, NQH = 128, 32, 4, 16
REC_BYTES, KOFF_META, VOFF, VOFF_META = 4736, 2048, 2560, 4608
OUTLIER_CHANNELS = (5, 37, 70, 101)

_lib = None


def build(force: bool = False) -> str:
    """Compile liboracle.so next to this file (gcc); returns its path."""
    so = os.path.join(HERE, "liboracle.so")
    src = os.path.join(HERE, "oracle.c")
    if force or not os.path.exists(so) or os.path.getmtime(so) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", HERE, "-s", "all"])
    return so


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(build())
        L = _lib
        vp, i32, sz = ctypes.c_void_p, ctypes.c_int, ctypes.c_size_t
        L.orc_kv_commit.argtypes = [vp, vp, vp, i32, i32, i32]
        L.orc_dequant_record.argtypes = [vp, i32, vp, vp]
        L.orc_attention.argtypes = [vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, vp, vp]
        L.orc_act_q8.argtypes = [vp, i32, vp, vp, vp]
        L.orc_fake_quant.argtypes = [vp, vp, sz, i32]
        L.orc_frag_pos.argtypes = [i32]
        L.orc_frag_pos.restype = i32
        L.orc_f2h.argtypes = [ctypes.c_float]
        L.orc_f2h.restype = ctypes.c_uint16
        L.orc_h2f.argtypes = [ctypes.c_uint16]
        L.orc_h2f.restype = ctypes.c_float
        L.orc_num_threads.restype = i32
        L.orc_qk_norm_rope.argtypes = [vp, vp, vp, vp, ctypes.c_float, vp, vp, vp, vp, i32]
        L.orc_dense_w4a8.argtypes = [vp, vp, vp, vp, vp, i32, i32, i32]
        L.orc_dense_w4a8.restype = None
    return _lib


def _p(a: np.ndarray):
    assert a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(ctypes.c_void_p)


# ------------------------------------------------------------------ C oracle wrappers

def kv_commit(Kf: np.ndarray, Vf: np.ndarray, cache: np.ndarray, max_blocks: int, blk: int) -> None:
    """Kf, Vf: float16 [nb][32][4][128]; cache: uint8 [4][max_blocks][4736], records blk..blk+nb-1 written."""
    assert Kf.dtype == np.float16 and Vf.dtype == np.float16 and cache.dtype == np.uint8
    nb = Kf.shape[0]
    assert Kf.shape == (nb, BLK, NKV, D) and Vf.shape == Kf.shape and cache.shape == (NKV, max_blocks, REC_BYTES)
    assert 0 <= blk and blk + nb <= max_blocks
    lib().orc_kv_commit(_p(Kf), _p(Vf), _p(cache), max_blocks, blk, nb)


def dequant_record(rec: np.ndarray, mode: int = 0):
    """One 4736-byte record -> (K, V) float64 [32][128]. mode 0 exact, 1 fp16-rounded FMA, 2 fp32 q*s+mn."""
    K = np.empty((BLK, D), np.float64)
    V = np.empty((BLK, D), np.float64)
    lib().orc_dequant_record(_p(np.ascontiguousarray(rec)), mode, _p(K), _p(V))
    return K, V


def attention(Q, Kf, Vf, cache, max_blocks, nblocks, dq_mode=0, acc_f32=False, pages=None):
    """One sequence. Q float16 [nb][32][16][128]; Kf, Vf float16 [nb][32][4][128]; cache uint8 records.
    Returns (O float32 [nb*32][16][128], LSE float32 [nb*32][16])."""
    nb = Q.shape[0]
    assert Q.shape == (nb, BLK, NQH, D) and Kf.shape == (nb, BLK, NKV, D) and Vf.shape == Kf.shape
    O = np.empty((nb * BLK, NQH, D), np.float32)
    LSE = np.empty((nb * BLK, NQH), np.float32)
    pg = None
    if pages is not None:
        pg = np.ascontiguousarray(pages, dtype=np.int32)
    lib().orc_attention(_p(Q), _p(Kf), _p(Vf), _p(cache), _p(pg) if pg is not None else None, max_blocks, nblocks,
                        nb, dq_mode, 1 if acc_f32 else 0, _p(O), _p(LSE))
    return O, LSE


def act_q8(O: np.ndarray):
    """O float32 [rows][16][128] -> (q8 int8 [rows][2048] fragment order, s8 float32 [rows][16], sum8 int32)."""
    rows = O.shape[0]
    O = np.ascontiguousarray(O, np.float32)
    q8 = np.empty((rows, 2048), np.int8)
    s8 = np.empty((rows, NQH), np.float32)
    sum8 = np.empty((rows, NQH), np.int32)
    lib().orc_act_q8(_p(O), rows, _p(q8), _p(s8), _p(sum8))
    return q8, s8, sum8


def fake_quant_c(x: np.ndarray, group: int) -> np.ndarray:
    x = np.ascontiguousarray(x, np.float32)
    y = np.empty_like(x)
    lib().orc_fake_quant(_p(x), _p(y), x.size // group, group)
    return y


def qk_norm_rope(qkv, pos, gq, gk, eps, inv_freq):
    """Producer of the attention inputs (engine/ops.cu:429-453) in double precision with the kernel's bf16 / fp16
    roundings. qkv float32 [T][3072], pos int32 [T], gq/gk float32 [128], inv_freq float32 [32].
    Returns q float16 [T][16][128], k, v float16 [T][4][128]."""
    T = qkv.shape[0]
    q = np.empty((T, NQH, D), np.float16)
    k = np.empty((T, NKV, D), np.float16)
    v = np.empty((T, NKV, D), np.float16)
    lib().orc_qk_norm_rope(_p(np.ascontiguousarray(qkv, np.float32)), _p(np.ascontiguousarray(pos, np.int32)),
                           _p(np.ascontiguousarray(gq, np.float32)), _p(np.ascontiguousarray(gk, np.float32)), float(eps),
                           _p(np.ascontiguousarray(inv_freq, np.float32)), _p(q), _p(k), _p(v), T)
    return q, k, v


def dense_w4a8(W: np.ndarray, q: np.ndarray, s: np.ndarray, qsum: np.ndarray, Y: np.ndarray) -> None:
    """Y [ntokens][rows] float32 += the W4.A8 projection (engine/moe_i8.cu:295-400, MODE 2). W: uint8 strips in the
    engine's device layout [rows/16][K/128 * 1024 + K/128 * 48]; q int8 [ntokens][K] in fragment order; s float32 and
    qsum int32 [ntokens][K/128]."""
    ntokens, K = q.shape
    rows = Y.shape[1]
    assert W.dtype == np.uint8 and W.size == rows // 16 * (K // 128) * 1072 and Y.dtype == np.float32
    lib().orc_dense_w4a8(_p(W), _p(q), _p(np.ascontiguousarray(s, np.float32)), _p(np.ascontiguousarray(qsum, np.int32)), _p(Y),
                         ntokens, rows, K)


def frag_pos(c: int) -> int:
    return lib().orc_frag_pos(c)


def num_threads() -> int:
    return lib().orc_num_threads()


# ------------------------------------------------------------------ numpy restatements (independent of the C code)

def _meta(mn: np.ndarray, mx: np.ndarray):
    """fp16 scale (with the 6.2e-5 floor) and fp16 min of groups, from fp32 min/max (engine/attn.cu:383)."""
    s = np.maximum((mx - mn) / np.float32(15.0), np.float32(6.2e-5)).astype(np.float16)
    return np.ascontiguousarray(s), np.ascontiguousarray(mn.astype(np.float16))


def pack_records_np(Kf: np.ndarray, Vf: np.ndarray) -> np.ndarray:
    """Kf, Vf float16 [nb][32][4][128] -> records uint8 [4][nb][4736] (numpy form of engine/attn.cu:369-418)."""
    nb = Kf.shape[0]
    K = Kf.astype(np.float32).transpose(2, 0, 1, 3)          # [4][nb][32][128]
    V = Vf.astype(np.float32).transpose(2, 0, 1, 3)
    ks, km = _meta(K.min(axis=2), K.max(axis=2))              # per channel over tokens: [4][nb][128]
    vs, vm = _meta(V.min(axis=3), V.max(axis=3))              # per token over dims:     [4][nb][32]
    with np.errstate(over="ignore"):
        kq = np.clip(np.rint((K - km.astype(np.float32)[:, :, None, :]) / ks.astype(np.float32)[:, :, None, :]), 0, 15)
        vq = np.clip(np.rint((V - vm.astype(np.float32)[:, :, :, None]) / vs.astype(np.float32)[:, :, :, None]), 0, 15)
    kq = kq.astype(np.uint8)
    vq = vq.astype(np.uint8)
    rec = np.zeros((NKV, nb, REC_BYTES), np.uint8)
    rec[:, :, 0:KOFF_META] = (kq[..., 0::2] | (kq[..., 1::2] << 4)).reshape(NKV, nb, 2048)
    rec[:, :, KOFF_META:KOFF_META + 256] = ks.view(np.uint8).reshape(NKV, nb, 256)
    rec[:, :, KOFF_META + 256:VOFF] = km.view(np.uint8).reshape(NKV, nb, 256)
    rec[:, :, VOFF:VOFF_META] = (vq[..., 0::2] | (vq[..., 1::2] << 4)).reshape(NKV, nb, 2048)
    rec[:, :, VOFF_META:VOFF_META + 64] = vs.view(np.uint8).reshape(NKV, nb, 64)
    rec[:, :, VOFF_META + 64:REC_BYTES] = vm.view(np.uint8).reshape(NKV, nb, 64)
    return rec


def unpack_records_np(rec: np.ndarray):
    """records uint8 [...][4736] -> dict of codes (uint8 [...][32][128]) and fp16 meta arrays."""
    lead = rec.shape[:-1]
    kb = rec[..., 0:KOFF_META].reshape(*lead, BLK, 64)
    vb = rec[..., VOFF:VOFF_META].reshape(*lead, BLK, 64)
    kc = np.empty((*lead, BLK, D), np.uint8)
    vc = np.empty((*lead, BLK, D), np.uint8)
    kc[..., 0::2], kc[..., 1::2] = kb & 15, kb >> 4
    vc[..., 0::2], vc[..., 1::2] = vb & 15, vb >> 4
    f16 = lambda a: np.ascontiguousarray(a).view(np.float16)
    return dict(kc=kc, vc=vc,
                ks=f16(rec[..., KOFF_META:KOFF_META + 256]), km=f16(rec[..., KOFF_META + 256:VOFF]),
                vs=f16(rec[..., VOFF_META:VOFF_META + 64]), vm=f16(rec[..., VOFF_META + 64:REC_BYTES]))


def dequant_records_np(rec: np.ndarray, mode: int = 2):
    """records -> (K, V) [...][32][128]. mode 2: fp32 q*s + mn (fake_quant's value); mode 0: float64 exact;
    mode 1: rounded once to fp16 (returned as float32)."""
    u = unpack_records_np(rec)
    if mode == 2:
        f = np.float32
        K = u["kc"].astype(f) * u["ks"].astype(f)[..., None, :] + u["km"].astype(f)[..., None, :]
        V = u["vc"].astype(f) * u["vs"].astype(f)[..., :, None] + u["vm"].astype(f)[..., :, None]
        return K, V
    f = np.float64
    K = u["kc"].astype(f) * u["ks"].astype(f)[..., None, :] + u["km"].astype(f)[..., None, :]
    V = u["vc"].astype(f) * u["vs"].astype(f)[..., :, None] + u["vm"].astype(f)[..., :, None]
    if mode == 1:
        # float64 -> float16 is a single rounding in numpy
        return K.astype(np.float16).astype(np.float32), V.astype(np.float16).astype(np.float32)
    return K, V


def fake_quant_np(x: np.ndarray, group: int) -> np.ndarray:
    """numpy form of quant/s06_arbitrate.py:78-89 for bits=4 (fp32 in, fp32 dequantised out)."""
    sh = x.shape
    xf = x.astype(np.float32).reshape(*sh[:-1], sh[-1] // group, group)
    mn, mx = xf.min(-1, keepdims=True), xf.max(-1, keepdims=True)
    s = np.maximum((mx - mn) / np.float32(15), np.float32(6.2e-5)).astype(np.float16).astype(np.float32)
    mn = mn.astype(np.float16).astype(np.float32)
    q = np.clip(np.rint((xf - mn) / s), 0, 15)
    return (q * s + mn).reshape(sh).astype(np.float32)


def simquant_context_np(Kctx: np.ndarray, Vctx: np.ndarray):
    """fp16 context K/V [nblk][32][4][128] -> fake-quantised fp32 in the same layout: K per channel over each
    block's 32 tokens, V per token over the 128 dims (quant/student_case.py:63-66 with the rotation R = I)."""
    Kt = np.ascontiguousarray(Kctx.astype(np.float32).transpose(0, 2, 3, 1))     # [nblk][4][128][32]
    Kq = fake_quant_np(Kt, 32).transpose(0, 3, 1, 2)
    Vq = fake_quant_np(Vctx.astype(np.float32), D)
    return np.ascontiguousarray(Kq), Vq


def simquant_attention_np(Q, Kf, Vf, Kctx, Vctx):
    """The fp32 simulated-quantisation reference for ONE query block: fake-quantise the context, then softmax
    attention in fp32 over [quantised context | fresh block] with GQA head repeat (quant/student_case.py:68-73).
    Q float16 [32][16][128]; Kf, Vf float16 [32][4][128]; Kctx, Vctx float16 [nblk][32][4][128].
    Returns (O float32 [32][16][128], LSE float32 [32][16])."""
    f = np.float32
    if Kctx.shape[0]:
        Kq, Vq = simquant_context_np(Kctx, Vctx)
        K = np.concatenate([Kq.reshape(-1, NKV, D), Kf.astype(f)], 0)
        V = np.concatenate([Vq.reshape(-1, NKV, D), Vf.astype(f)], 0)
    else:
        K, V = Kf.astype(f), Vf.astype(f)
    q = Q.astype(f).reshape(BLK, NKV, NQH // NKV, D)
    s = np.einsum("thgd,khd->thgk", q, K, dtype=f) * f(1.0 / np.sqrt(D))
    m = s.max(-1, keepdims=True)
    p = np.exp(s - m, dtype=f)
    l = p.sum(-1, keepdims=True, dtype=f)
    O = np.einsum("thgk,khd->thgd", p / l, V, dtype=f)
    return O.reshape(BLK, NQH, D), (m + np.log(l)).reshape(BLK, NQH).astype(f)
