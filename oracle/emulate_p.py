"""Test infrastructure: a numpy emulation of how the sm_100a attention kernel forms and rounds the softmax
probabilities, used to attribute its residual error to the fp16 rounding of P. Not part of the product path.

The kernel (csrc/attn_kernel.cuh) differs from exact attention over the same fp16-dequantised records in one place
that matters: p = 2^(s * scale * log2e - mref) is rounded to fp16 before the P.V product, where the row's reference
mref is the exact maximum of the run's first 128 keys and moves to a later 32-key chunk's maximum only when that
exceeds it by more than 8 powers of two (the reference kernel rescales lazily in the same way, engine/attn.cu:237-263).
Numerator and denominator use the same rounded p (the kernel sums P on the tensor core through a column of ones).
Everything else (fp16 products accumulated in fp32) is orders of magnitude smaller and is done in float64 here.

p_mode: "fp16"    the kernel's default path
        "fp16x2"  fp16 value + fp16 remainder (LLATTN_IO_PRECISE_P)
        "fp32"    no rounding of P at all (what is left is the emulation's own float64 arithmetic)
"""
from __future__ import annotations

import numpy as np

import oracle as orc

SLACK = 8.0
TILE_KEYS = 128
CHUNK_KEYS = 32


def _round_p(p: np.ndarray, p_mode: str) -> np.ndarray:
    if p_mode == "fp32":
        return p.astype(np.float32).astype(np.float64)
    hi = p.astype(np.float32).astype(np.float16)
    if p_mode == "fp16":
        return hi.astype(np.float64)
    lo = (p.astype(np.float32) - hi.astype(np.float32)).astype(np.float16)
    return hi.astype(np.float64) + lo.astype(np.float64)


def attention_rounded_p(Q, Kf, Vf, cache, max_blocks, nblocks, p_mode="fp16", scale=None):
    """One sequence, ONE query block, each (kv head) processed as a single run from the first committed key to the
    fresh block (what the kernel does when its plan is given a single CTA). Q float16 [1][32][16][128]; Kf, Vf float16
    [1][32][4][128]; cache uint8 [4][max_blocks][4736]. Returns O float64 [32][16][128]."""
    assert Q.shape[0] == 1
    scale = (1.0 / np.sqrt(orc.D)) if scale is None else scale
    sl2 = np.float32(np.float32(scale) * np.float32(1.4426950408889634))
    O = np.zeros((orc.BLK, orc.NQH, orc.D), np.float64)
    for h in range(orc.NKV):
        if nblocks:
            Kc, Vc = orc.dequant_records_np(cache[h, :nblocks], mode=1)          # [nblocks][32][128], fp16 values
            K = np.concatenate([Kc.reshape(-1, orc.D).astype(np.float64), Kf[0, :, h].astype(np.float64)])
            V = np.concatenate([Vc.reshape(-1, orc.D).astype(np.float64), Vf[0, :, h].astype(np.float64)])
        else:
            K, V = Kf[0, :, h].astype(np.float64), Vf[0, :, h].astype(np.float64)
        q = Q[0, :, 4 * h:4 * h + 4].astype(np.float64).reshape(-1, orc.D)       # row = token * 4 + head
        S = (q @ K.T).astype(np.float32)                                           # fp32 scores as the tensor core leaves them
        nk = S.shape[1]
        mref = S[:, :min(TILE_KEYS, nk)].max(axis=1) * sl2                         # float32
        num = np.zeros((q.shape[0], orc.D), np.float64)
        den = np.zeros(q.shape[0], np.float64)
        for c0 in range(0, nk, CHUNK_KEYS):
            s = S[:, c0:c0 + CHUNK_KEYS]
            cs = s.max(axis=1) * sl2
            move = cs > mref + np.float32(SLACK)
            if move.any():
                corr = np.where(move, np.exp2((mref - cs).astype(np.float64)), 1.0)
                num *= corr[:, None]
                den *= corr
                mref = np.where(move, cs, mref).astype(np.float32)
            x = s * sl2 - mref[:, None]                                            # float32 (the kernel uses one fused multiply-add)
            p = _round_p(np.exp2(x.astype(np.float64)), p_mode)
            num += p @ V[c0:c0 + CHUNK_KEYS]
            den += p.sum(axis=1)
        o = num / den[:, None]
        O[:, 4 * h:4 * h + 4] = o.reshape(orc.BLK, 4, orc.D)
    return O
