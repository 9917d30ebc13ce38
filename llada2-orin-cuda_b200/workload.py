"""Seeded synthetic inputs for the block-attention path.

They stand in for real model activations: the reference itself checks this path only on synthetic N(0,1) data
(engine/tests/test_attn.cu:20-27 draws Q/K/V ~ N(0,1) and turns one K channel into an outlier). Here Q, K, V are
N(0,1) rounded to fp16 and four fixed K channels of every kv head are multiplied by 8.

Everything is drawn from numpy's counter-based Philox generator keyed by (seed, stream id), so any host in any
process regenerates identical bytes for a given (sequence, layer, kind).
"""
from __future__ import annotations

import numpy as np

D, BLK, NKV, NQH = 128, 32, 4, 16
REC_BYTES = 4736
OUTLIER_CHANNELS = (5, 37, 70, 101)
OUTLIER_GAIN = 8.0
BASE_SEED = 7

_KIND = {"ctx_k": 1, "ctx_v": 2, "q": 3, "fresh_k": 4, "fresh_v": 5}


def _rng(seed: int, seq: int, layer: int, kind: str) -> np.random.Generator:
    return np.random.Generator(np.random.Philox(key=[seed, (seq << 24) | (layer << 8) | _KIND[kind]]))


def _normal16(g: np.random.Generator, shape) -> np.ndarray:
    return g.standard_normal(shape, dtype=np.float32).astype(np.float16)


def _add_outliers(K: np.ndarray) -> np.ndarray:
    Kf = K.astype(np.float32)
    Kf[..., list(OUTLIER_CHANNELS)] *= OUTLIER_GAIN
    return Kf.astype(np.float16)


def context_blocks(nblocks: int, seq: int = 0, layer: int = 0, seed: int = BASE_SEED):
    """fp16 K, V of `nblocks` committed blocks: [nblocks][32][4][128] each (K carries the outlier channels)."""
    K = _add_outliers(_normal16(_rng(seed, seq, layer, "ctx_k"), (nblocks, BLK, NKV, D)))
    V = _normal16(_rng(seed, seq, layer, "ctx_v"), (nblocks, BLK, NKV, D))
    return K, V


def query_blocks(nq: int, seq: int = 0, layer: int = 0, seed: int = BASE_SEED):
    """Q [nq][32][16][128] and the fresh K, V [nq][32][4][128] of nq query blocks, fp16."""
    Q = _normal16(_rng(seed, seq, layer, "q"), (nq, BLK, NQH, D))
    Kf = _add_outliers(_normal16(_rng(seed, seq, layer, "fresh_k"), (nq, BLK, NKV, D)))
    Vf = _normal16(_rng(seed, seq, layer, "fresh_v"), (nq, BLK, NKV, D))
    return Q, Kf, Vf


def ragged_lengths(nseq: int, lo_tokens: int = 128, hi_tokens: int = 32768, seed: int = BASE_SEED) -> np.ndarray:
    """Committed context lengths in blocks, uniform over the multiples of 32 in [lo_tokens, hi_tokens]."""
    g = np.random.Generator(np.random.Philox(key=[seed, 0xA66ED]))
    return g.integers(lo_tokens // BLK, hi_tokens // BLK + 1, size=nseq).astype(np.int32)


def algorithmic_bytes(nblocks: int, int8_out: bool = False) -> int:
    """Bytes one (sequence, layer, 32-token query block) must move at `nblocks` committed blocks: the packed
    records of the 4 kv heads, Q, the fresh K and V, and the output."""
    out = 69632 if int8_out else 131072
    return nblocks * NKV * REC_BYTES + 131072 + 65536 + out


def algorithmic_flops(nblocks: int) -> int:
    """QK^T + PV flops (multiply-add = 2) for one (sequence, layer, query block)."""
    return 4 * BLK * NQH * D * (nblocks * BLK + BLK)


def dense_weights(rows: int, K: int, seed: int = 0):
    """Seeded 4-bit weight matrix in the engine's device strip layout (engine/moe_i8.cu:34-41): uint8
    [rows/16][K/128 * 1024 code bytes, then K/128 metas of 48 bytes]. Codes uniform in 0..15, fp16 scales log-uniform
    around 0.01, zero points 5..10. Returns (strips, codes [rows][K] uint8, scale [rows][K/128] float16, zero uint8)."""
    import numpy as np
    g = np.random.default_rng([seed, rows, K, 77])
    ktot = K // 128
    codes = g.integers(0, 16, (rows, K), dtype=np.uint8)
    scale = (0.01 * np.exp(g.normal(0, 0.5, (rows, ktot)))).astype(np.float16)
    zero = g.integers(5, 11, (rows, ktot), dtype=np.uint8)
    strips = np.zeros((rows // 16, ktot * 1072), np.uint8)
    # code tile: byte (w < 4 ? 0 : 512) + 16 * (4 g + t) + 4 * (w % 4) + e holds logical k = 32 (w / 2) + 16 (w % 2) + 4 t + e
    # of row g (low nibble) and row g + 8 (high nibble)
    w = np.arange(8); t = np.arange(4); e = np.arange(4); gg = np.arange(8)
    W_, G_, T_, E_ = np.meshgrid(w, gg, t, e, indexing="ij")
    byte = np.where(W_ < 4, 0, 512) + 16 * (4 * G_ + T_) + 4 * (W_ % 4) + E_
    kk = 32 * (W_ // 2) + 16 * (W_ % 2) + 4 * T_ + E_
    for sidx in range(rows // 16):
        blk = codes[16 * sidx:16 * sidx + 16].reshape(16, ktot, 128)
        for kt in range(ktot):
            tile = np.zeros(1024, np.uint8)
            tile[byte] = blk[G_, kt, kk] | (blk[G_ + 8, kt, kk] << 4)
            strips[sidx, kt * 1024:(kt + 1) * 1024] = tile
            meta = np.zeros(48, np.uint8)
            sc = scale[16 * sidx:16 * sidx + 16, kt].view(np.uint16)
            pair = sc[:8].astype(np.uint32) | (sc[8:].astype(np.uint32) << 16)
            meta[:32] = pair.view(np.uint8)
            zz = zero[16 * sidx:16 * sidx + 16, kt]
            meta[32:48] = np.stack([zz[:8], zz[8:]], axis=1).reshape(-1)
            strips[sidx, ktot * 1024 + kt * 48: ktot * 1024 + (kt + 1) * 48] = meta
    return strips, codes, scale, zero


def int8_activations(ntokens: int, K: int, seed: int = 0):
    """Seeded moe8::Act triple (engine/moe_i8.cu:55-66): int8 [ntokens][K] (any order: the values are random), fp32
    scale and int32 sum per token and 128-group."""
    import numpy as np
    g = np.random.default_rng([seed, ntokens, K, 78])
    q = g.integers(-127, 128, (ntokens, K), dtype=np.int8)
    s = (0.02 * np.exp(g.normal(0, 0.5, (ntokens, K // 128)))).astype(np.float32)
    qsum = q.reshape(ntokens, K // 128, 128).astype(np.int32).sum(axis=2).astype(np.int32)
    return q, s, qsum
