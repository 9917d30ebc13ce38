"""ctypes binding of libllattn.so and the host-side mirror of the reference's `attn` operator interface.

Names follow the reference (engine/attn.cu): `Args`, `pick_bpc`, `chunks_for`, `kv_commit`, `attn_partial`,
`attn_combine`, the record constants. `Context` / `Plan` / `attention` are the batched path (many sequences, ragged
lengths, paged or contiguous caches). Device memory is held in torch tensors; only their data pointers cross the
C ABI. There is no fallback: loading fails loudly when the CUDA library has not been built.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, Structure, byref, c_char_p, c_float, c_int, c_int32, c_int64, c_size_t, c_void_p
from dataclasses import dataclass
from typing import Optional, Sequence

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("LLATTN_LIB", os.path.join(HERE, "libllattn.so"))   # LLATTN_LIB: another build of the same library

D, BLK, NKV, NQH = 128, 32, 4, 16
KV_BLOCK_BYTES, KOFF_META, VOFF, VOFF_META = 4736, 2048, 2560, 4608
SCALE = 0.08838834764831845  # 1/sqrt(128), the constant engine/engine.cu:430 passes

OK, EINVAL, ECUDA, ENOMEM, EDEVICE = 0, 1, 2, 3, 4
IO_PRECISE_P = 1  # llattn_io.flags

EXPORTS = (
    "llattn_version", "llattn_last_error", "llattn_pick_bpc", "llattn_chunks_for", "llattn_tile_units", "llattn_kv_commit",
    "llattn_kv_commit_paged", "llattn_qk_norm_rope", "llattn_qkv_prepare_commit", "llattn_attn_partial", "llattn_attn_combine", "llattn_create", "llattn_destroy",
    "llattn_plan_create", "llattn_plan_destroy", "llattn_plan_get_stats", "llattn_plan_preview", "llattn_attention",
    "llattn_plan_update", "llattn_attention_host", "llattn_host_flush", "llattn_device_status",
    "llattn_dense_w4a8", "llattn_kvpool_create", "llattn_kvpool_destroy", "llattn_kvpool_open", "llattn_kvpool_append", "llattn_kvpool_pages", "llattn_kvpool_mark_committed",
    "llattn_kvpool_close", "llattn_kvpool_stats", "llattn_attention_static", "llattn_wait_selftest",
)


class LlattnError(RuntimeError):
    def __init__(self, code: int, msg: str):
        super().__init__(f"llattn status {code}: {msg}")
        self.code = code


class _Args(Structure):
    _fields_ = [("Q", c_void_p), ("Kf", c_void_p), ("Vf", c_void_p), ("cache", c_void_p), ("max_blocks", c_int),
                ("nblocks", c_int), ("blocks_per_chunk", c_int), ("nchunks", c_int), ("scale", c_float),
                ("Opart", c_void_p), ("Mpart", c_void_p), ("Lpart", c_void_p)]


class _Seq(Structure):
    _fields_ = [("cache", c_void_p), ("pages", c_void_p), ("head_stride", c_int32), ("nblocks", c_int32),
                ("nq", c_int32), ("q_first", c_int32)]


class _IO(Structure):
    _fields_ = [("Q", c_void_p), ("Kf", c_void_p), ("Vf", c_void_p), ("O16", c_void_p), ("O32", c_void_p),
                ("LSE", c_void_p), ("q8", c_void_p), ("s8", c_void_p), ("sum8", c_void_p), ("scale", c_float),
                ("flags", ctypes.c_uint32), ("cache_offset", c_int64)]


class PlanStats(Structure):
    _fields_ = [("nseq", c_int32), ("nq_total", c_int32), ("nitems", c_int32), ("nslots", c_int32), ("nctas", c_int32),
                ("total_units", c_int64), ("max_cta_units", c_int64), ("workspace_bytes", c_size_t)]


_lib = None


def lib() -> ctypes.CDLL:
    """Loads libllattn.so (built by build.py). Raises if it is missing: there is no other implementation."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise FileNotFoundError(f"{LIB_PATH} is not built; run `python __graft_entry__.py` or build.build()")
        L = ctypes.CDLL(LIB_PATH)
        L.llattn_version.restype = c_char_p
        L.llattn_last_error.restype = c_char_p
        L.llattn_pick_bpc.argtypes = [c_int, c_int]
        L.llattn_chunks_for.argtypes = [c_int, c_int]
        L.llattn_kv_commit.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]
        L.llattn_kv_commit_paged.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p]
        L.llattn_qk_norm_rope.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_void_p,
                                          c_void_p, c_int, c_void_p]
        L.llattn_qkv_prepare_commit.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_void_p,
                                                c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_void_p]
        L.llattn_attn_partial.argtypes = [POINTER(_Args), c_int, c_void_p, c_void_p]
        L.llattn_attn_combine.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p,
                                          c_void_p, c_void_p, c_int, c_void_p]
        L.llattn_create.argtypes = [c_int, POINTER(c_void_p)]
        L.llattn_destroy.argtypes = [c_void_p]
        L.llattn_destroy.restype = None
        L.llattn_plan_create.argtypes = [c_void_p, POINTER(_Seq), c_int, c_int, POINTER(c_void_p)]
        L.llattn_plan_destroy.argtypes = [c_void_p]
        L.llattn_plan_destroy.restype = None
        L.llattn_plan_get_stats.argtypes = [c_void_p, POINTER(PlanStats)]
        L.llattn_plan_preview.argtypes = [POINTER(_Seq), c_int, c_int, POINTER(PlanStats), c_void_p, c_int, c_void_p, c_int]
        L.llattn_attention.argtypes = [c_void_p, c_void_p, POINTER(_IO), c_void_p]
        L.llattn_plan_update.argtypes = [c_void_p, POINTER(_Seq), c_int, c_void_p]
        L.llattn_attention_host.argtypes = [c_void_p, c_void_p, POINTER(_IO), c_void_p]
        L.llattn_host_flush.argtypes = [c_void_p, c_void_p]
        L.llattn_dense_w4a8.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p]
        L.llattn_kvpool_create.argtypes = [c_int, POINTER(c_void_p)]
        L.llattn_kvpool_destroy.argtypes = [c_void_p]
        L.llattn_kvpool_destroy.restype = None
        L.llattn_kvpool_open.argtypes = [c_void_p, c_void_p, c_int, POINTER(c_int32), POINTER(c_int32), c_void_p, c_int]
        L.llattn_kvpool_append.argtypes = [c_void_p, c_int32, c_void_p, POINTER(c_int32), POINTER(c_int32)]
        L.llattn_kvpool_pages.argtypes = [c_void_p, c_int32, c_void_p, c_int, POINTER(c_int32)]
        L.llattn_kvpool_mark_committed.argtypes = [c_void_p, c_int32, c_int]
        L.llattn_kvpool_close.argtypes = [c_void_p, c_int32]
        L.llattn_kvpool_stats.argtypes = [c_void_p, c_void_p]
        L.llattn_device_status.argtypes = [c_void_p, c_void_p, POINTER(c_int)]
        L.llattn_wait_selftest.argtypes = [ctypes.c_uint64, c_void_p, c_void_p, c_void_p]
        L.llattn_attention_static.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_float,
                                              c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]
        _lib = L
    return _lib


def _check(rc: int) -> None:
    if rc != OK:
        raise LlattnError(rc, lib().llattn_last_error().decode())


def _ptr(t) -> Optional[int]:
    """Data pointer of a torch tensor (device or host) or None."""
    if t is None:
        return None
    if not t.is_contiguous():
        raise ValueError("tensors crossing the C ABI must be contiguous")
    return t.data_ptr()


def _stream(stream) -> Optional[int]:
    if stream is None:
        import torch
        return torch.cuda.current_stream().cuda_stream
    return getattr(stream, "cuda_stream", stream)


# ------------------------------------------------------------------ reference policy helpers

def pick_bpc(nblocks: int, nbatch: int) -> int:
    """attn::pick_bpc (engine/attn.cu:361-364)."""
    return lib().llattn_pick_bpc(nblocks, nbatch)


def tile_units() -> int:
    """32-token blocks per MMA tile of the loaded build."""
    return lib().llattn_tile_units()


def chunks_for(nblocks: int, bpc: int) -> int:
    """attn::chunks_for (engine/attn.cu:67)."""
    return lib().llattn_chunks_for(nblocks, bpc)


def wait_selftest(limit_ns: int, err_word, waited_ns, stream=None) -> None:
    """llattn_wait_selftest: four warps wait on barriers nothing completes, a fifth on a counter nothing counts into;
    err_word (int32 [1]) and waited_ns (int64 [6]) are device tensors."""
    _check(lib().llattn_wait_selftest(limit_ns, _ptr(err_word), _ptr(waited_ns), _stream(stream)))


# ------------------------------------------------------------------ commit

def kv_commit(Kf, Vf, cache, max_blocks: int, blk: int, stream=None) -> None:
    """attn::kv_commit<<<dim3(4, nb), 128>>>(Kf, Vf, cache, max_blocks, blk) (engine/attn.cu:369).
    Kf, Vf: fp16 [nb][32][4][128]; cache: uint8 [4][max_blocks][4736]."""
    nb = Kf.shape[0] if Kf.dim() == 4 else 1
    _check(lib().llattn_kv_commit(_ptr(Kf), _ptr(Vf), _ptr(cache), max_blocks, blk, nb, _stream(stream)))


def kv_commit_paged(Kf, Vf, pool, pages, stream=None) -> None:
    """Same quantiser into a record pool: pages is an int32 device tensor [nb][4] of record indices."""
    nb = Kf.shape[0]
    if pages.numel() != nb * NKV:
        raise ValueError("pages must hold nb * 4 indices")
    _check(lib().llattn_kv_commit_paged(_ptr(Kf), _ptr(Vf), _ptr(pool), _ptr(pages), nb, _stream(stream)))


def commit_needs_forward(final_ids, last_forward_ids) -> bool:
    """The decoder's commit policy (Decoder::commit, engine/decode.cu:267-280): when the last denoising forward of a
    block ran on exactly the ids the block ends with, the fresh K/V that forward left behind are the block's final K/V
    and only the quantiser has to run (`kv_commit` on them); otherwise one more forward pass on the final ids comes
    first (`qkv_prepare_commit` is that pass's producer and commit in one kernel). Host logic only."""
    a, b = [int(x) for x in final_ids], None if last_forward_ids is None else [int(x) for x in last_forward_ids]
    return b is None or len(a) != len(b) or a != b


def commit_block(final_ids, last_forward_ids, Kf, Vf, cache, max_blocks: int, blk: int, forward=None, stream=None) -> bool:
    """Commit one decoded block the way the reference decoder does. Kf, Vf: the fresh fp16 K/V [1][32][4][128] of the
    last denoising forward. If that forward did not run on `final_ids`, `forward(final_ids)` is called first and must
    refill Kf and Vf (raises if it is needed and missing). Returns True when only the quantiser ran."""
    kv_only = not commit_needs_forward(final_ids, last_forward_ids)
    if not kv_only:
        if forward is None:
            raise ValueError("the last forward did not run on the final ids: a forward pass is needed before the commit")
        forward(final_ids)
    kv_commit(Kf, Vf, cache, max_blocks, blk, stream)
    return kv_only


# ------------------------------------------------------------------ consumer

def dense_w4a8(W, q, s, qsum, Y, err_word=None, stream=None) -> None:
    """Engine::gemm<4, 2>(Ly.dense, ..., oA.a, ones, HID, HID, nullptr, h, 1, 2) (engine/engine.cu:434) for any number of
    tokens: Y [ntokens][rows] fp32 += W4.A8 projection of the int8 activations (q [ntokens][K] in fragment order, s and
    qsum [ntokens][K/128]) with the weight strips W in the engine's device layout. Bit-identical to the reference."""
    ntokens, K = q.shape
    rows = Y.shape[1]
    _check(lib().llattn_dense_w4a8(_ptr(W), _ptr(q), _ptr(s), _ptr(qsum), _ptr(Y), ntokens, rows, K,
                                   _ptr(err_word) if err_word is not None else None, _stream(stream)))


# ------------------------------------------------------------------ producer

def inv_freq(theta: float = 3e6):
    """The 32 RoPE frequencies the engine uploads (engine/engine.cu:275-277): theta^(-2i/64) as float32."""
    import numpy as np
    return np.array([np.float32(1.0 / (float(theta) ** (2.0 * i / 64.0))) for i in range(32)], np.float32)


def qk_norm_rope(qkv, pos, gq, gk, eps, inv_freq_t, q, k, v, stream=None) -> None:
    """ops::qk_norm_rope<<<dim3(T, 3), 256>>>(qkv, pos, gq, gk, eps, inv_freq, q, k, v) (engine/ops.cu:429).
    qkv fp32 [T][3072], pos int32 [T], gq/gk fp32 [128], inv_freq fp32 [32]; q fp16 [T][16][128], k/v fp16 [T][4][128]."""
    T = qkv.shape[0]
    _check(lib().llattn_qk_norm_rope(_ptr(qkv), _ptr(pos), _ptr(gq), _ptr(gk), eps, _ptr(inv_freq_t), _ptr(q), _ptr(k),
                                     _ptr(v), T, _stream(stream)))


def qkv_prepare_commit(qkv, pos, gq, gk, eps, inv_freq_t, q, k, v, cache, max_blocks: int = 0, blk: int = 0, pages=None,
                       stream=None) -> None:
    """The producer for whole 32-token blocks fused with their commit (engine/engine.cu:589-591 in one kernel): q, k, v as
    qk_norm_rope writes them, and block j becomes record blk + j of `cache` [4][max_blocks][4736] (or, with `pages`
    int32 [nb][4], record pages[j][h] of the pool `cache`)."""
    T = qkv.shape[0]
    if T % BLK:
        raise ValueError("a prefill pass commits whole 32-token blocks")
    _check(lib().llattn_qkv_prepare_commit(_ptr(qkv), _ptr(pos), _ptr(gq), _ptr(gk), eps, _ptr(inv_freq_t), _ptr(q), _ptr(k),
                                           _ptr(v), T // BLK, _ptr(cache), _ptr(pages), max_blocks, blk, _stream(stream)))


# ------------------------------------------------------------------ the reference operator pair

@dataclass
class Args:
    """attn::Args (engine/attn.cu:51-64); tensors instead of raw pointers."""
    Q: object
    Kf: object
    Vf: object
    cache: object
    max_blocks: int
    nblocks: int
    blocks_per_chunk: int
    nchunks: int
    scale: float
    Opart: object
    Mpart: object
    Lpart: object


def attn_partial(a: Args, nb: int = 1, err_word=None, stream=None) -> None:
    """attn::attn_partial<<<dim3(4, nchunks, nb)>>>(a) (engine/attn.cu:145)."""
    s = _Args(_ptr(a.Q), _ptr(a.Kf), _ptr(a.Vf), _ptr(a.cache), a.max_blocks, a.nblocks, a.blocks_per_chunk, a.nchunks,
              a.scale, _ptr(a.Opart), _ptr(a.Mpart), _ptr(a.Lpart))
    _check(lib().llattn_attn_partial(byref(s), nb, _ptr(err_word), _stream(stream)))


def attn_combine(Opart, Mpart, Lpart, nchunks: int, nblocks: int, bpc: int, O=None, q8=None, s8=None, sum8=None,
                 nb: int = 1, stream=None) -> None:
    """attn::attn_combine<<<dim3(4, 16, nb), 256>>>(...) (engine/attn.cu:319)."""
    _check(lib().llattn_attn_combine(_ptr(Opart), _ptr(Mpart), _ptr(Lpart), nchunks, nblocks, bpc, _ptr(O), _ptr(q8),
                                     _ptr(s8), _ptr(sum8), nb, _stream(stream)))


def attention_static(Q, Kf, Vf, cache, max_blocks: int, nblocks: int, O16=None, O32=None, LSE=None, q8=None, s8=None,
                     sum8=None, scale: float = 0.0, err_word=None, stream=None) -> None:
    """One sequence's attention with no device allocation anywhere in the call: partial results live in an array built
    into the library (10.16 MiB per GPU, shared by every call on that GPU, so calls that may overlap on the GPU race).
    For hosts that must not allocate: a fixed, audited memory plan, a foreign runtime's allocator, a no-allocation
    region. At most 16 query blocks (Q.shape[0]) per call; make the first call on a device before stream capture."""
    nb = Q.shape[0]
    _check(lib().llattn_attention_static(_ptr(Q), _ptr(Kf), _ptr(Vf), _ptr(cache), max_blocks, nblocks, nb, scale,
                                         _ptr(O16), _ptr(O32), _ptr(LSE), _ptr(q8), _ptr(s8), _ptr(sum8), _ptr(err_word),
                                         _stream(stream)))


# ------------------------------------------------------------------ batched path

@dataclass
class Seq:
    """One sequence of a batched call. `cache` is this layer's [4][head_stride][4736] uint8 tensor, or the record
    pool when `pages` (int32 [4][head_stride]) is given. Query block j of the sequence sees nblocks + j records."""
    cache: object
    nblocks: int
    nq: int = 1
    q_first: int = 0
    pages: object = None
    head_stride: Optional[int] = None

    def _c(self) -> _Seq:
        hs = self.head_stride
        if hs is None:
            hs = self.pages.shape[-1] if self.pages is not None else (self.cache.shape[1] if self.cache is not None else 0)
        return _Seq(_ptr(self.cache), _ptr(self.pages), hs, self.nblocks, self.nq, self.q_first)


def plan_preview(lengths, nctas: int, nq=None):
    """Host-only planner run (no GPU needed): lengths[i] = committed blocks of sequence i, nq[i] its query blocks.
    Returns (PlanStats, items int32 [n][8], cta_first int32 [nctas_used + 1])."""
    import numpy as np
    n = len(lengths)
    nq = [1] * n if nq is None else list(nq)
    q0, arr = 0, (_Seq * n)()
    for i in range(n):
        arr[i] = _Seq(0x1000, None, int(lengths[i]) + nq[i], int(lengths[i]), nq[i], q0)   # placeholder, aligned cache address
        q0 += nq[i]
    st = PlanStats()
    _check(lib().llattn_plan_preview(arr, n, nctas, byref(st), None, 0, None, 0))
    items = np.zeros((st.nitems, 8), np.int32)
    cta_first = np.zeros(st.nctas + 1, np.int32)
    _check(lib().llattn_plan_preview(arr, n, nctas, byref(st), items.ctypes.data, st.nitems, cta_first.ctypes.data, st.nctas))
    return st, items, cta_first


class Context:
    def __init__(self, device: int = 0):
        self._h = c_void_p()
        self.device = device
        _check(lib().llattn_create(device, byref(self._h)))

    def close(self) -> None:
        if self._h:
            lib().llattn_destroy(self._h)
            self._h = c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def plan(self, seqs: Sequence[Seq], nctas: int = 0) -> "Plan":
        return Plan(self, seqs, nctas)

    def attention(self, plan: "Plan", Q, Kf, Vf, O16=None, O32=None, LSE=None, q8=None, s8=None, sum8=None,
                  scale: float = 0.0, stream=None, precise: bool = False, cache_offset: int = 0) -> None:
        """One launch. precise: carry the softmax probabilities as fp16 value + fp16 remainder (LLATTN_IO_PRECISE_P).
        cache_offset: bytes added to every sequence's cache pointer (the layer, when one plan serves all layers)."""
        io = _IO(_ptr(Q), _ptr(Kf), _ptr(Vf), _ptr(O16), _ptr(O32), _ptr(LSE), _ptr(q8), _ptr(s8), _ptr(sum8), scale,
                 IO_PRECISE_P if precise else 0, cache_offset)
        _check(lib().llattn_attention(self._h, plan._h, byref(io), _stream(stream)))

    def attention_host(self, plan: "Plan", Q, Kf, Vf, O16=None, O32=None, LSE=None, q8=None, s8=None, sum8=None,
                       scale: float = 0.0, stream=None, precise: bool = False, cache_offset: int = 0) -> None:
        """Q/Kf/Vf and the outputs are HOST tensors (pinned for asynchronous copies)."""
        io = _IO(_ptr(Q), _ptr(Kf), _ptr(Vf), _ptr(O16), _ptr(O32), _ptr(LSE), _ptr(q8), _ptr(s8), _ptr(sum8), scale,
                 IO_PRECISE_P if precise else 0, cache_offset)
        _check(lib().llattn_attention_host(self._h, plan._h, byref(io), _stream(stream)))

    def host_flush(self, stream=None) -> None:
        """Orders every download issued by attention_host so far before later work on `stream`."""
        _check(lib().llattn_host_flush(self._h, _stream(stream)))

    def device_status(self, stream=None) -> int:
        code = c_int(0)
        _check(lib().llattn_device_status(self._h, _stream(stream), byref(code)))
        return code.value


class Plan:
    def __init__(self, ctx: Context, seqs: Sequence[Seq], nctas: int = 0):
        self.ctx = ctx
        self._keep = list(seqs)          # keeps the cache / page tensors alive
        arr = (_Seq * len(seqs))(*[s._c() for s in seqs])
        self._h = c_void_p()
        _check(lib().llattn_plan_create(ctx._h, arr, len(seqs), nctas, byref(self._h)))
        st = PlanStats()
        _check(lib().llattn_plan_get_stats(self._h, byref(st)))
        self.stats = st

    def update(self, seqs: Sequence[Seq], stream=None) -> None:
        """New lengths / pointers for the same sequences (llattn_plan_update): no allocation, one asynchronous copy
        on `stream`; a captured graph that uses this plan stays valid."""
        arr = (_Seq * len(seqs))(*[s._c() for s in seqs])
        _check(lib().llattn_plan_update(self._h, arr, len(seqs), _stream(stream)))
        self._keep = list(seqs)
        st = PlanStats()
        _check(lib().llattn_plan_get_stats(self._h, byref(st)))
        self.stats = st

    def close(self) -> None:
        if self._h:
            lib().llattn_plan_destroy(self._h)
            self._h = c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class KvPool:
    """Host-side page manager with prefix reuse (llattn_kvpool_*): pages are committed 32-token blocks, shared by
    sequences with a common prefix of token blocks, recycled least-recently-used once no open sequence holds them.
    A page is reported as reused, and kept after its last holder closes, only after mark_committed said its records exist.
    Record of (page p, kv head h) in any layer's pool: p * 4 + h."""

    def __init__(self, npages: int):
        self._h = c_void_p()
        _check(lib().llattn_kvpool_create(npages, byref(self._h)))

    def close_pool(self) -> None:
        if self._h:
            lib().llattn_kvpool_destroy(self._h)
            self._h = c_void_p()

    def __del__(self):
        try:
            self.close_pool()
        except Exception:
            pass

    def open(self, tokens):
        """-> (seq_id, reused_blocks, pages of the prompt's full blocks)."""
        import numpy as np
        tok = np.ascontiguousarray(tokens, np.int32)
        full = len(tok) // 32
        pages = np.zeros(max(full, 1), np.int32)
        sid, reused = c_int32(0), c_int32(0)
        _check(lib().llattn_kvpool_open(self._h, tok.ctypes.data, len(tok), byref(sid), byref(reused), pages.ctypes.data, full))
        return sid.value, reused.value, pages[:full].copy()

    def append(self, seq_id: int, block_tokens):
        import numpy as np
        tok = np.ascontiguousarray(block_tokens, np.int32)
        if tok.size != 32:
            raise ValueError("a block is 32 token ids")
        page, reused = c_int32(0), c_int32(0)
        _check(lib().llattn_kvpool_append(self._h, seq_id, tok.ctypes.data, byref(page), byref(reused)))
        return page.value, bool(reused.value)

    def mark_committed(self, seq_id: int, nblocks: int = -1) -> None:
        """The records of the sequence's first `nblocks` pages (default: all) exist now; only such pages are reused."""
        _check(lib().llattn_kvpool_mark_committed(self._h, seq_id, nblocks))

    def pages(self, seq_id: int):
        import numpy as np
        n = c_int32(0)
        _check(lib().llattn_kvpool_pages(self._h, seq_id, None, 0, byref(n)))
        out = np.zeros(max(n.value, 1), np.int32)
        _check(lib().llattn_kvpool_pages(self._h, seq_id, out.ctypes.data, n.value, byref(n)))
        return out[:n.value].copy()

    def close(self, seq_id: int) -> None:
        _check(lib().llattn_kvpool_close(self._h, seq_id))

    def stats(self) -> dict:
        import numpy as np
        o = np.zeros(6, np.int64)
        _check(lib().llattn_kvpool_stats(self._h, o.ctypes.data))
        return dict(zip(("pages", "free", "cached", "hits", "misses", "evictions"), (int(x) for x in o)))

    @staticmethod
    def page_table(pages, head_stride=None):
        """int32 [4][head_stride] record indices (page * 4 + head) for llattn_seq.pages / Seq(pages=...)."""
        import numpy as np
        pages = np.asarray(pages, np.int32)
        hs = len(pages) if head_stride is None else head_stride
        t = np.zeros((NKV, hs), np.int32)
        t[:, :len(pages)] = pages[None, :] * NKV + np.arange(NKV, dtype=np.int32)[:, None]
        return t
