"""ctypes face of oracle/_ref/libattn_ref.so: the reference's own attn.cu kernels compiled for sm_100a by
oracle/Makefile (`make ref`) where the reference checkout exists. Test and measurement infrastructure only: the GPU
parity tests use it as the reference-kernel oracle and bench.py times it beside the new kernel. `available()` is
False when the file did not travel; tests that need it skip."""
import ctypes
import os

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PATH = os.path.join(ROOT, "oracle", "_ref", "libattn_ref.so")
_lib = None


def available() -> bool:
    return os.path.exists(PATH)


def lib():
    global _lib
    if _lib is None:
        L = ctypes.CDLL(PATH)
        vp, i = ctypes.c_void_p, ctypes.c_int
        L.ref_pick_bpc.argtypes = [i, i]
        L.ref_chunks_for.argtypes = [i, i]
        L.ref_kv_commit.argtypes = [vp, vp, vp, i, i, i, vp]
        L.ref_attention.argtypes = [vp, vp, vp, vp, i, i, i, i, vp, vp, vp, vp, vp, vp, vp, vp]
        _lib = L
    return _lib


def kv_commit(Kf, Vf, cache, max_blocks, blk):
    import torch
    rc = lib().ref_kv_commit(Kf.data_ptr(), Vf.data_ptr(), cache.data_ptr(), max_blocks, blk, Kf.shape[0],
                             torch.cuda.current_stream().cuda_stream)
    assert rc == 0, rc


def attention(Q, Kf, Vf, cache, max_blocks, nblocks, bpc=0, int8=False):
    """Runs attn_partial + attn_combine of the reference. Returns fp16 O [nb*32][16][128] (or (q8, s8, sum8))."""
    import torch
    nb = Q.shape[0]
    L = lib()
    if bpc <= 0:
        bpc = L.ref_pick_bpc(nblocks + nb - 1, nb)
    nch = L.ref_chunks_for(nblocks + nb - 1, bpc)
    dev = Q.device
    Op = torch.empty((nb, 4, nch, 128, 128), dtype=torch.float32, device=dev)
    Mp = torch.empty((nb, 4, nch, 128), dtype=torch.float32, device=dev)
    Lp = torch.empty((nb, 4, nch, 128), dtype=torch.float32, device=dev)
    O = torch.empty((nb * 32, 16, 128), dtype=torch.float16, device=dev)
    q8 = s8 = sum8 = None
    if int8:
        q8 = torch.empty((nb * 32, 2048), dtype=torch.int8, device=dev)
        s8 = torch.empty((nb * 32, 16), dtype=torch.float32, device=dev)
        sum8 = torch.empty((nb * 32, 16), dtype=torch.int32, device=dev)
    rc = L.ref_attention(Q.data_ptr(), Kf.data_ptr(), Vf.data_ptr(), cache.data_ptr(), max_blocks, nblocks, nb, bpc,
                         Op.data_ptr(), Mp.data_ptr(), Lp.data_ptr(), O.data_ptr(),
                         q8.data_ptr() if int8 else None, s8.data_ptr() if int8 else None,
                         sum8.data_ptr() if int8 else None, torch.cuda.current_stream().cuda_stream)
    assert rc == 0, rc
    torch.cuda.synchronize()
    return (q8, s8, sum8) if int8 else O


class BatchRunner:
    """The reference's attn_partial + attn_combine for a batch of independent sequences, one query block each: the
    reference serves one sequence per launch pair, so a batch is one launch pair per sequence, spread over `nstreams`
    streams so that the GPU can overlap them. Partial buffers are allocated once."""

    def __init__(self, nseq, nblocks, device, nstreams=8):
        import torch
        L = lib()
        self.bpc = L.ref_pick_bpc(nblocks, 1)
        self.nch = L.ref_chunks_for(nblocks, self.bpc)
        self.nblocks = nblocks
        self.Op = torch.empty((nseq, 4, self.nch, 128, 128), dtype=torch.float32, device=device)
        self.Mp = torch.empty((nseq, 4, self.nch, 128), dtype=torch.float32, device=device)
        self.Lp = torch.empty((nseq, 4, self.nch, 128), dtype=torch.float32, device=device)
        self.O = torch.empty((nseq * 32, 16, 128), dtype=torch.float16, device=device)
        self.streams = [torch.cuda.Stream(device=device) for _ in range(nstreams)]

    def launch(self, Q, Kf, Vf, caches, max_blocks):
        """Q [nseq][32][16][128], Kf/Vf [nseq][32][4][128], caches [nseq][4][max_blocks][4736]; launches only."""
        L = lib()
        for s in range(Q.shape[0]):
            st = self.streams[s % len(self.streams)]
            rc = L.ref_attention(Q[s].data_ptr(), Kf[s].data_ptr(), Vf[s].data_ptr(), caches[s].data_ptr(), max_blocks,
                                 self.nblocks, 1, self.bpc, self.Op[s].data_ptr(), self.Mp[s].data_ptr(), self.Lp[s].data_ptr(),
                                 self.O[32 * s:32 * s + 32].data_ptr(), None, None, None, st.cuda_stream)
            assert rc == 0, rc


OPS_PATH = os.path.join(ROOT, "oracle", "_ref", "libops_ref.so")
_ops = None


def ops_available() -> bool:
    return os.path.exists(OPS_PATH)


def qk_norm_rope(qkv, pos, gq, gk, eps, inv_freq, q, k, v):
    """The reference's own ops::qk_norm_rope (engine/ops.cu:429) on device tensors."""
    import torch
    global _ops
    if _ops is None:
        _ops = ctypes.CDLL(OPS_PATH)
        vp = ctypes.c_void_p
        _ops.ref_qk_norm_rope.argtypes = [vp, vp, vp, vp, ctypes.c_float, vp, vp, vp, vp, ctypes.c_int, vp]
    rc = _ops.ref_qk_norm_rope(qkv.data_ptr(), pos.data_ptr(), gq.data_ptr(), gk.data_ptr(), eps, inv_freq.data_ptr(),
                               q.data_ptr(), k.data_ptr(), v.data_ptr(), qkv.shape[0], torch.cuda.current_stream().cuda_stream)
    assert rc == 0, rc


GEMM_PATH = os.path.join(ROOT, "oracle", "_ref", "libgemm_ref.so")
_gemm = None


def gemm_available() -> bool:
    return os.path.exists(GEMM_PATH)


def dense_aux(ntokens, dev):
    """Work items of 32 tokens, a one-entry expert table and unit slot weights for dense_w4a8 (device tensors)."""
    import numpy as np
    import torch
    work = torch.from_numpy(np.array([[0, 32 * j, 32] for j in range(ntokens // 32)], np.int32)).to(dev)
    return (work, torch.zeros(1, dtype=torch.int64, device=dev), torch.full((1,), 4, dtype=torch.int8, device=dev),
            torch.ones(ntokens, dtype=torch.float32, device=dev))


def dense_w4a8(W, q, s, qsum, Y, aux=None, sync=True):
    """The reference's own moe8::gemm<4, 4, 2, 2> (engine/moe_i8.cu:408), launched as the engine launches its attention
    output projection (engine/engine.cu:434): Y += projection, tokens in work items of 32."""
    import torch
    global _gemm
    if _gemm is None:
        _gemm = ctypes.CDLL(GEMM_PATH)
        vp, i = ctypes.c_void_p, ctypes.c_int
        _gemm.ref_dense_w4a8.argtypes = [vp, vp, vp, vp, vp, i, i, i, vp, vp, vp, vp, i, vp]
    ntokens, K = q.shape
    rows = Y.shape[1]
    work, off, bits, ones = aux if aux is not None else dense_aux(ntokens, q.device)
    rc = _gemm.ref_dense_w4a8(W.data_ptr(), q.data_ptr(), s.data_ptr(), qsum.data_ptr(), Y.data_ptr(), ntokens, rows, K,
                              work.data_ptr(), off.data_ptr(), bits.data_ptr(), ones.data_ptr(), 2,
                              torch.cuda.current_stream().cuda_stream)
    assert rc == 0, rc
    if sync:
        torch.cuda.synchronize()
