"""The reference's CPU flow for this path, restated with the same torch operators it uses. TEST / CPU-BASELINE
INFRASTRUCTURE ONLY (bench.py's CPU-baseline and reference arms time it; nothing that ships calls it).

Follows quant/s06_arbitrate.py:78-89 (fake_quant: per-group asymmetric 4-bit with fp16 scale and min, returned as
fp32 q*s + mn) and quant/student_case.py:49-74 (block_attention: K quantised per channel over each committed
32-token block, V per token, the query block attends [quantised context | its own fresh K/V] through
scaled_dot_product_attention with the GQA heads repeated). The value rotation of student_case.py:65-66 is the
identity for synthetic inputs that are taken to be in the engine's basis already.
"""
import torch

FP16_MIN_SCALE = 6.2e-5


def fake_quant(x: torch.Tensor, bits: int, group: int) -> torch.Tensor:
    sh = x.shape
    xf = x.float().reshape(*sh[:-1], sh[-1] // group, group)
    mn, mx = xf.amin(-1, keepdim=True), xf.amax(-1, keepdim=True)
    maxq = 2 ** bits - 1
    s = ((mx - mn) / maxq).clamp_min(FP16_MIN_SCALE).half().float()
    mn = mn.half().float()
    q = torch.round((xf - mn) / s).clamp(0, maxq)
    return (q * s + mn).reshape(sh)


def block_attention(Q: torch.Tensor, Kf: torch.Tensor, Vf: torch.Tensor, Kctx: torch.Tensor, Vctx: torch.Tensor):
    """Q fp16 [32][16][128]; Kf, Vf fp16 [32][4][128]; Kctx, Vctx fp16 [nblk][32][4][128] (CPU tensors).
    Returns O fp32 [32][16][128]."""
    nblk = Kctx.shape[0]
    k = Kctx.float().permute(2, 0, 1, 3)                                    # [4][nblk][32][128]
    v = Vctx.float().permute(2, 0, 1, 3)
    kq = fake_quant(k.transpose(-1, -2), 4, 32).transpose(-1, -2)           # group = 32 tokens per channel
    vq = fake_quant(v, 4, 128)
    K = torch.cat([kq.reshape(4, nblk * 32, 128), Kf.float().permute(1, 0, 2)], 1)
    V = torch.cat([vq.reshape(4, nblk * 32, 128), Vf.float().permute(1, 0, 2)], 1)
    q = Q.float().permute(1, 0, 2)[None]                                    # [1][16][32][128]
    K = K.repeat_interleave(4, 0)[None]
    V = V.repeat_interleave(4, 0)[None]
    O = torch.nn.functional.scaled_dot_product_attention(q, K, V)
    return O[0].permute(1, 0, 2).contiguous()
