"""Generates the golden fixtures of this folder by importing the REFERENCE's own simulated quantiser.

Run in a container that has the reference checkout (it cannot run on the GPU box):
    PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_golden.py --ref <reference checkout>

What it writes (small, committed):
  fakequant_cases.npz  fp16 K/V blocks (seeded + hand-made edge groups) and, for each, the fp32 output of the
                       reference's fake_quant (quant/s06_arbitrate.py:78-89) applied the way the engine's cache
                       groups values: K per channel over the block's 32 tokens, V per token over 128 dims
                       (quant/student_case.py:63-66 with the value rotation taken as the identity).
  simquant_attn.npz    output and log-sum-exp of torch fp32 scaled-dot-product attention over
                       [fake-quantised context | fresh block] for one seeded query block, the flow of
                       quant/student_case.py:68-73 (block_attention) with GQA by head repeat.
Inputs are regenerated from the workload generator's seeds by the tests, so only the expected outputs (and the
hand-made edge inputs) are stored.
"""
import argparse
import importlib
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
wl = importlib.import_module("llada2-orin-cuda_b200").workload

ap = argparse.ArgumentParser()
ap.add_argument("--ref", required=True, help="path of the reference checkout (its quant/ directory is imported)")
a = ap.parse_args()
sys.path.insert(0, os.path.join(a.ref, "quant"))
sys.dont_write_bytecode = True
import s06_arbitrate as S  # noqa: E402  (the reference module; only fake_quant is used)


def ref_quant_blocks(K16: np.ndarray, V16: np.ndarray):
    """K16, V16 float16 [nb][32][4][128] -> reference-dequantised fp32 in the same layout."""
    K = torch.from_numpy(K16.astype(np.float32))
    V = torch.from_numpy(V16.astype(np.float32))
    kt = K.permute(0, 2, 3, 1).contiguous()                       # [nb][4][128][32]: group = 32 tokens per channel
    Kq = S.fake_quant(kt, 4, 32).permute(0, 3, 1, 2).contiguous()
    Vq = S.fake_quant(V, 4, 128)
    return Kq.numpy(), Vq.numpy()


def edge_blocks():
    """Hand-made groups that exercise the scale floor, clamping and fp16 rounding of scale/min."""
    g = np.random.default_rng(1234)
    K = g.standard_normal((6, 32, 4, 128)).astype(np.float16)
    V = g.standard_normal((6, 32, 4, 128)).astype(np.float16)
    K[0] = 0                                     # all-zero groups: scale floor, codes 0
    V[0] = 0
    K[1] = np.float16(3.25)                      # constant groups
    V[1] = np.float16(-0.0625)
    K[2] = (g.standard_normal((32, 4, 128)) * 1e-4).astype(np.float16)     # tiny range near the floor
    V[2] = (g.standard_normal((32, 4, 128)) * 1e-4).astype(np.float16)
    K[3] = (g.standard_normal((32, 4, 128)) * 300).astype(np.float16)      # large magnitudes
    V[3] = (g.standard_normal((32, 4, 128)) * 300).astype(np.float16)
    K[4, :, :, 5] = K[4, :, :, 5] * np.float16(8) + np.float16(3)          # the reference test's outlier channel
    V[4, 0] = np.float16(60000)                                           # huge constant token
    V[4, 1, :, :64] = np.float16(-60000)                                   # range beyond fp16 (fp32 range 1.2e5)
    V[4, 1, :, 64:] = np.float16(60000)
    K[5] = np.abs(K[5])                                                    # one-signed groups
    V[5] = -np.abs(V[5])
    return K, V


Ke, Ve = edge_blocks()
Ks, Vs = wl.context_blocks(8, seq=3, layer=1)
cases = {}
for name, (K, V) in {"edge": (Ke, Ve), "seeded": (Ks, Vs)}.items():
    Kq, Vq = ref_quant_blocks(K, V)
    cases[f"{name}_Kq"], cases[f"{name}_Vq"] = Kq, Vq
cases["edge_K"], cases["edge_V"] = Ke, Ve
cases["seeded_args"] = np.array([8, 3, 1], np.int32)            # nblocks, seq, layer of workload.context_blocks
np.savez_compressed(os.path.join(HERE, "fakequant_cases.npz"), **cases)

# simulated-quantisation attention, one query block over 8 committed blocks
NB = 8
Kc, Vc = wl.context_blocks(NB, seq=5, layer=2)
Q, Kf, Vf = wl.query_blocks(1, seq=5, layer=2)
Kq, Vq = ref_quant_blocks(Kc, Vc)
k = torch.cat([torch.from_numpy(Kq).reshape(-1, 4, 128), torch.from_numpy(Kf[0].astype(np.float32))], 0)
v = torch.cat([torch.from_numpy(Vq).reshape(-1, 4, 128), torch.from_numpy(Vf[0].astype(np.float32))], 0)
q = torch.from_numpy(Q[0].astype(np.float32)).permute(1, 0, 2)[None]            # [1][16][32][128]
k = k.permute(1, 0, 2).repeat_interleave(4, 0)[None]                            # [1][16][ctx][128]
v = v.permute(1, 0, 2).repeat_interleave(4, 0)[None]
torch.backends.cuda.enable_math_sdp(True)
O = torch.nn.functional.scaled_dot_product_attention(q, k, v)                   # default scale 1/sqrt(128)
lse = torch.logsumexp((q @ k.transpose(-1, -2)) / (128 ** 0.5), -1)
np.savez_compressed(os.path.join(HERE, "simquant_attn.npz"),
                    O=O[0].permute(1, 0, 2).contiguous().numpy().astype(np.float32),   # [32][16][128]
                    LSE=lse[0].permute(1, 0).contiguous().numpy().astype(np.float32),  # [32][16]
                    args=np.array([NB, 5, 2], np.int32))
print("wrote", os.listdir(HERE))
