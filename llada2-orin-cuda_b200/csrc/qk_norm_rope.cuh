// Producer of the attention inputs: per-head RMSNorm of q and k, partial RoPE on the first 64 dims (rotate-half pairs
// (d, d + 32), cos/sin rounded to bf16 as the reference model computes them), v passed through; fp32 qkv in, the
// fp16 Q / fresh K / fresh V of the attention step out. Replaces the reference's ops::qk_norm_rope
// (engine/ops.cu:429-453) with the same arithmetic in the same order, so outputs are bit-identical to it.
// qkv: [T][3072] fp32 (16 q heads, 4 k heads, 4 v heads of 128). One warp per (token, head): lane l holds dims
// l, l+32, l+64, l+96, so every load and store of a warp is one contiguous 128- or 64-byte segment and the rotate-half
// partners share a lane. HBM-bound: 12,288 B read + 6,144 B written per token.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include "common.cuh"

namespace llattn {

constexpr int ROPE_THREADS = 256;          // 8 heads per CTA; grid (T, 3) covers the 24 heads of a token

__global__ void __launch_bounds__(ROPE_THREADS)
qk_norm_rope_kernel(const float* __restrict__ qkv, const int* __restrict__ pos, const float* __restrict__ gq,
                    const float* __restrict__ gk, float eps, const float* __restrict__ inv_freq, half* __restrict__ q,
                    half* __restrict__ k, half* __restrict__ v) {
    const int t = blockIdx.x, hd = blockIdx.y * 8 + (threadIdx.x >> 5), l = threadIdx.x & 31;
    const float* src = qkv + size_t(t) * 3072 + hd * 128;
    float x[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) x[i] = src[l + 32 * i];
    if (hd >= 20) {                                     // v head: conversion only
#pragma unroll
        for (int i = 0; i < 4; ++i) v[(size_t(t) * NKV + (hd - 20)) * D + l + 32 * i] = __float2half(x[i]);
        return;
    }
    float ss = x[0] * x[0] + x[1] * x[1] + x[2] * x[2] + x[3] * x[3];
#pragma unroll
    for (int o = 16; o; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    const float r = rsqrtf(ss / 128.f + eps);
    const float* gm = hd < 16 ? gq : gk;
    float n[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) n[i] = x[i] * r * gm[l + 32 * i];
    float sn, cs;
    sincosf(float(pos[t]) * inv_freq[l], &sn, &cs);
    cs = __bfloat162float(__float2bfloat16(cs));
    sn = __bfloat162float(__float2bfloat16(sn));
    const float o0 = n[0] * cs - n[1] * sn, o1 = n[1] * cs + n[0] * sn;
    half* dst = hd < 16 ? q + (size_t(t) * NQH + hd) * D : k + (size_t(t) * NKV + (hd - 16)) * D;
    dst[l] = __float2half(o0);
    dst[l + 32] = __float2half(o1);
    dst[l + 64] = __float2half(n[2]);
    dst[l + 96] = __float2half(n[3]);
}

}  // namespace llattn
