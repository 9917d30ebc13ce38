// Producer of the attention inputs, fused with the block commit for prefill.
//
// Stands in for the reference's ops::qk_norm_rope (engine/ops.cu:429-453): per head RMSNorm of q and k with a learned
// gain, rotary embedding on the first 64 dims of each head (rotate-half pairs (d, d + 32), cos/sin rounded to bf16 as
// the model computes them), v converted; fp32 qkv [T][3072] (16 q heads, 4 k heads, 4 v heads of 128) in, fp16 Q [T][16][128]
// and fresh K, V [T][4][128] out. In a prefill pass the reference then runs attn::kv_commit on those fp16 K/V
// (engine/engine.cu:589-591), reading them back from memory; here the CTA that produces a 32-token block of one kv
// head keeps the fp16 K and V it has just rounded in shared memory and quantises the block's record from there
// (kv_commit.cuh), so a prefill block goes from fp32 qkv to its 4736-byte record in one pass: 12,288 B read and
// 6,144 + 592 B written per token, against 14,336 read and the same written by the two-kernel sequence.
//
// Grid (blocks of 32 tokens, 8): y < 4 is a group of four q heads, y >= 4 the k and v head of kv head y - 4.
// 256 threads; a warp takes whole (token, head) rows, lane l holding dims l, l+32, l+64, l+96: the rotate-half partners
// then share a lane and every global access of a warp is one contiguous segment. The float operations and their order
// are the reference kernel's (sum of squares folded lane-wise then by a xor butterfly, rsqrtf, x*r*g, sincosf, one
// fused multiply-add per rotated output), which is what makes the outputs bit-identical to it.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include "common.cuh"
#include "kv_commit.cuh"

namespace llattn {

constexpr int PREP_THREADS = 256;

struct PrepArgs {
    const float* qkv;        // [T][3072]
    const int* pos;          // [T]
    const float* gq;         // [128]
    const float* gk;         // [128]
    const float* inv_freq;   // [32]
    float eps;
    half* q;                 // [T][16][128]
    half* k;                 // [T][4][128]
    half* v;                 // [T][4][128]
    int T;
    // commit of the blocks this launch produces (records == nullptr: none). Block j of the launch, head h:
    // pages ? records + pages[j * 4 + h] * 4736 : records + (h * max_blocks + blk + j) * 4736
    uint8_t* records;
    const int32_t* pages;
    int max_blocks, blk;
};

// One head row of a token: the four values a lane holds, normalised and rotated in place.
__device__ __forceinline__ void norm_rope_lane(float (&x)[4], const float* __restrict__ gain, int lane, float eps, float cs, float sn) {
    float ss = x[0] * x[0] + x[1] * x[1] + x[2] * x[2] + x[3] * x[3];
#pragma unroll
    for (int o = 16; o; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    const float r = rsqrtf(ss / 128.f + eps);
#pragma unroll
    for (int i = 0; i < 4; ++i) x[i] = x[i] * r * gain[lane + 32 * i];
    // written out: the first product of each pair goes into the fused multiply-add, the second is rounded on its own.
    // That is what the compiler makes of the reference's `n0 * cs - n1 * sn` and `n1 * cs + n0 * sn`, and the other
    // choice differs from it in the last fp16 bit of about one output in 20,000.
    const float lo = __fmaf_rn(x[0], cs, -__fmul_rn(x[1], sn));
    const float hi = __fmaf_rn(x[1], cs, __fmul_rn(x[0], sn));
    x[0] = lo; x[1] = hi;
}

__global__ void __launch_bounds__(PREP_THREADS) qkv_prepare_kernel(const PrepArgs a) {
    __shared__ CommitSmem sm;
    const int jb = blockIdx.x, grp = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t0 = jb * BLK;
    const float freq = a.inv_freq[lane];
    if (grp < 4) {
        // ---- four q heads x 32 tokens = 128 rows, 16 per warp
        for (int i = warp; i < 4 * BLK; i += PREP_THREADS / 32) {
            const int t = t0 + (i >> 2), hd = 4 * grp + (i & 3);
            if (t >= a.T) break;
            const float* src = a.qkv + size_t(t) * 3072 + hd * D;
            float x[4];
#pragma unroll
            for (int c = 0; c < 4; ++c) x[c] = src[lane + 32 * c];
            float sn, cs;
            sincosf(float(a.pos[t]) * freq, &sn, &cs);
            cs = __bfloat162float(__float2bfloat16(cs));
            sn = __bfloat162float(__float2bfloat16(sn));
            norm_rope_lane(x, a.gq, lane, a.eps, cs, sn);
            half* dst = a.q + (size_t(t) * NQH + hd) * D;
#pragma unroll
            for (int c = 0; c < 4; ++c) dst[lane + 32 * c] = __float2half(x[c]);
        }
        return;
    }
    // ---- kv head h: the block's K (normalised, rotated) and V (converted) as fp16 tiles in shared memory
    const int h = grp - 4;
    for (int tok = warp; tok < BLK; tok += PREP_THREADS / 32) {
        const int t = t0 + tok;
        float xk[4], xv[4];
        if (t < a.T) {
            const float* ks = a.qkv + size_t(t) * 3072 + (NQH + h) * D;
            const float* vs = a.qkv + size_t(t) * 3072 + (NQH + NKV + h) * D;
#pragma unroll
            for (int c = 0; c < 4; ++c) { xk[c] = ks[lane + 32 * c]; xv[c] = vs[lane + 32 * c]; }
            float sn, cs;
            sincosf(float(a.pos[t]) * freq, &sn, &cs);
            cs = __bfloat162float(__float2bfloat16(cs));
            sn = __bfloat162float(__float2bfloat16(sn));
            norm_rope_lane(xk, a.gk, lane, a.eps, cs, sn);
        } else {
#pragma unroll
            for (int c = 0; c < 4; ++c) { xk[c] = 0.f; xv[c] = 0.f; }
        }
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            sm.Ks[tok][lane + 32 * c] = __float2half(xk[c]);
            sm.Vs[tok][lane + 32 * c] = __float2half(xv[c]);
        }
    }
    __syncthreads();
    // ---- fp16 K and V of the block to global memory, 16 bytes per thread and store
    for (int i = threadIdx.x; i < BLK * 16; i += PREP_THREADS) {
        const int tok = i >> 4, ch = i & 15, t = t0 + tok;
        if (t >= a.T) continue;
        *reinterpret_cast<uint4*>(a.k + (size_t(t) * NKV + h) * D + ch * 8) = *reinterpret_cast<const uint4*>(&sm.Ks[tok][ch * 8]);
        *reinterpret_cast<uint4*>(a.v + (size_t(t) * NKV + h) * D + ch * 8) = *reinterpret_cast<const uint4*>(&sm.Vs[tok][ch * 8]);
    }
    if (a.records) {
        const size_t ridx = a.pages ? size_t(a.pages[jb * NKV + h]) : size_t(h) * a.max_blocks + a.blk + jb;
        commit_tiles(sm, a.records + ridx * REC_BYTES, threadIdx.x, PREP_THREADS);
    }
}

}  // namespace llattn
