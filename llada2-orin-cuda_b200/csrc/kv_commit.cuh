// Block-commit quantiser: a finished block's fp16 K/V -> one 4736-byte "4c/4" record per kv head.
// Replaces the reference's attn::kv_commit (engine/attn.cu:369-418) and must produce the same bytes:
//   K: per channel over the block's 32 tokens, V: per token over the 128 dims;
//   scale = half(max((max - min) / 15, 6.2e-5f)), min = half(min), code = clamp(rint((v - min) / scale), 0, 15),
//   all in IEEE fp32 with round-to-nearest-even; two codes per byte, even channel in the low nibble.
// One CTA of 128 threads per (kv head, block). The record is assembled in shared memory and leaves as 16-byte
// stores; the inputs arrive as 16-byte loads.
#pragma once
#include <cuda_fp16.h>
#include "common.cuh"

namespace llattn {

constexpr int COMMIT_THREADS = 128;

__device__ __forceinline__ void commit_meta(float mn, float mx, half& sh, half& mh) {
    sh = __float2half_rn(fmaxf(__fdiv_rn(__fsub_rn(mx, mn), 15.f), 6.2e-5f));
    mh = __float2half_rn(mn);
}
__device__ __forceinline__ uint32_t commit_code(float v, float m0, float s) {
    return uint32_t(max(0, min(15, __float2int_rn(__fdiv_rn(__fsub_rn(v, m0), s)))));
}

// Kf, Vf: [nb][32 tok][4 heads][128] fp16. Record of (input block j, head h):
//   pages == nullptr: records + (h * max_blocks + blk + j) * 4736      (the reference's contiguous layer cache)
//   pages != nullptr: records + pages[j * 4 + h] * 4736                (record pool)
__device__ __forceinline__ void kv_commit_body(const half* __restrict__ Kf, const half* __restrict__ Vf,
                                               uint8_t* __restrict__ records, const int32_t* __restrict__ pages,
                                               int max_blocks, int blk) {
    __shared__ __align__(16) half Ks[BLK][D + 8];            // +8 halves: rows 272 B apart, 16-byte aligned
    __shared__ __align__(16) uint8_t kq[BLK][D];             // one code per byte before packing
    __shared__ __align__(16) uint8_t rec[REC_BYTES];
    const int h = blockIdx.x, j = blockIdx.y, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const size_t in0 = size_t(j) * BLK * NKV * D + size_t(h) * D;
    const size_t ridx = pages ? size_t(pages[j * NKV + h]) : size_t(h) * max_blocks + blk + j;
    uint8_t* dst = records + ridx * REC_BYTES;

    // ---- K slice into shared memory (32 tokens x 256 B, 16-byte loads)
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int idx = tid + COMMIT_THREADS * i, tok = idx >> 4, ch = idx & 15;
        *reinterpret_cast<uint4*>(&Ks[tok][ch * 8]) =
            *reinterpret_cast<const uint4*>(Kf + in0 + size_t(tok) * NKV * D + ch * 8);
    }
    // ---- V: warp w owns tokens 8w .. 8w+7, a lane owns dims 4*lane .. 4*lane+3
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int tok = warp * 8 + i;
        const uint2 raw = *reinterpret_cast<const uint2*>(Vf + in0 + size_t(tok) * NKV * D + lane * 4);
        const half2 a = *reinterpret_cast<const half2*>(&raw.x), b = *reinterpret_cast<const half2*>(&raw.y);
        const float v0 = __low2float(a), v1 = __high2float(a), v2 = __low2float(b), v3 = __high2float(b);
        float mn = fminf(fminf(v0, v1), fminf(v2, v3)), mx = fmaxf(fmaxf(v0, v1), fmaxf(v2, v3));
#pragma unroll
        for (int o = 16; o; o >>= 1) {
            mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        }
        half sh, mh;
        commit_meta(mn, mx, sh, mh);
        const float s = __half2float(sh), m0 = __half2float(mh);
        const uint32_t packed = commit_code(v0, m0, s) | (commit_code(v1, m0, s) << 4) |
                                (commit_code(v2, m0, s) << 8) | (commit_code(v3, m0, s) << 12);
        *reinterpret_cast<uint16_t*>(rec + VOFF + tok * 64 + lane * 2) = uint16_t(packed);
        if (lane == 0) {
            reinterpret_cast<half*>(rec + VOFF_META)[tok] = sh;
            reinterpret_cast<half*>(rec + VOFF_META)[BLK + tok] = mh;
        }
    }
    __syncthreads();
    // ---- K: thread c owns channel c
    {
        const int c = tid;
        float mn = INFINITY, mx = -INFINITY;
#pragma unroll
        for (int tk = 0; tk < BLK; ++tk) {
            const float v = __half2float(Ks[tk][c]);
            mn = fminf(mn, v); mx = fmaxf(mx, v);
        }
        half sh, mh;
        commit_meta(mn, mx, sh, mh);
        const float s = __half2float(sh), m0 = __half2float(mh);
#pragma unroll
        for (int tk = 0; tk < BLK; ++tk) kq[tk][c] = uint8_t(commit_code(__half2float(Ks[tk][c]), m0, s));
        reinterpret_cast<half*>(rec + KOFF_META)[c] = sh;
        reinterpret_cast<half*>(rec + KOFF_META)[D + c] = mh;
    }
    __syncthreads();
    // ---- pack K codes: thread -> 16 output bytes = 32 codes
    {
        const int tok = tid >> 2, part = tid & 3;             // 4 threads per token, 32 channels each
        const uint4 a = *reinterpret_cast<const uint4*>(&kq[tok][part * 32]);
        const uint4 b = *reinterpret_cast<const uint4*>(&kq[tok][part * 32 + 16]);
        auto pk = [](uint32_t x) -> uint32_t {                // 4 codes (one per byte) -> 2 packed bytes
            return (x & 0xfu) | ((x >> 4) & 0xf0u) | ((x >> 8) & 0xf00u) | ((x >> 12) & 0xf000u);
        };
        uint4 o;
        o.x = pk(a.x) | (pk(a.y) << 16); o.y = pk(a.z) | (pk(a.w) << 16);
        o.z = pk(b.x) | (pk(b.y) << 16); o.w = pk(b.z) | (pk(b.w) << 16);
        *reinterpret_cast<uint4*>(rec + tok * 64 + part * 16) = o;
    }
    __syncthreads();
    for (int i = tid; i < REC_BYTES / 16; i += COMMIT_THREADS)
        reinterpret_cast<uint4*>(dst)[i] = reinterpret_cast<const uint4*>(rec)[i];
}

__global__ void __launch_bounds__(COMMIT_THREADS)
kv_commit_kernel(const half* __restrict__ Kf, const half* __restrict__ Vf, uint8_t* __restrict__ records,
                 const int32_t* __restrict__ pages, int max_blocks, int blk) {
    kv_commit_body(Kf, Vf, records, pages, max_blocks, blk);
}

}  // namespace llattn
