// Block-commit quantiser: a finished block's fp16 K/V -> one 4736-byte "4c/4" record per kv head.
// Replaces the reference's attn::kv_commit (engine/attn.cu:369-418) and must produce the same bytes:
//   K: per channel over the block's 32 tokens, V: per token over the 128 dims;
//   scale = half(max((max - min) / 15, 6.2e-5f)), min = half(min), code = clamp(rint((v - min) / scale), 0, 15),
//   all in IEEE fp32 with round-to-nearest-even; two codes per byte, even channel in the low nibble.
// One CTA per (kv head, block). The block's K and V slices sit in shared memory as fp16 tiles - loaded with 16-byte
// loads by kv_commit_kernel, or left there by the producer kernel that has just computed them (qkv_prepare.cuh) -, the
// record is assembled in shared memory and leaves as 16-byte stores.
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

constexpr int TILE_LD = D + 8;           // halves per tile row: rows 272 B apart, 16-byte aligned, no bank conflicts by column

// Shared memory of one (block, kv head) commit: the fp16 K and V slices, one K code per byte, the assembled record.
struct CommitSmem {
    __align__(16) half Ks[BLK][TILE_LD];
    __align__(16) half Vs[BLK][TILE_LD];
    __align__(16) uint8_t kq[BLK][D];
    __align__(16) uint8_t rec[REC_BYTES];
};

// The quantiser proper, from tiles already in shared memory (filled by 16-byte loads of fp16 K/V, or by the producer
// kernel that has just computed them) to the record at `dst`. Any multiple of 32 threads up to 128 per 32 K channels:
// called by CTAs of 128 or 256 threads; the tiles must be complete (a __syncthreads before the call).
__device__ __forceinline__ void commit_tiles(CommitSmem& sm, uint8_t* __restrict__ dst, int tid, int nthreads) {
    const int lane = tid & 31, warp = tid >> 5, nwarps = nthreads >> 5;
    // ---- V: a warp takes tokens warp, warp + nwarps, ...; a lane owns dims 4*lane .. 4*lane+3
    for (int tok = warp; tok < BLK; tok += nwarps) {
        const uint2 raw = *reinterpret_cast<const uint2*>(&sm.Vs[tok][lane * 4]);
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
        *reinterpret_cast<uint16_t*>(sm.rec + VOFF + tok * 64 + lane * 2) = uint16_t(packed);
        if (lane == 0) {
            reinterpret_cast<half*>(sm.rec + VOFF_META)[tok] = sh;
            reinterpret_cast<half*>(sm.rec + VOFF_META)[BLK + tok] = mh;
        }
    }
    // ---- K: a thread owns a channel
    for (int c = tid; c < D; c += nthreads) {
        float mn = INFINITY, mx = -INFINITY;
#pragma unroll
        for (int tk = 0; tk < BLK; ++tk) {
            const float v = __half2float(sm.Ks[tk][c]);
            mn = fminf(mn, v); mx = fmaxf(mx, v);
        }
        half sh, mh;
        commit_meta(mn, mx, sh, mh);
        const float s = __half2float(sh), m0 = __half2float(mh);
#pragma unroll
        for (int tk = 0; tk < BLK; ++tk) sm.kq[tk][c] = uint8_t(commit_code(__half2float(sm.Ks[tk][c]), m0, s));
        reinterpret_cast<half*>(sm.rec + KOFF_META)[c] = sh;
        reinterpret_cast<half*>(sm.rec + KOFF_META)[D + c] = mh;
    }
    __syncthreads();
    // ---- pack K codes: 4 threads per token, 32 channels = 16 output bytes each
    for (int i = tid; i < BLK * 4; i += nthreads) {
        const int tok = i >> 2, part = i & 3;
        const uint4 a = *reinterpret_cast<const uint4*>(&sm.kq[tok][part * 32]);
        const uint4 b = *reinterpret_cast<const uint4*>(&sm.kq[tok][part * 32 + 16]);
        auto pk = [](uint32_t x) -> uint32_t {                // 4 codes (one per byte) -> 2 packed bytes
            return (x & 0xfu) | ((x >> 4) & 0xf0u) | ((x >> 8) & 0xf00u) | ((x >> 12) & 0xf000u);
        };
        uint4 o;
        o.x = pk(a.x) | (pk(a.y) << 16); o.y = pk(a.z) | (pk(a.w) << 16);
        o.z = pk(b.x) | (pk(b.y) << 16); o.w = pk(b.z) | (pk(b.w) << 16);
        *reinterpret_cast<uint4*>(sm.rec + tok * 64 + part * 16) = o;
    }
    __syncthreads();
    for (int i = tid; i < REC_BYTES / 16; i += nthreads)
        reinterpret_cast<uint4*>(dst)[i] = reinterpret_cast<const uint4*>(sm.rec)[i];
}

// Kf, Vf: [nb][32 tok][4 heads][128] fp16. Record of (input block j, head h):
//   pages == nullptr: records + (h * max_blocks + blk + j) * 4736      (the reference's contiguous layer cache)
//   pages != nullptr: records + pages[j * 4 + h] * 4736                (record pool)
__device__ __forceinline__ void kv_commit_body(const half* __restrict__ Kf, const half* __restrict__ Vf,
                                               uint8_t* __restrict__ records, const int32_t* __restrict__ pages,
                                               int max_blocks, int blk) {
    __shared__ CommitSmem sm;
    const int h = blockIdx.x, j = blockIdx.y, tid = threadIdx.x;
    const size_t in0 = size_t(j) * BLK * NKV * D + size_t(h) * D;
    const size_t ridx = pages ? size_t(pages[j * NKV + h]) : size_t(h) * max_blocks + blk + j;
    // ---- both slices into shared memory (32 tokens x 256 B each, 16-byte loads)
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int idx = tid + COMMIT_THREADS * i, tok = idx >> 4, ch = idx & 15;
        *reinterpret_cast<uint4*>(&sm.Ks[tok][ch * 8]) = *reinterpret_cast<const uint4*>(Kf + in0 + size_t(tok) * NKV * D + ch * 8);
        *reinterpret_cast<uint4*>(&sm.Vs[tok][ch * 8]) = *reinterpret_cast<const uint4*>(Vf + in0 + size_t(tok) * NKV * D + ch * 8);
    }
    __syncthreads();
    commit_tiles(sm, records + ridx * REC_BYTES, tid, COMMIT_THREADS);
}

__global__ void __launch_bounds__(COMMIT_THREADS)
kv_commit_kernel(const half* __restrict__ Kf, const half* __restrict__ Vf, uint8_t* __restrict__ records,
                 const int32_t* __restrict__ pages, int max_blocks, int blk) {
    kv_commit_body(Kf, Vf, records, pages, max_blocks, blk);
}

}  // namespace llattn
