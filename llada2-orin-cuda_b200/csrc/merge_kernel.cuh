// Log-sum-exp merge of the partial results of one output tile (query block x kv head) and the output formats.
// Replaces the reference's attn::attn_combine (engine/attn.cu:314-358):
//   M = max_c m_c;  O = sum_c 2^(m_c - M) O_c / sum_c 2^(m_c - M) l_c        (m in log2 units)
// and writes any of: fp16 O, fp32 O, the natural-log sum of exponentials, and the int8 activation form the
// reference's dense projection reads (per (token, head): scale = max|v|/127 floored at 1e-30, q = clamp(rint(v/scale)),
// stored in the fragment order of engine/attn.cu:308-312, plus the integer row sum).
// A warp owns one query row; a lane owns dims 4*lane .. 4*lane+3 (a run of 4 stays contiguous in fragment order).
#pragma once
#include <cuda_fp16.h>
#include "common.cuh"

namespace llattn {

constexpr int MERGE_ROWS = 8;                 // rows per CTA
constexpr int MERGE_THREADS = 32 * MERGE_ROWS;

struct MergeOut {
    half* O16;
    float* O32;
    float* LSE;
    int8_t* q8;
    float* s8;
    int32_t* sum8;
};

__device__ __forceinline__ int frag_pos(int c) {
    const int base = c & ~127, r = c & 127;
    return base + 32 * ((r >> 2) & 3) + 8 * (r >> 5) + 4 * ((r >> 4) & 1) + (r & 3);
}

// r: query row of the tile (0..127), q_index: global query block, slots [slot0, slot0 + nslots).
__device__ __forceinline__ void merge_row(const float* __restrict__ Opart, const float* __restrict__ Mpart,
                                          const float* __restrict__ Lpart, int slot0, int nslots, int q_index, int kvh,
                                          int r, int lane, const MergeOut& o) {
    float M = -INFINITY;
    for (int c = 0; c < nslots; ++c) M = fmaxf(M, Mpart[size_t(slot0 + c) * QR + r]);
    float4 num = make_float4(0.f, 0.f, 0.f, 0.f);
    float den = 0.f;
    for (int c = 0; c < nslots; ++c) {
        const size_t i = size_t(slot0 + c) * QR + r;
        const float w = exp2f(Mpart[i] - M);
        const float4 v = *reinterpret_cast<const float4*>(Opart + i * D + 4 * lane);
        num.x += w * v.x; num.y += w * v.y; num.z += w * v.z; num.w += w * v.w;
        den += w * Lpart[i];
    }
    const float inv = 1.f / den;
    const float val[4] = {num.x * inv, num.y * inv, num.z * inv, num.w * inv};
    const int head = 4 * kvh + (r & 3);
    const size_t row = size_t(q_index) * BLK + (r >> 2);
    if (o.O32) *reinterpret_cast<float4*>(o.O32 + (row * NQH + head) * D + 4 * lane) = make_float4(val[0], val[1], val[2], val[3]);
    if (o.O16) {
        half2* d = reinterpret_cast<half2*>(o.O16 + (row * NQH + head) * D + 4 * lane);
        d[0] = __floats2half2_rn(val[0], val[1]);
        d[1] = __floats2half2_rn(val[2], val[3]);
    }
    if (o.LSE && lane == 0) o.LSE[row * NQH + head] = 0.6931471805599453f * (M + log2f(den));
    if (o.q8) {
        float m = fmaxf(fmaxf(fabsf(val[0]), fabsf(val[1])), fmaxf(fabsf(val[2]), fabsf(val[3])));
#pragma unroll
        for (int s = 16; s; s >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, s));
        const float sc = fmaxf(__fdiv_rn(m, 127.f), 1e-30f);
        int sm = 0;
        char4 qv;
        int8_t* qq = reinterpret_cast<int8_t*>(&qv);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            qq[k] = int8_t(max(-127, min(127, __float2int_rn(__fdiv_rn(val[k], sc)))));
            sm += qq[k];
        }
        *reinterpret_cast<char4*>(o.q8 + row * 2048 + frag_pos(head * D + 4 * lane)) = qv;
#pragma unroll
        for (int s = 16; s; s >>= 1) sm += __shfl_xor_sync(0xffffffffu, sm, s);
        if (lane == 0) { o.s8[row * NQH + head] = sc; o.sum8[row * NQH + head] = sm; }
    }
}

// Planned path: grid (output tiles, 128 / MERGE_ROWS).
__global__ void __launch_bounds__(MERGE_THREADS)
merge_kernel(const MergeDesc* __restrict__ md, const float* __restrict__ Opart, const float* __restrict__ Mpart,
             const float* __restrict__ Lpart, MergeOut o) {
    const MergeDesc d = md[blockIdx.x];
    const int r = blockIdx.y * MERGE_ROWS + (threadIdx.x >> 5);
    merge_row(Opart, Mpart, Lpart, d.slot_begin, d.nslots, d.q_index, d.kvh, r, threadIdx.x & 31, o);
}

// Reference-shaped path: grid (4 kv heads, 128 / MERGE_ROWS, nb), slots laid out [jb][kvh][nchunks] as the
// reference's partial buffers, the live chunk count of block jb given by chunks_for(nblocks + jb, bpc).
__global__ void __launch_bounds__(MERGE_THREADS)
combine_ref_kernel(const float* __restrict__ Opart, const float* __restrict__ Mpart, const float* __restrict__ Lpart,
                   int nchunks, int nblocks, int bpc, MergeOut o) {
    const int kvh = blockIdx.x, jb = blockIdx.z;
    const int r = blockIdx.y * MERGE_ROWS + (threadIdx.x >> 5);
    const int nbl = nblocks + jb;
    const int nch = nbl <= 0 ? 1 : (nbl + bpc - 1) / bpc;
    merge_row(Opart, Mpart, Lpart, (jb * NKV + kvh) * nchunks, nch, jb, kvh, r, threadIdx.x & 31, o);
}

}  // namespace llattn
