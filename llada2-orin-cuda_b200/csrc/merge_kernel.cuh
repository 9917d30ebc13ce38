// Folding the partial results of one output tile (query block x kv head) together and writing the output formats.
// Stands in for the reference's attn::attn_combine (engine/attn.cu:314-358):
//   M = max_c m_c;  O = sum_c 2^(m_c - M) O_c / sum_c 2^(m_c - M) l_c        (m in log2 units)
// Outputs, any of: fp16 O, fp32 O, the natural-log sum of exponentials, and the int8 activation form the reference's
// dense projection reads (per (token, head): scale = max|v| / 127 floored at 1e-30, q = clamp(rint(v / scale), +-127),
// stored in the fragment order of engine/attn.cu:308-312, plus the integer row sum).
//
// One THREAD owns one query row (all 128 dims): that is how the attention kernel holds its accumulator (one tensor-memory
// lane per row), so the same code finishes a row whether its values come from tensor memory (the attention kernel's
// epilogue: a tile made of a single run, or the run that arrives last at a tile) or from the partial slots in global
// memory (the reference-shaped operator pair, combine_ref_kernel below). A row is handled 32 dims at a time; the slots
// of a tile are always added in slot order, so the result does not depend on which run finishes last.
#pragma once
#include <cuda_fp16.h>
#include "common.cuh"

namespace llattn {

constexpr int MERGE_ROWS = 128;               // rows per CTA of combine_ref_kernel: one thread each
constexpr int MERGE_THREADS = MERGE_ROWS;

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

// Reference maximum and weighted row sum of a row over the slots [slot0, slot0 + nslots).
__device__ __forceinline__ void row_scale(const float* __restrict__ Mpart, const float* __restrict__ Lpart, int slot0, int nslots,
                                          int row, float& M, float& den) {
    M = -INFINITY;
    for (int s = 0; s < nslots; ++s) M = fmaxf(M, Mpart[size_t(slot0 + s) * QR + row]);
    den = 0.f;
    for (int s = 0; s < nslots; ++s) {
        const size_t i = size_t(slot0 + s) * QR + row;
        den += exp2f(Mpart[i] - M) * Lpart[i];
    }
}

// Dims [32 c, 32 c + 32) of the row's weighted, un-normalised sum over the slots, in dim order.
__device__ __forceinline__ void row_gather(const float* __restrict__ Opart, const float* __restrict__ Mpart, int slot0, int nslots,
                                           int row, float M, int c, float (&acc)[32]) {
#pragma unroll
    for (int j = 0; j < 32; ++j) acc[j] = 0.f;
    for (int s = 0; s < nslots; ++s) {
        const size_t i = size_t(slot0 + s) * QR + row;
        const float w = exp2f(Mpart[i] - M);
        const float4* src = reinterpret_cast<const float4*>(Opart + i * D + 32 * c);
#pragma unroll
        for (int g = 0; g < 8; ++g) {
            const float4 v = src[g];
            acc[4 * g] += w * v.x; acc[4 * g + 1] += w * v.y; acc[4 * g + 2] += w * v.z; acc[4 * g + 3] += w * v.w;
        }
    }
}

// Where a finished row goes: global token row, query head, and what is known before its values are walked.
struct RowOut {
    size_t row;        // q_index * 32 + token
    int head;          // 4 * kvh + (tile row % 4)
    float qscale;      // int8 form: max|v| / 127 floored, known after a first walk over the values
    int qsum;          // int8 form: running sum of the codes
};

// 32 normalised values of a row (dims [32 c, 32 c + 32), dim order) to every requested output.
__device__ __forceinline__ void row_store(const MergeOut& o, RowOut& ro, int c, const float (&v)[32]) {
    const size_t base = (ro.row * NQH + ro.head) * D + 32 * c;
    if (o.O32) {
#pragma unroll
        for (int g = 0; g < 8; ++g)
            *reinterpret_cast<float4*>(o.O32 + base + 4 * g) = make_float4(v[4 * g], v[4 * g + 1], v[4 * g + 2], v[4 * g + 3]);
    }
    if (o.O16) {
#pragma unroll
        for (int g = 0; g < 4; ++g) {
            const half2 a = __floats2half2_rn(v[8 * g], v[8 * g + 1]), b = __floats2half2_rn(v[8 * g + 2], v[8 * g + 3]);
            const half2 cc = __floats2half2_rn(v[8 * g + 4], v[8 * g + 5]), d = __floats2half2_rn(v[8 * g + 6], v[8 * g + 7]);
            uint4 pk;
            pk.x = *reinterpret_cast<const uint32_t*>(&a); pk.y = *reinterpret_cast<const uint32_t*>(&b);
            pk.z = *reinterpret_cast<const uint32_t*>(&cc); pk.w = *reinterpret_cast<const uint32_t*>(&d);
            *reinterpret_cast<uint4*>(o.O16 + base + 8 * g) = pk;
        }
    }
    if (o.q8) {
#pragma unroll
        for (int g = 0; g < 8; ++g) {      // a run of 4 dims stays contiguous in fragment order
            char4 qv;
            int8_t* qq = reinterpret_cast<int8_t*>(&qv);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                qq[k] = int8_t(max(-127, min(127, __float2int_rn(__fdiv_rn(v[4 * g + k], ro.qscale)))));
                ro.qsum += qq[k];
            }
            *reinterpret_cast<char4*>(o.q8 + ro.row * 2048 + frag_pos(ro.head * D + 32 * c + 4 * g)) = qv;
        }
    }
}
__device__ __forceinline__ float absmax32(const float (&v)[32]) {
    float m = 0.f;
#pragma unroll
    for (int j = 0; j < 32; ++j) m = fmaxf(m, fabsf(v[j]));
    return m;
}
// Per-row scalars once all values are out: the log-sum-exp and the int8 form's scale and code sum.
__device__ __forceinline__ void row_finish(const MergeOut& o, const RowOut& ro, float M, float den) {
    if (o.LSE) o.LSE[ro.row * NQH + ro.head] = 0.6931471805599453f * (M + log2f(den));
    if (o.q8) { o.s8[ro.row * NQH + ro.head] = ro.qscale; o.sum8[ro.row * NQH + ro.head] = ro.qsum; }
}

// Reference-shaped path: grid (4 kv heads, nb), 128 threads = the tile's rows; slots laid out [jb][kvh][nchunks] as
// the reference's partial buffers, the live chunk count of block jb given by chunks_for(nblocks + jb, bpc).
__device__ __forceinline__ void combine_ref_body(const float* __restrict__ Opart, const float* __restrict__ Mpart,
                                                 const float* __restrict__ Lpart, int nchunks, int nblocks, int bpc, int kvh, int jb,
                                                 int r, const MergeOut& o) {
    const int nbl = nblocks + jb;
    const int nch = nbl <= 0 ? 1 : (nbl + bpc - 1) / bpc;
    const int slot0 = (jb * NKV + kvh) * nchunks;
    float M, den;
    row_scale(Mpart, Lpart, slot0, nch, r, M, den);
    const float inv = 1.f / den;
    RowOut ro{size_t(jb) * BLK + (r >> 2), 4 * kvh + (r & 3), 0.f, 0};
    float v[32];
    if (o.q8) {
        float m = 0.f;
        for (int c = 0; c < 4; ++c) {
            row_gather(Opart, Mpart, slot0, nch, r, M, c, v);
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] *= inv;
            m = fmaxf(m, absmax32(v));
        }
        ro.qscale = fmaxf(__fdiv_rn(m, 127.f), 1e-30f);
    }
    for (int c = 0; c < 4; ++c) {
        row_gather(Opart, Mpart, slot0, nch, r, M, c, v);
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] *= inv;
        row_store(o, ro, c, v);
    }
    row_finish(o, ro, M, den);
}

__global__ void __launch_bounds__(MERGE_THREADS)
combine_ref_kernel(const float* __restrict__ Opart, const float* __restrict__ Mpart, const float* __restrict__ Lpart,
                   int nchunks, int nblocks, int bpc, MergeOut o) {
    combine_ref_body(Opart, Mpart, Lpart, nchunks, nblocks, bpc, blockIdx.x, blockIdx.y, threadIdx.x, o);
}

}  // namespace llattn
