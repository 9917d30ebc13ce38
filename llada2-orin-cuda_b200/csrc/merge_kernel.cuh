// Folding the partial results of one output tile (query block x kv head) together and writing the output formats.
// Stands in for the reference's attn::attn_combine (engine/attn.cu:314-358):
//   M = max_c m_c;  O = sum_c 2^(m_c - M) O_c / sum_c 2^(m_c - M) l_c        (m in log2 units)
// Outputs, any of: fp16 O, fp32 O, the natural-log sum of exponentials, and the int8 activation form the reference's
// dense projection reads (per (token, head): scale = max|v| / 127 floored at 1e-30, q = clamp(rint(v / scale), +-127),
// stored in the fragment order of engine/attn.cu:308-312, plus the integer row sum).
//
// Two forms. In the attention kernel's epilogue one THREAD owns one query row (that is how the kernel holds its
// accumulator: one tensor-memory lane per row) and writes a row 32 dims at a time straight from tensor memory
// (row_store, row_finish): a tile that a single run covers needs no folding. Everywhere partial slots have to be folded -
// the attention kernel's split tiles, the reference-shaped operator pair, the allocation-free entry point, the source
// shim - a WARP owns a row (fold_row_warp and friends, below). The slots of a tile are always added in slot order, so
// the result does not depend on which run finishes last.
#pragma once
#include <cuda_fp16.h>
#include "common.cuh"

namespace llattn {

constexpr int MERGE_ROWS = 8;                 // rows per CTA of combine_ref_kernel: one warp each
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

// ------------------------------------------------------------------------------------------------------------------
// Shared folding of a split tile (the attention kernel's own path). Every run of a tile that was cut into several runs
// stores its partial result and counts itself in; when a CTA has no runs left it comes back to each of its split tiles,
// waits until all of that tile's runs are counted, and finishes an equal share of the tile's rows: run k of n takes
// rows k, k + n, k + 2n, ... So a tile cut into n runs is folded by n SMs at once, each reading as much as it wrote.
// Here a WARP owns a row: lane l holds dims 4l .. 4l+3, a slot's row is one coalesced 512-byte read, and the loads of up
// to FOLD_BATCH slots are in flight together. The sums run in slot order, like everywhere else.
constexpr int FOLD_BATCH = 12;

__device__ __forceinline__ int load_acquire(const int* p) {
    int v;
    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// Warp-uniform bounded wait until *counter reaches `target`. False if the CTA gave up elsewhere or the limit ran out.
__device__ __forceinline__ bool wait_count(const int* counter, int target, volatile int* abort_flag, unsigned long long limit_ns) {
    unsigned long long t0 = 0;
    for (unsigned it = 0;; ++it) {
        if (load_acquire(counter) >= target) return true;
        if (*abort_flag) return false;
        if ((it & 15u) == 15u) {
            unsigned long long t;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
            if (t0 == 0) t0 = t;
            else if (t - t0 > limit_ns) return false;
        }
        __nanosleep(100);
    }
}

// A folded row (reference exponent M, weighted row sum den, un-normalised dims 4 lane .. 4 lane + 3) to every requested
// output, by the warp that owns the row.
__device__ __forceinline__ void emit_row_warp(float M, float den, const float4& acc, const MergeDesc& md, int r, int lane,
                                              const MergeOut& o) {
    const float inv = 1.f / den;
    const float val[4] = {acc.x * inv, acc.y * inv, acc.z * inv, acc.w * inv};
    const size_t row = size_t(md.q_index) * BLK + (r >> 2);
    const int head = 4 * md.kvh + (r & 3);
    const size_t at = (row * NQH + head) * D + 4 * lane;
    if (o.O32) *reinterpret_cast<float4*>(o.O32 + at) = make_float4(val[0], val[1], val[2], val[3]);
    if (o.O16) {
        const half2 a = __floats2half2_rn(val[0], val[1]), b = __floats2half2_rn(val[2], val[3]);
        *reinterpret_cast<uint2*>(o.O16 + at) = make_uint2(*reinterpret_cast<const uint32_t*>(&a), *reinterpret_cast<const uint32_t*>(&b));
    }
    if (o.LSE && lane == 0) o.LSE[row * NQH + head] = 0.6931471805599453f * (M + log2f(den));
    if (o.q8) {
        float m = fmaxf(fmaxf(fabsf(val[0]), fabsf(val[1])), fmaxf(fabsf(val[2]), fabsf(val[3])));
#pragma unroll
        for (int d = 16; d; d >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, d));
        const float qscale = fmaxf(__fdiv_rn(m, 127.f), 1e-30f);
        int code[4], total = 0;
#pragma unroll
        for (int k = 0; k < 4; ++k) { code[k] = max(-127, min(127, __float2int_rn(__fdiv_rn(val[k], qscale)))); total += code[k]; }
        const uint32_t packed = uint32_t(code[0] & 0xff) | uint32_t(code[1] & 0xff) << 8 | uint32_t(code[2] & 0xff) << 16 | uint32_t(code[3] & 0xff) << 24;
        *reinterpret_cast<uint32_t*>(o.q8 + row * 2048 + frag_pos(head * D + 4 * lane)) = packed;
#pragma unroll
        for (int d = 16; d; d >>= 1) total += __shfl_xor_sync(0xffffffffu, total, d);
        if (lane == 0) { o.s8[row * NQH + head] = qscale; o.sum8[row * NQH + head] = total; }
    }
}

// One row of a split tile, by one warp: fold the slots, normalise, write every requested output.
constexpr int FOLD_MAX_SLOTS = 160;           // slots of one tile: at most one per CTA of the launch (148 SMs)
__device__ __forceinline__ void fold_row_warp(const float* Opart, const float* Mpart, const float* Lpart, const MergeDesc& md,
                                              int r, int lane, const MergeOut& o) {
    const int n = md.nslots;
    const size_t i0 = size_t(md.slot_begin) * QR + r;              // the row in the tile's first slot; + QR per slot
    // reference exponents and row sums of all slots at once: lane l holds slots l, l + 32, ...
    float mm[FOLD_MAX_SLOTS / 32], ll[FOLD_MAX_SLOTS / 32];
    float M = -INFINITY;
#pragma unroll
    for (int c = 0; c < FOLD_MAX_SLOTS / 32; ++c) {
        const int s = 32 * c + lane;
        mm[c] = s < n ? __ldcg(Mpart + i0 + size_t(s) * QR) : -INFINITY;
        ll[c] = s < n ? __ldcg(Lpart + i0 + size_t(s) * QR) : 0.f;
        M = fmaxf(M, mm[c]);
    }
#pragma unroll
    for (int d = 16; d; d >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, d));
#pragma unroll
    for (int c = 0; c < FOLD_MAX_SLOTS / 32; ++c) mm[c] = exp2f(mm[c] - M);      // now the slots' weights
    float den = 0.f;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int c = 0; c < FOLD_MAX_SLOTS / 32; ++c) {
        if (32 * c >= n) break;
        const int nc = min(32, n - 32 * c);
#pragma unroll 1
        for (int s0 = 0; s0 < nc; s0 += FOLD_BATCH) {
            float4 v[FOLD_BATCH];
#pragma unroll
            for (int k = 0; k < FOLD_BATCH; ++k)       // past the end: the chunk's last slot again, not used below
                v[k] = __ldcg(reinterpret_cast<const float4*>(Opart + (i0 + size_t(32 * c + min(s0 + k, nc - 1)) * QR) * D) + lane);
#pragma unroll
            for (int k = 0; k < FOLD_BATCH; ++k) {
                const float f = __shfl_sync(0xffffffffu, mm[c], (s0 + k) & 31), l = __shfl_sync(0xffffffffu, ll[c], (s0 + k) & 31);
                if (s0 + k < nc) {
                    den += f * l;
                    acc.x += f * v[k].x; acc.y += f * v[k].y; acc.z += f * v[k].z; acc.w += f * v[k].w;
                }
            }
        }
    }
    emit_row_warp(M, den, acc, md, r, lane, o);
}

// A few rows at once for tiles cut into NS <= 4 runs (what a large batch produces: a tile straddling two CTAs): the
// loads of R rows x NS slots are all issued before the first sum, so a warp's share of a tile takes one round trip to
// the L2 instead of one per row. rows[q] < 0: no row.
template <int R, int NS>
__device__ __forceinline__ void fold_rows_few(const float* Opart, const float* Mpart, const float* Lpart, const MergeDesc& md,
                                              const int (&rows)[R], int lane, const MergeOut& o) {
    const int n = md.nslots;
    float m[R][NS], l[R][NS];
    float4 v[R][NS];
#pragma unroll
    for (int q = 0; q < R; ++q)
#pragma unroll
        for (int s = 0; s < NS; ++s) {
            const size_t i = (size_t(md.slot_begin) + min(s, n - 1)) * QR + max(rows[q], 0);
            m[q][s] = __ldcg(Mpart + i);
            l[q][s] = __ldcg(Lpart + i);
            v[q][s] = __ldcg(reinterpret_cast<const float4*>(Opart + i * D) + lane);
        }
#pragma unroll
    for (int q = 0; q < R; ++q) {
        if (rows[q] < 0) continue;
        float M = m[q][0];
#pragma unroll
        for (int s = 1; s < NS; ++s) if (s < n) M = fmaxf(M, m[q][s]);
        float den = 0.f;
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int s = 0; s < NS; ++s)
            if (s < n) {
                const float f = exp2f(m[q][s] - M);
                den += f * l[q][s];
                acc.x += f * v[q][s].x; acc.y += f * v[q][s].y; acc.z += f * v[q][s].z; acc.w += f * v[q][s].w;
            }
        emit_row_warp(M, den, acc, md, rows[q], lane, o);
    }
}

// Reference-shaped path (the operator pair on caller-owned partial buffers, and the allocation-free entry point): slots
// laid out [jb][kvh][nchunks] as the reference's partial buffers, the live chunk count of block jb given by
// chunks_for(nblocks + jb, bpc). Grid (4 kv heads, 128 / MERGE_ROWS, nb), a warp per query row.
__global__ void __launch_bounds__(MERGE_THREADS)
combine_ref_kernel(const float* __restrict__ Opart, const float* __restrict__ Mpart, const float* __restrict__ Lpart,
                   int nchunks, int nblocks, int bpc, MergeOut o) {
    const int kvh = blockIdx.x, jb = blockIdx.z, nbl = nblocks + jb;
    const MergeDesc md{jb, kvh, (jb * NKV + kvh) * nchunks, nbl <= 0 ? 1 : (nbl + bpc - 1) / bpc};
    fold_row_warp(Opart, Mpart, Lpart, md, int(blockIdx.y) * MERGE_ROWS + int(threadIdx.x >> 5), int(threadIdx.x & 31), o);
}

}  // namespace llattn
