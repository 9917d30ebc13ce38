// Block attention over int4 "4c/4" KV records on tcgen05 tensor cores.
//
// One CTA per SM walks a list of work items. An item is a run of KV units of one (sequence, query block, kv head):
// committed records (4736 packed bytes = 32 keys each) and, on the run that ends the context, the query block's own
// fp16 K/V. The 128 query rows of the kv head (32 tokens x 4 GQA heads) are the M dimension of every MMA.
// Per tile of up to 4 units (128 keys):
//   producer warps: cp.async.bulk of whole records global -> shared ring, completion on an mbarrier (two warps take
//                   alternate records: one service warp per scheduler keeps the schedulers' loads alike)
//   dequant warps : nibbles -> fp16 (magic-number unpack, one fp16 FMA per pair as the reference's __hfma2), written
//                   straight into the 128-byte-swizzle UMMA operand layout; fresh fp16 K/V are copied into the same layout
//   MMA warps     : S = Q K^T  (tcgen05.mma kind::f16, A = Q in TMEM, B = K K-major in shared memory, fp32 S in TMEM)
//                   O += P V   (A = P read from TMEM as packed fp16, B = V MN-major in shared memory, fp32 O in TMEM);
//                   V carries one extra column of ones, so the same MMA also accumulates the softmax row sum from
//                   exactly the fp16 P the numerator uses (numerator and denominator then share their rounding)
//   softmax warps : four warps, one thread per query row (TMEM lane), all keys of the row: no exchange between warps.
//                   One pass per tile: p = 2^(s*scale*log2e - mref) for 16 scores at a time while the next 16 arrive
//                   from tensor memory, the chunk maximum taken on the way; P goes back over S in TMEM as fp16 pairs
//                   (the 32 keys of chunk g at columns 32 g .. 32 g + 15, the first half of the S columns they were
//                   computed from). The reference exponent mref is the exact row maximum of the run's first tile and
//                   moves only when a later score exceeds it by more than 8 in log2 units (engine/attn.cu:237-255
//                   rescales lazily in the same way); that rare path rescales O in tensor memory, out of line
// A run that is a tile's only one normalises and writes the outputs in its epilogue. Otherwise its un-normalised O (fp32),
// reference maximum (log2 units) and row sum go to a partial slot in the format of the reference's Opart/Mpart/Lpart
// (engine/attn.cu:291-305) and it counts itself in at the tile's arrival counter. When a CTA has no runs left it returns
// to its split tiles: it waits (bounded) until every run of the tile is counted, then folds its share of the tile's
// rows (run k of n takes rows k, k + n, ...; all sixteen warps, a warp per row; merge_kernel.cuh) and writes their
// outputs, so a tile cut into n runs is folded by n SMs at once. A CTA only ever waits after all of its own runs are
// out, so the waits cannot form a cycle; they need every CTA of the launch to be on an SM, which a grid of at most one
// CTA per SM launched cooperatively guarantees. With the reference-shaped operator pair the caller's attn_combine
// launch folds instead.
//
// Operands. Q (the A operand of S = Q K^T) lives in tensor memory for the whole item: row i in lane i, 64 columns of
// fp16 pairs. K and V tiles live in shared memory in the 128-byte-swizzle layout: a tile is made of blocks of
// 128 keys x 128 bytes (64 channels of one key per row; K has two blocks, V a third one whose first column is all
// ones), and the 16-byte chunk c of key k sits at chunk position c ^ (k % 8). K is read K-major (S), V MN-major (PV).
// The layout is chosen to make every access of the dequantisation conflict-free: a warp loads the packed
// codes of two whole keys (128 contiguous bytes) and each quarter warp stores the eight 16-byte chunks of one key's
// row. Within each group of 8 channels the order is (0,4,1,5,2,6,3,7): that is what the shift-free nibble unpack
// produces, Q and the fresh K are stored in the same order (a dot product does not care) and V's order is undone when
// O is written out.
//
// Every wait is bounded (ptx::mbar_wait); a wait that runs out sets a bit in the error word and every role leaves.
#pragma once
#include <cuda_fp16.h>
#include "common.cuh"
#include "ptx.cuh"
#include "merge_kernel.cuh"

namespace llattn {

// Timeline hooks for kernel tuning: compiled out unless LLATTN_TRACE is defined (the shipped library never defines it).
#ifdef LLATTN_TRACE
__device__ unsigned long long* g_trace_buf;      // [warps][LLATTN_TRACE_EVENTS] of (clock << 24 | tile << 8 | event)
constexpr int LLATTN_TRACE_EVENTS = 2048;
#ifndef LLATTN_TRACE_ONLY
#define LLATTN_TRACE_ONLY (ev)          // tuning: keep a single event (less disturbance)
#endif
#define LLATTN_TR(ev, tile)                                                                                    \
    do {                                                                                                       \
        if ((ev) == (LLATTN_TRACE_ONLY) && trace_ptr && trace_n < LLATTN_TRACE_EVENTS)                                                        \
            trace_ptr[trace_n++] =                                 \
                (static_cast<unsigned long long>(clock64()) << 24) | (static_cast<unsigned long long>((tile) & 0xffff) << 8) | (ev); \
    } while (0)
#else
#define LLATTN_TR(ev, tile) do {} while (0)
#endif
#ifndef LLATTN_SKIP
#define LLATTN_SKIP 0      // tuning builds only: bit 0 = no dequantisation, bit 1 = no exponentials (results are garbage)
#endif

constexpr int TILE_UNITS = 4;
constexpr int KBLOCK = 128 * 128;                  // 16384: 128 keys x 64 channels of fp16, one swizzled block
constexpr int TILE_BYTES = 2 * KBLOCK;             // K tile: channels 0-63, 64-127
constexpr int VTILE_BYTES = 3 * KBLOCK;            // V tile: dims 0-63, 64-127, then the block with the ones column
constexpr int UNIT_BYTES = 32 * 128;               // a unit's 32 keys inside a block
constexpr int PV_N = 144;                          // dims 0..127, column 128 = row sum, 129..143 unused
#ifndef LLATTN_NRAW
#define LLATTN_NRAW 8
#endif
constexpr int NRAW = LLATTN_NRAW;                  // records in flight (8 = two tiles' worth)
constexpr int RAW_STRIDE = 4864;                   // 4736 rounded up to a multiple of 128
constexpr int SM_K = 0;                            // two K tiles (every tile base is 1024-byte aligned)
constexpr int SM_V = SM_K + 2 * TILE_BYTES;        // two V tiles
constexpr int SM_RAW = SM_V + 2 * VTILE_BYTES;
constexpr int SM_BAR = SM_RAW + NRAW * RAW_STRIDE;
constexpr int SM_MISC = SM_BAR + 512;
constexpr int SM_FIRST = SM_MISC + 16;             // the CTA's first run descriptor (64 bytes), fetched during set-up
constexpr int ATTN_SMEM_BYTES = SM_FIRST + 64;
// warps 0-3 softmax (warp w: TMEM lanes 32 w .. 32 w + 31, one query row per thread), 4-11 dequant (four groups of two
// warps, group g takes unit g of every tile: a thread's scale / minimum words then serve eight passes over the record),
// then the service warps. Every scheduler carries one softmax warp, two dequantising warps and one service warp.
#ifndef LLATTN_DEQUANT_WARPS
#define LLATTN_DEQUANT_WARPS 8
#endif
#ifndef LLATTN_GROUP_WARPS
#define LLATTN_GROUP_WARPS 2
#endif
#ifndef LLATTN_SINGLE_ISSUER
#define LLATTN_SINGLE_ISSUER 0     // 1: one warp issues PV(t) and then S(t+2); the tensor pipe runs one thread's MMAs in order
#endif
#ifndef LLATTN_WARP_ARRIVE
#define LLATTN_WARP_ARRIVE 0       // 1: one arrival per softmax warp on the P barrier instead of one per thread
#endif
constexpr int SOFTMAX_WARPS = 4, DEQUANT_WARPS = LLATTN_DEQUANT_WARPS, GROUP_WARPS = LLATTN_GROUP_WARPS, DEQUANT_GROUPS = DEQUANT_WARPS / GROUP_WARPS;
constexpr int GROUP_THREADS = 32 * GROUP_WARPS, DQ_PASSES = 16 / GROUP_WARPS;      // a group converts one record: 32 keys, two per warp and pass
constexpr int WARP_SERVICE = SOFTMAX_WARPS + DEQUANT_WARPS;
// Service warps, one per scheduler (a warp runs on scheduler warp % 4 and the softmax warps cannot move): PV issue, S
// issue and two copy producers that take alternate records, so that no scheduler carries much more than the others.
constexpr int WARP_MMA_PV = WARP_SERVICE, WARP_MMA = WARP_SERVICE + 1, WARP_PRODUCER = WARP_SERVICE + 2, PRODUCERS = 2;
constexpr int ATTN_THREADS = 32 * (WARP_SERVICE + 2 + PRODUCERS);  // 512
constexpr int P_ARRIVALS = LLATTN_WARP_ARRIVE ? SOFTMAX_WARPS : 32 * SOFTMAX_WARPS;
constexpr int TMEM_COLS = 512;
constexpr int TM_S = 0, TM_O = 256, TM_L = TM_O + 128, TM_Q = 400;   // S at columns 0 and 128, O at 256..383, row sum at 384, Q at 400..463
// The reference exponent of a row moves when a score exceeds it by more than this many powers of two, the reference's own
// threshold (engine/attn.cu:237-255): p = 2^(x - mref), stored as fp16, then stays below 2^8, and a row that a late key
// dominates gets that key as its new reference (p = 1 for it, no rounding).
constexpr float RESCALE_SLACK = 8.f;

// barrier indices
enum { B_RAW_FULL = 0, B_RAW_EMPTY = B_RAW_FULL + NRAW, B_K_FULL = B_RAW_EMPTY + NRAW, B_V_FULL = B_K_FULL + 2,
       B_K_FREE = B_V_FULL + 2, B_PV_DONE = B_K_FREE + 2, B_S_FULL = B_PV_DONE + 2, B_P_FULL = B_S_FULL + 2,
       B_Q_FULL = B_P_FULL + 2, B_O_FREE, B_SPARE, B_COUNT = B_SPARE + 2 };
static_assert(B_COUNT * 8 <= 512, "barrier area");
static_assert(ATTN_SMEM_BYTES <= 232448, "shared memory budget");
static_assert((GROUP_WARPS == 2 || GROUP_WARPS == 4) && DEQUANT_WARPS % GROUP_WARPS == 0 && DEQUANT_GROUPS >= 1 && TILE_UNITS % DEQUANT_GROUPS == 0,
              "dequant warps: groups of two or four, 1, 2 or 4 groups");

struct KParams {
    const RunDesc* items;          // list mode: runs in plan order, each with its sequence; nullptr = reference-grid mode
    const int32_t* cta_first;      // [gridDim.x + 1]
    const half* Q;
    const half* Kf;
    const half* Vf;
    float* Opart;
    float* Mpart;
    float* Lpart;
    float sl2;                     // softmax scale * log2(e)
    int* err;
    // list mode with folding in the kernel (merge != nullptr)
    const MergeDesc* merge;        // per output tile (WorkItem::tile indexes it)
    int* tile_counters;            // [tiles][4]: [0] softmax warps whose rows of a run are out (4 per run), [1] warps that
                                   // have folded their share (16 per run); both back at 0 when the launch ends
    MergeOut out;
    size_t cache_offset;           // bytes added to every sequence's cache pointer: the layer this launch reads
    // reference-grid mode (items == nullptr): CTA i is (kvh = i % 4, chunk = (i / 4) % ref_nchunks, jb = i / (4 * ref_nchunks))
    SeqDesc ref_seq;
    int ref_bpc;
    int ref_nchunks;
};

__device__ __forceinline__ bool fetch_item(const KParams& p, int idx, WorkItem& w, SeqDesc& s, const RunDesc* first, int first_idx) {
    if (p.items) {
        const uint4* src = reinterpret_cast<const uint4*>(idx == first_idx ? first : p.items + idx);   // the first one is in shared memory
        RunDesc r;
        uint4* dst = reinterpret_cast<uint4*>(&r);
#pragma unroll
        for (int k = 0; k < 4; ++k) dst[k] = src[k];
        w = r.w;
        s = r.s;
        s.cache += p.cache_offset;
        return true;
    }
    const int kvh = idx & 3, chunk = (idx >> 2) % p.ref_nchunks, jb = (idx >> 2) / p.ref_nchunks;
    s = p.ref_seq;
    const int nbl = s.nblocks + jb;
    const int nch = nbl <= 0 ? 1 : (nbl + p.ref_bpc - 1) / p.ref_bpc;
    if (chunk >= nch) return false;
    const int b0 = chunk * p.ref_bpc;
    w.seq = 0; w.qblk = jb; w.kvh = kvh; w.rec_begin = b0;
    w.rec_count = nbl <= 0 ? 0 : min(p.ref_bpc, nbl - b0);
    w.fresh = chunk == nch - 1;
    w.slot = (jb * NKV + kvh) * p.ref_nchunks + chunk;
    w.tile = 0;
    return true;
}

// The same value in every lane, in a form the compiler can see is warp-uniform (a warp reduction): the MMA-issuing warps
// run warp-uniform code whose operands then stay in uniform registers instead of being moved there before every MMA.
__device__ __forceinline__ uint32_t uniform_u32(uint32_t x) { return __reduce_max_sync(0xffffffffu, x); }
__device__ __forceinline__ int uniform_i32(int x) { return __reduce_max_sync(0xffffffffu, x); }

// 8 nibbles of w -> 4 half2 holding channels (0,4) (1,5) (2,6) (3,7), each value the nibble exactly.
// Low nibbles of a 16-bit half land in the mantissa of 1024 (0x6400), nibbles at bits 4-7 in the mantissa of 64
// (0x5400, whose ulp is 1/16); subtracting the bias leaves the integer.
__device__ __forceinline__ void unpack8(uint32_t w, half2 (&h)[4]) {
    const uint32_t w8 = w >> 8;
    uint32_t x0, x1, x2, x3;
    asm("lop3.b32 %0, %1, %2, %3, 0xea;" : "=r"(x0) : "r"(w), "r"(0x000f000fu), "r"(0x64006400u));
    asm("lop3.b32 %0, %1, %2, %3, 0xea;" : "=r"(x1) : "r"(w), "r"(0x00f000f0u), "r"(0x54005400u));
    asm("lop3.b32 %0, %1, %2, %3, 0xea;" : "=r"(x2) : "r"(w8), "r"(0x000f000fu), "r"(0x64006400u));
    asm("lop3.b32 %0, %1, %2, %3, 0xea;" : "=r"(x3) : "r"(w8), "r"(0x00f000f0u), "r"(0x54005400u));
    const half2 b1024 = __half2half2(__ushort_as_half(0x6400)), b64 = __half2half2(__ushort_as_half(0x5400));
    h[0] = __hsub2(*reinterpret_cast<half2*>(&x0), b1024);
    h[1] = __hsub2(*reinterpret_cast<half2*>(&x1), b64);
    h[2] = __hsub2(*reinterpret_cast<half2*>(&x2), b1024);
    h[3] = __hsub2(*reinterpret_cast<half2*>(&x3), b64);
}

// 8 fp16 in channel order (uint4) -> the (0,4,1,5,2,6,3,7) order.
__device__ __forceinline__ uint4 permute8(uint4 v) {
    uint4 o;
    o.x = __byte_perm(v.x, v.z, 0x5410);
    o.y = __byte_perm(v.x, v.z, 0x7632);
    o.z = __byte_perm(v.y, v.w, 0x5410);
    o.w = __byte_perm(v.y, v.w, 0x7632);
    return o;
}

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Two fp32 multiply-adds in one instruction (sm_100 packed fp32): (a0, a1) * (b, b) + (c, c), each rounded like fmaf.
__device__ __forceinline__ void fma2(uint32_t a0, uint32_t a1, unsigned long long bb, unsigned long long cc, float& d0, float& d1) {
    unsigned long long a, d;
    asm("mov.b64 %0, {%1, %2};" : "=l"(a) : "r"(a0), "r"(a1));
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(bb), "l"(cc));
    asm("mov.b64 {%0, %1}, %2;" : "=f"(d0), "=f"(d1) : "l"(d));
}
__device__ __forceinline__ unsigned long long dup2(float x) {
    unsigned long long d;
    asm("mov.b64 %0, {%1, %1};" : "=l"(d) : "f"(x));
    return d;
}

__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

// Maximum of the 32 scores of a chunk (two chains of 3-input maxima).
__device__ __forceinline__ float rowmax32(const uint32_t (&r)[32]) {
    float a = max3(__uint_as_float(r[0]), __uint_as_float(r[1]), __uint_as_float(r[2]));
    float b = max3(__uint_as_float(r[16]), __uint_as_float(r[17]), __uint_as_float(r[18]));
#pragma unroll
    for (int j = 3; j < 15; j += 2) {
        a = max3(a, __uint_as_float(r[j]), __uint_as_float(r[j + 1]));
        b = max3(b, __uint_as_float(r[16 + j]), __uint_as_float(r[16 + j + 1]));
    }
    return max3(max3(a, b, __uint_as_float(r[15])), __uint_as_float(r[31]), __uint_as_float(r[31]));
}
// Score pairs J0 .. J1-1 of a chunk -> p = 2^(s * sl2 - mref) as packed fp16 (the multiply-add on two scores at a time).
template <int J0, int J1>
__device__ __forceinline__ void exp_pairs(const uint32_t (&r)[32], uint32_t (&pk)[16], unsigned long long sl2x2, unsigned long long nm2) {
#pragma unroll
    for (int j = J0; j < J1; ++j) {
        if (LLATTN_SKIP & 2) { pk[j] = r[2 * j] & 0x03ff03ffu; continue; }
        float x0, x1;
        fma2(r[2 * j], r[2 * j + 1], sl2x2, nm2, x0, x1);
        const half2 h = __floats2half2_rn(ex2(x0), ex2(x1));
        pk[j] = *reinterpret_cast<const uint32_t*>(&h);
    }
}

// Maximum of 16 scores.
__device__ __forceinline__ float rowmax16(const uint32_t (&r)[16]) {
    float a = max3(__uint_as_float(r[0]), __uint_as_float(r[1]), __uint_as_float(r[2]));
    float b = max3(__uint_as_float(r[8]), __uint_as_float(r[9]), __uint_as_float(r[10]));
#pragma unroll
    for (int j = 3; j < 7; j += 2) {
        a = max3(a, __uint_as_float(r[j]), __uint_as_float(r[j + 1]));
        b = max3(b, __uint_as_float(r[8 + j]), __uint_as_float(r[8 + j + 1]));
    }
    return max3(max3(a, b, __uint_as_float(r[7])), __uint_as_float(r[15]), __uint_as_float(r[15]));
}
#ifndef LLATTN_POLY_MOD
#define LLATTN_POLY_MOD 0      // n > 0: every n-th score pair takes its 2^x from the multiply-add pipes instead of the MUFU
#endif
// 2^x for two values on the multiply-add pipes: x is held above -125, split into round(x) and a fraction in [-0.5, 0.5]
// by the add-a-large-constant trick, 2^fraction comes from a degree-4 polynomial (relative error 2e-6, far below the
// fp16 rounding that follows) and round(x) is added into the exponent field.
__device__ __forceinline__ void exp2_pair_poly(float x0, float x1, float& e0, float& e1) {
    x0 = fmaxf(x0, -125.f); x1 = fmaxf(x1, -125.f);
    unsigned long long x, t, n, f, q;
    asm("mov.b64 %0, {%1, %2};" : "=l"(x) : "f"(x0), "f"(x1));
    asm("{\n\t.reg .b64 m;\n\tmov.b64 m, 0x4b4000004b400000;\n\tadd.rn.f32x2 %0, %1, m;\n\t}" : "=l"(t) : "l"(x));        // 1.5 * 2^23 + round(x)
    asm("{\n\t.reg .b64 m;\n\tmov.b64 m, 0xcb400000cb400000;\n\tadd.rn.f32x2 %0, %1, m;\n\t}" : "=l"(n) : "l"(t));        // round(x)
    asm("{\n\t.reg .b64 m;\n\tmov.b64 m, 0xbf800000bf800000;\n\tfma.rn.f32x2 %0, %1, m, %2;\n\t}" : "=l"(f) : "l"(n), "l"(x));   // x - round(x)
    asm("{\n\t.reg .b64 a, b;\n\tmov.b64 a, 0x3c1803f73c1803f7;\n\tmov.b64 b, 0x3d64d2b93d64d2b9;\n\tfma.rn.f32x2 %0, %1, a, b;\n\t}" : "=l"(q) : "l"(f));   // 0.009278289 f + 0.055865023
    asm("{\n\t.reg .b64 c;\n\tmov.b64 c, 0x3e76138d3e76138d;\n\tfma.rn.f32x2 %0, %0, %1, c;\n\t}" : "+l"(q) : "l"(f));                              // 0.24030896
    asm("{\n\t.reg .b64 c;\n\tmov.b64 c, 0x3f3170f03f3170f0;\n\tfma.rn.f32x2 %0, %0, %1, c;\n\t}" : "+l"(q) : "l"(f));                              // 0.69312954
    asm("{\n\t.reg .b64 c;\n\tmov.b64 c, 0x3f7fffdc3f7fffdc;\n\tfma.rn.f32x2 %0, %0, %1, c;\n\t}" : "+l"(q) : "l"(f));                              // 0.99999785
    uint32_t q0, q1, t0, t1;
    asm("mov.b64 {%0, %1}, %2;" : "=r"(q0), "=r"(q1) : "l"(q));
    asm("mov.b64 {%0, %1}, %2;" : "=r"(t0), "=r"(t1) : "l"(t));
    e0 = __uint_as_float(q0 + (t0 << 23));
    e1 = __uint_as_float(q1 + (t1 << 23));
}

// Score pairs J0 .. J1-1 of 16 scores -> packed fp16 p. PRECISE: also the fp16 remainder p - fp16(p) (exact in fp32, then
// rounded once more: together the pair carries p to about 22 bits).
template <int J0, int J1, bool PRECISE>
__device__ __forceinline__ void exp_pairs16(const uint32_t (&r)[16], uint32_t* pk, uint32_t* pkl, unsigned long long sl2x2, unsigned long long nm2) {
#pragma unroll
    for (int j = J0; j < J1; ++j) {
        if (LLATTN_SKIP & 2) { pk[j] = r[2 * j] & 0x03ff03ffu; continue; }
        float x0, x1;
        fma2(r[2 * j], r[2 * j + 1], sl2x2, nm2, x0, x1);
        float e0, e1;
        if (LLATTN_POLY_MOD > 0 && j % (LLATTN_POLY_MOD > 0 ? LLATTN_POLY_MOD : 1) == LLATTN_POLY_MOD - 1) exp2_pair_poly(x0, x1, e0, e1);
        else { e0 = ex2(x0); e1 = ex2(x1); }
        const half2 h = __floats2half2_rn(e0, e1);
        pk[j] = *reinterpret_cast<const uint32_t*>(&h);
        if (PRECISE) {
            const float2 hf = __half22float2(h);
            const half2 l = __floats2half2_rn(e0 - hf.x, e1 - hf.y);
            pkl[j] = *reinterpret_cast<const uint32_t*>(&l);
        }
    }
}

// p = 2^(s * scale * log2e - mref) must stay below the fp16 maximum. Rows whose chunk maximum `cs` is more than
// RESCALE_SLACK above their reference (`over`) move the reference to that maximum; what was accumulated under the old
// reference - O and the row sum of earlier tiles (`have_acc`), and the `chunks_done` chunks of this tile already turned
// into P - is rescaled. Warp-uniform call, rare (a key 2^8 times heavier than everything before it in the run), kept out
// of line so that the common path stays small.
// tlane: tensor-memory address of the warp's lanes at column 0; ts: the tile's S / P buffer; bar_pv, par_pv: barrier and
// parity of "PV of the previous tile has completed". Returns the row's new reference, NaN when that wait ran out.
__device__ __noinline__ float raise_reference(float mref, float cs, bool over, int chunks_done, bool have_acc, bool precise, uint32_t tlane,
                                              uint32_t ts, uint32_t bar_pv, uint32_t par_pv, volatile int* abort_flag) {
    const float mnew = over ? cs : mref;
    const float corr = over ? ex2(mref - mnew) : 1.f;      // 0 for a row that had no reference yet
    if (have_acc) {
        if (!ptx::mbar_wait(bar_pv, par_pv, abort_flag)) return __int_as_float(0x7fc00000);
        ptx::tc_fence_after();
#pragma unroll 1
        for (int oc = 0; oc < 4; ++oc) {
            uint32_t r[32];
            ptx::tmem_ld32(tlane + TM_O + 32 * oc, r);
            ptx::tmem_wait_ld_tied(r);
#pragma unroll
            for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) * corr);
            ptx::tmem_st32(tlane + TM_O + 32 * oc, r);
        }
        uint32_t r[16];
        ptx::tmem_ld16(tlane + TM_L, r);
        ptx::tmem_wait_ld_tied(r);
        r[0] = __float_as_uint(__uint_as_float(r[0]) * corr);
        ptx::tmem_st16(tlane + TM_L, r);
    }
    const half2 ch = __float2half2_rn(corr);
    // P chunk pc sits in columns 32 pc .. 32 pc + 15, its remainder (precise mode) in the 16 columns after them
#pragma unroll 1
    for (int pc = 0; pc < (precise ? 2 : 1) * chunks_done; ++pc) {
        uint32_t r[16];
        const uint32_t col = precise ? 16 * pc : 32 * pc;
        ptx::tmem_ld16(ts + col, r);
        ptx::tmem_wait_ld_tied(r);
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            const half2 h = __hmul2(*reinterpret_cast<const half2*>(&r[j]), ch);
            r[j] = *reinterpret_cast<const uint32_t*>(&h);
        }
        ptx::tmem_st16(ts + col, r);
    }
    ptx::tmem_wait_st();
    return mnew;
}

// One tile of NU 32-key chunks for one query row: S -> P in a single pass, branch-free except for the vote that guards
// the rare path. Scores arrive 16 columns at a time; the second half of the next chunk is requested once the first half
// of the current one has been consumed, its maximum is taken between the last exponentials of the current chunk, and P
// goes back over the first 16 of the 32 S columns it came from. Before the last chunk's exponentials the barrier of the
// next tile's S is tested (next_bar != 0), so that the test's latency is covered and the next tile starts without a wait
// when its S is already there. Returns false when a wait of the rare path ran out.
template <int NU, bool PRECISE>
__device__ __forceinline__ bool softmax_tile(float& mref, float sl2, unsigned long long sl2x2, uint32_t tlane, uint32_t ts, bool have_acc,
                                             uint32_t bar_pv, uint32_t par_pv, volatile int* abort_flag, uint32_t next_bar, uint32_t next_par,
                                             bool& next_ready) {
    unsigned long long nm2 = dup2(-mref);
    uint32_t a0[16], a1[16], b0[16], b1[16];
    ptx::tmem_ld16(ts, a0);
    ptx::tmem_ld16(ts + 16, a1);
    ptx::tmem_wait_ld_tied(a0, a1);
    float cm = fmaxf(rowmax16(a0), rowmax16(a1));
#pragma unroll
    for (int c = 0; c < NU; ++c) {
        uint32_t (&c0)[16] = (c & 1) ? b0 : a0;
        uint32_t (&c1)[16] = (c & 1) ? b1 : a1;
        uint32_t (&n0)[16] = (c & 1) ? a0 : b0;
        uint32_t (&n1)[16] = (c & 1) ? a1 : b1;
        const float cs = cm * sl2;
        const bool over = cs > mref + RESCALE_SLACK;
        if (__any_sync(0xffffffffu, over)) {
            mref = raise_reference(mref, cs, over, c, have_acc, PRECISE, tlane, ts, bar_pv, par_pv, abort_flag);
            if (__any_sync(0xffffffffu, mref != mref)) return false;
            nm2 = dup2(-mref);
        }
        uint32_t pk[16], pkl[PRECISE ? 16 : 1];
        if (c + 1 < NU) ptx::tmem_ld16(ts + 32 * (c + 1), n0);
        else next_ready = next_bar != 0 && ptx::mbar_try_wait(next_bar, next_par);
        exp_pairs16<0, 8, PRECISE>(c0, pk, pkl, sl2x2, nm2);
        ptx::tmem_st8(ts + 32 * c, pk);
        if (c + 1 < NU) ptx::tmem_ld16(ts + 32 * (c + 1) + 16, n1);
        exp_pairs16<0, 5, PRECISE>(c1, pk + 8, pkl + (PRECISE ? 8 : 0), sl2x2, nm2);
        if (c + 1 < NU) { ptx::tmem_wait_ld_tied(n0, n1); cm = fmaxf(rowmax16(n0), rowmax16(n1)); }
        exp_pairs16<5, 8, PRECISE>(c1, pk + 8, pkl + (PRECISE ? 8 : 0), sl2x2, nm2);
        ptx::tmem_st8(ts + 32 * c + 8, pk + 8);
        // the remainders go over the second half of the chunk's S columns: all 32 have been read by now
        if (PRECISE) { ptx::tmem_st8(ts + 32 * c + 16, pkl); ptx::tmem_st8(ts + 32 * c + 24, pkl + 8); }
    }
    return true;
}

// Byte offset of (key, 16-byte chunk c16 of its 128 channels) inside a K or V tile.
__device__ __forceinline__ int tile_off(int key, int c16) {
    return (c16 >> 3) * KBLOCK + key * 128 + (((c16 & 7) ^ (key & 7)) << 4);
}

// What a dequantising thread knows about itself: warp `wg` of its group, half `h16` of the warp, chunk `c16`.
// With G warps in a group, K pass p handles key 2 G p + 2 wg + h16 and V pass p key (32 / G) wg + 2 p + h16: either way
// a warp's load covers two adjacent keys (128 contiguous bytes of codes) and a quarter warp stores one key's row.
struct DqThread {
    int k_src, k_dst;      // pass p: k_src + 128 G p; (k_dst ^ swizzle flip of odd passes when G = 2) + 256 G p
    int v_src, v_dst;      // pass p adds 128 to v_src; v_dst: (v_dst ^ 32 (p % 4)) + 256 p
    int c16, wg;
    uint32_t hsel;         // byte-permute selector that broadcasts this thread's half of a word of two fp16
};
__device__ __forceinline__ DqThread dq_thread(int dt) {
    DqThread d;
    const int lane = dt & 31, h16 = lane >> 4;
    d.wg = dt >> 5; d.c16 = lane & 15;
    const int kb = 2 * d.wg + h16, vb = (32 / GROUP_WARPS) * d.wg + h16;
    d.k_src = kb * 64 + d.c16 * 4;
    d.k_dst = tile_off(kb, d.c16);
    d.v_src = VOFF + vb * 64 + d.c16 * 4;
    d.v_dst = tile_off(vb, d.c16);
    d.hsel = h16 ? 0x3232u : 0x1010u;
    return d;
}

// K half of one staged record -> fp16 rows of a K tile (Kt points at the unit's first key). Scale and minimum are per
// channel: one pair of 16-byte loads per thread and record.
__device__ __forceinline__ void dequant_k(const uint8_t* raw, uint8_t* Kt, const DqThread& d) {
    const uint4 s4 = permute8(*reinterpret_cast<const uint4*>(raw + KOFF_META + d.c16 * 16));
    const uint4 m4 = permute8(*reinterpret_cast<const uint4*>(raw + KOFF_META + 256 + d.c16 * 16));
    const half2* ks = reinterpret_cast<const half2*>(&s4);
    const half2* km = reinterpret_cast<const half2*>(&m4);
    // every code word of the thread first: the compiler cannot tell the record ring from the operand tile, so a load
    // written after a store would wait for it, and each pass would pay the full shared-memory latency
    uint32_t w[DQ_PASSES];
#pragma unroll
    for (int p = 0; p < DQ_PASSES; ++p) w[p] = *reinterpret_cast<const uint32_t*>(raw + d.k_src + p * 128 * GROUP_WARPS);
#pragma unroll
    for (int p = 0; p < DQ_PASSES; ++p) {
        half2 kh[4];
        unpack8(w[p], kh);
#pragma unroll
        for (int j = 0; j < 4; ++j) kh[j] = __hfma2(kh[j], ks[j], km[j]);
        // key 2 G p + kb: with G = 2 the odd passes land 4 keys further, which flips bit 2 of the swizzled chunk position
        const int flip = GROUP_WARPS == 2 ? 64 * (p & 1) : 0;
        *reinterpret_cast<uint4*>(Kt + (d.k_dst ^ flip) + p * 256 * GROUP_WARPS) = *reinterpret_cast<const uint4*>(kh);
    }
}
// V half: scale and minimum per key; the warp's eight keys' values arrive in one broadcast 16-byte load each.
__device__ __forceinline__ void dequant_v(const uint8_t* raw, uint8_t* Vt, const DqThread& d) {
    uint4 s4[DQ_PASSES / 4], m4[DQ_PASSES / 4];       // scale and minimum of the warp's 32 / G keys
#pragma unroll
    for (int k = 0; k < DQ_PASSES / 4; ++k) {
        s4[k] = *reinterpret_cast<const uint4*>(raw + VOFF_META + (d.wg * (DQ_PASSES / 4) + k) * 16);
        m4[k] = *reinterpret_cast<const uint4*>(raw + VOFF_META + 2 * BLK + (d.wg * (DQ_PASSES / 4) + k) * 16);
    }
    const uint32_t* sw = reinterpret_cast<const uint32_t*>(s4);
    const uint32_t* mw = reinterpret_cast<const uint32_t*>(m4);
    uint32_t w[DQ_PASSES];
#pragma unroll
    for (int p = 0; p < DQ_PASSES; ++p) w[p] = *reinterpret_cast<const uint32_t*>(raw + d.v_src + p * 128);
#pragma unroll
    for (int p = 0; p < DQ_PASSES; ++p) {
        const uint32_t vsu = __byte_perm(sw[p], sw[p], d.hsel), vmu = __byte_perm(mw[p], mw[p], d.hsel);
        const half2 vs = *reinterpret_cast<const half2*>(&vsu), vm = *reinterpret_cast<const half2*>(&vmu);
        half2 vh[4];
        unpack8(w[p], vh);
#pragma unroll
        for (int j = 0; j < 4; ++j) vh[j] = __hfma2(vh[j], vs, vm);
        *reinterpret_cast<uint4*>(Vt + (d.v_dst ^ (32 * (p & 3))) + 256 * p) = *reinterpret_cast<const uint4*>(vh);
    }
}
// The query block's own fp16 K or V (32 keys x 128 channels, row stride NKV * D halves) into a unit of a tile.
__device__ __forceinline__ void copy_fresh(const half* src, uint8_t* tile_unit, int dt) {
#pragma unroll
    for (int k = 0; k < 512 / GROUP_THREADS; ++k) {
        const int idx = dt + GROUP_THREADS * k, tok = idx >> 4, c16 = idx & 15;
        *reinterpret_cast<uint4*>(tile_unit + tile_off(tok, c16)) =
            permute8(__ldg(reinterpret_cast<const uint4*>(src + size_t(tok) * NKV * D + c16 * 8)));
    }
}

// The whole CTA's work. `cta` is the CTA's index in the plan (list mode) or in the flattened reference grid
// (kv head fastest, then chunk, then query block).
// PRECISE: P is carried as fp16 value + fp16 remainder (two PV chains per tile), for callers that need the result to
// within 2e-3 of the output RMS at long contexts and accept about half the throughput.
template <bool PRECISE>
__device__ __forceinline__ void attn_tile_body(const KParams& p, const int cta) {
    extern __shared__ __align__(1024) uint8_t smem[];
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + SM_BAR);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + SM_MISC);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + SM_MISC + 4);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t bar0 = ptx::smem_u32(bars);
    auto BAR = [&](int i) -> uint32_t { return bar0 + 8u * uint32_t(i); };

    int i0, i1;
    if (p.items) { i0 = p.cta_first[cta]; i1 = p.cta_first[cta + 1]; }
    else { i0 = cta; i1 = cta + 1; }
    const int i0_any = i0, i1_any = i1;
    if (ptx::smem_u32(smem) & 1023u) {          // the swizzled tiles need a 1024-byte aligned base: report, do nothing
        if (tid == 0 && p.err) atomicOr(p.err, ERR_SMEM_ALIGN);
        return;
    }

    if (tid == 0) {
        for (int i = 0; i < NRAW; ++i) { ptx::mbar_init(BAR(B_RAW_FULL + i), 1); ptx::mbar_init(BAR(B_RAW_EMPTY + i), GROUP_THREADS); }
        for (int i = 0; i < 2; ++i) {
            ptx::mbar_init(BAR(B_K_FULL + i), 32 * DEQUANT_WARPS); ptx::mbar_init(BAR(B_V_FULL + i), 32 * DEQUANT_WARPS);
            ptx::mbar_init(BAR(B_K_FREE + i), 1); ptx::mbar_init(BAR(B_PV_DONE + i), 1);
            ptx::mbar_init(BAR(B_S_FULL + i), 1); ptx::mbar_init(BAR(B_P_FULL + i), P_ARRIVALS);
        }
        ptx::mbar_init(BAR(B_Q_FULL), 32 * SOFTMAX_WARPS); ptx::mbar_init(BAR(B_O_FREE), 32 * SOFTMAX_WARPS);
        ptx::mbar_init(BAR(B_SPARE), 1);
        ptx::mbar_init(BAR(B_SPARE + 1), 1);
        ptx::fence_mbar_init();
        *abort_flag = 0;
    }
    // the first run's descriptor comes in while the barriers and tensor memory are being set up
    const RunDesc* first_run = reinterpret_cast<const RunDesc*>(smem + SM_FIRST);
    if (p.items && i0 < i1 && warp == 1 && lane < 16)
        reinterpret_cast<uint32_t*>(smem + SM_FIRST)[lane] = __ldg(reinterpret_cast<const uint32_t*>(p.items + i0) + lane);
    if (warp == WARP_MMA) { ptx::tmem_alloc(ptx::smem_u32(tmem_slot), TMEM_COLS); ptx::tmem_relinquish(); }
    ptx::tc_fence_before();
    __syncthreads();
    ptx::tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    const uint32_t tmem_any = tmem;
    int errbits = 0;
#ifdef LLATTN_TRACE
    int trace_n = 0;
    unsigned long long* trace_ptr = (blockIdx.x == 0 && lane == 0 && g_trace_buf) ? g_trace_buf + warp * LLATTN_TRACE_EVENTS : nullptr;
#endif

    if (warp < SOFTMAX_WARPS) {
        // ================================================================== softmax + epilogue
        // thread = query row = TMEM lane (warp w owns lanes 32 w .. 32 w + 31): it sees all keys of its row, so the row
        // maximum needs no exchange with other warps. One pass per tile: a 32-key chunk of S is loaded while the previous
        // chunk's exponentials run, its maximum is taken between them, and P goes back over the first 16 of the S columns
        // it came from.
        const int row = warp * 32 + lane;
        const uint32_t tlane = tmem + (uint32_t(warp * 32) << 16);
        const unsigned long long sl2x2 = dup2(p.sl2);
        uint32_t t = 0;
        bool alive = true;
#pragma unroll 1
        for (int ii = i0; ii < i1 && alive; ++ii) {
            WorkItem w; SeqDesc s;
            if (!fetch_item(p, ii, w, s, first_run, i0_any)) continue;
            const int U = w.rec_count + w.fresh, ntiles = (U + TILE_UNITS - 1) / TILE_UNITS;
            // Reference exponent of the row, log2 units: the exact maximum of the run's first tile (a row dominated by a
            // key of that tile then has p = 1 for it, without rounding); it moves only when a later score exceeds it by
            // more than RESCALE_SLACK (engine/attn.cu:237-255 moves its reference lazily in the same way).
            float mref = -INFINITY;
            bool s_ready = false;              // the tile's S has been seen complete already (tested during the previous tile)
            {   // this thread's query row into tensor memory as fp16 pairs. Every S MMA of the previous item has completed:
                // this warp has seen the S of its last tile.
                const half* src = p.Q + ((size_t(s.q_first + w.qblk) * BLK + (row >> 2)) * NQH + 4 * w.kvh + (row & 3)) * D;
#pragma unroll 1
                for (int c = 0; c < 4; ++c) {
                    uint32_t r[16];
#pragma unroll
                    for (int g = 0; g < 4; ++g) {
                        const uint4 v = permute8(__ldg(reinterpret_cast<const uint4*>(src + 32 * c + 8 * g)));
                        r[4 * g] = v.x; r[4 * g + 1] = v.y; r[4 * g + 2] = v.z; r[4 * g + 3] = v.w;
                    }
                    ptx::tmem_st16(tlane + TM_Q + 16 * c, r);
                }
                ptx::tmem_wait_st();
                ptx::tc_fence_before();
                ptx::mbar_arrive(BAR(B_Q_FULL));
            }
#pragma unroll 1
            for (int i = 0; i < ntiles && alive; ++i, ++t) {
                const int b = t & 1, nu = min(TILE_UNITS, U - TILE_UNITS * i);
                LLATTN_TR(1, t);
                if (!s_ready && !ptx::mbar_wait(BAR(B_S_FULL + b), (t >> 1) & 1, abort_flag)) { alive = false; errbits |= ERR_WAIT_SOFTMAX; break; }
                LLATTN_TR(2, t);
                ptx::tc_fence_after();
                const uint32_t ts = tlane + TM_S + b * 128, bar_pv = BAR(B_PV_DONE + (b ^ 1)), par_pv = ((t - 1) >> 1) & 1;
                // the next tile's S (other buffer) is tested for during this tile's last chunk, except across runs
                const uint32_t next_bar = i + 1 < ntiles ? BAR(B_S_FULL + (b ^ 1)) : 0u, next_par = ((t + 1) >> 1) & 1;
                if (i == 0) {
                    float mx = -INFINITY;
#pragma unroll 1
                    for (int c = 0; c < nu; ++c) {
                        uint32_t r[32];
                        ptx::tmem_ld32(ts + 32 * c, r);
                        ptx::tmem_wait_ld_tied(r);
                        mx = fmaxf(mx, rowmax32(r));
                    }
                    mref = mx * p.sl2;
                }
                bool ok;
                if (nu == TILE_UNITS) ok = softmax_tile<TILE_UNITS, PRECISE>(mref, p.sl2, sl2x2, tlane, ts, i > 0, bar_pv, par_pv, abort_flag, next_bar, next_par, s_ready);      // every tile of a run but its last
                else if (nu == 3) ok = softmax_tile<3, PRECISE>(mref, p.sl2, sl2x2, tlane, ts, i > 0, bar_pv, par_pv, abort_flag, next_bar, next_par, s_ready);
                else if (nu == 2) ok = softmax_tile<2, PRECISE>(mref, p.sl2, sl2x2, tlane, ts, i > 0, bar_pv, par_pv, abort_flag, next_bar, next_par, s_ready);
                else ok = softmax_tile<1, PRECISE>(mref, p.sl2, sl2x2, tlane, ts, i > 0, bar_pv, par_pv, abort_flag, next_bar, next_par, s_ready);
                if (!ok) { alive = false; errbits |= ERR_WAIT_SOFTMAX; }
                if (!alive) break;
                ptx::tmem_wait_st();
                ptx::tc_fence_before();
#if LLATTN_WARP_ARRIVE
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(BAR(B_P_FULL + b));
#else
                ptx::mbar_arrive(BAR(B_P_FULL + b));
#endif
                LLATTN_TR(4, t);
            }
            if (!alive) break;
            // ---- epilogue. A run that is its tile's only one writes the outputs straight from tensor memory. Otherwise
            // it stores its un-normalised O, reference exponent and row sum as a partial result and counts itself in at
            // the tile's arrival counter; the tile's runs fold it together once the CTAs have no runs left (end of this
            // function).
            const uint32_t tl = t - 1;
            if (!ptx::mbar_wait(BAR(B_PV_DONE + (tl & 1)), (tl >> 1) & 1, abort_flag)) { alive = false; errbits |= ERR_WAIT_SOFTMAX; break; }
            ptx::tc_fence_after();
            float lsum;
            {
                uint32_t r[16];
                ptx::tmem_ld16(tlane + TM_L, r);
                ptx::tmem_wait_ld_tied(r);
                lsum = __uint_as_float(r[0]);
            }
            const bool fused = p.merge != nullptr;
            MergeDesc md{0, 0, 0, 1};
            if (fused) md = p.merge[w.tile];
            bool finish = fused && md.nslots == 1;
            float M = mref, den = lsum;
            if (!finish) {
                float* orow = p.Opart + (size_t(w.slot) * QR + row) * D;
#pragma unroll 1
                for (int c = 0; c < 4; ++c) {
                    uint32_t r[32];
                    ptx::tmem_ld32(tlane + TM_O + 32 * c, r);
                    ptx::tmem_wait_ld_tied(r);
#pragma unroll
                    for (int g = 0; g < 4; ++g) {      // positions (0..7) hold dims (0,4,1,5,2,6,3,7)
                        const float4 lo = make_float4(__uint_as_float(r[8 * g]), __uint_as_float(r[8 * g + 2]),
                                                      __uint_as_float(r[8 * g + 4]), __uint_as_float(r[8 * g + 6]));
                        const float4 hi = make_float4(__uint_as_float(r[8 * g + 1]), __uint_as_float(r[8 * g + 3]),
                                                      __uint_as_float(r[8 * g + 5]), __uint_as_float(r[8 * g + 7]));
                        *reinterpret_cast<float4*>(orow + 32 * c + 8 * g) = lo;
                        *reinterpret_cast<float4*>(orow + 32 * c + 8 * g + 4) = hi;
                    }
                }
                // the accumulator has been read: the next run's PV may start while the stores below drain
                ptx::tc_fence_before();
                ptx::mbar_arrive(BAR(B_O_FREE));
                p.Lpart[size_t(w.slot) * QR + row] = lsum;
                p.Mpart[size_t(w.slot) * QR + row] = mref;
                if (fused) {                   // this warp's 32 rows of the run are out: count it in
                    __threadfence();
                    __syncwarp();
                    if (lane == 0) atomicAdd(p.tile_counters + 4 * w.tile, 1);
                }
            }
            if (finish) {
                const float inv = 1.f / den;
                RowOut ro{size_t(md.q_index) * BLK + (row >> 2), 4 * md.kvh + (row & 3), 0.f, 0};
                if (p.out.q8) {        // the int8 form needs the row's largest magnitude first
                    float m = 0.f;
#pragma unroll 1
                    for (int c = 0; c < 4; ++c) {
                        uint32_t r[32];
                        ptx::tmem_ld32(tlane + TM_O + 32 * c, r);
                        ptx::tmem_wait_ld_tied(r);
#pragma unroll
                        for (int j = 0; j < 32; ++j) m = fmaxf(m, fabsf(__uint_as_float(r[j]) * inv));
                    }
                    ro.qscale = fmaxf(__fdiv_rn(m, 127.f), 1e-30f);
                }
#pragma unroll 1
                for (int c = 0; c < 4; ++c) {
                    uint32_t r[32];
                    float v[32];
                    ptx::tmem_ld32(tlane + TM_O + 32 * c, r);
                    ptx::tmem_wait_ld_tied(r);
#pragma unroll
                    for (int g = 0; g < 4; ++g)
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            v[8 * g + k] = __uint_as_float(r[8 * g + 2 * k]) * inv;
                            v[8 * g + 4 + k] = __uint_as_float(r[8 * g + 2 * k + 1]) * inv;
                        }
                    row_store(p.out, ro, c, v);
                }
                row_finish(p.out, ro, M, den);
                ptx::tc_fence_before();
                ptx::mbar_arrive(BAR(B_O_FREE));
            }
        }
    } else if (warp < WARP_SERVICE) {
        // ================================================================== dequant: records -> fp16 operand tiles
        const int da = tid - 32 * SOFTMAX_WARPS;      // over all groups
        const int grp = da / GROUP_THREADS, dt = da % GROUP_THREADS;       // group g owns units g, g + groups, ... of every tile
        const DqThread dq = dq_thread(dt);
        uint32_t t = 0, r = 0;
        bool alive = true;
        // third block of both V tiles: column 128 of V is all ones (O column 128 accumulates sum(P)), 129..143 zero.
        // Published by the first v_full arrival.
        for (int idx = da; idx < 2 * 128 * 8; idx += 32 * DEQUANT_WARPS) {
            const int buf = idx >> 10, key = (idx >> 3) & 127, pos = idx & 7;
            *reinterpret_cast<uint4*>(smem + SM_V + buf * VTILE_BYTES + 2 * KBLOCK + key * 128 + pos * 16) =
                make_uint4(pos == (key & 7) ? 0x00003C00u : 0u, 0u, 0u, 0u);
        }
#pragma unroll 1
        for (int ii = i0; ii < i1 && alive; ++ii) {
            WorkItem w; SeqDesc s;
            if (!fetch_item(p, ii, w, s, first_run, i0_any)) continue;
            const int U = w.rec_count + w.fresh, ntiles = (U + TILE_UNITS - 1) / TILE_UNITS;
            const size_t f0 = (size_t(s.q_first + w.qblk) * BLK) * NKV * D + size_t(w.kvh) * D;
            int i = 0;
            // ---- steady state: tiles made of four committed records. This group's units are always there, nothing is
            // decided per tile, and the loop carries only what changes (tile count, record count).
            const int nfull = w.rec_count / TILE_UNITS;
#pragma unroll 1
            for (; i < nfull; ++i, ++t) {
                const uint32_t b = t & 1, freed = ((t >> 1) - 1) & 1;      // phase in which tile t-2 let go of its buffers
                LLATTN_TR(10, t);
                if (t >= 2 && !ptx::mbar_wait(BAR(B_K_FREE + b), freed, abort_flag)) { alive = false; errbits |= ERR_WAIT_DEQUANT; break; }
                LLATTN_TR(15, t);
#pragma unroll
                for (int u = 0; u < TILE_UNITS / DEQUANT_GROUPS; ++u) {
                    const uint32_t rr = r + grp + u * DEQUANT_GROUPS, slot = rr % NRAW;
                    if (!ptx::mbar_wait(BAR(B_RAW_FULL + slot), (rr / NRAW) & 1, abort_flag)) { alive = false; errbits |= ERR_WAIT_DEQUANT; break; }
                    if (!(LLATTN_SKIP & 1))
                        dequant_k(smem + SM_RAW + slot * RAW_STRIDE, smem + SM_K + b * TILE_BYTES + (grp + u * DEQUANT_GROUPS) * UNIT_BYTES, dq);
                }
                if (!alive) break;
                LLATTN_TR(16, t);
                ptx::fence_proxy_async_smem();
                ptx::mbar_arrive(BAR(B_K_FULL + b));
                LLATTN_TR(12, t);
                if (t >= 2 && !ptx::mbar_wait(BAR(B_PV_DONE + b), freed, abort_flag)) { alive = false; errbits |= ERR_WAIT_DEQUANT; break; }
                LLATTN_TR(13, t);
#pragma unroll
                for (int u = 0; u < TILE_UNITS / DEQUANT_GROUPS; ++u) {
                    const uint32_t rr = r + grp + u * DEQUANT_GROUPS, slot = rr % NRAW;
                    if (!(LLATTN_SKIP & 1))
                        dequant_v(smem + SM_RAW + slot * RAW_STRIDE, smem + SM_V + b * VTILE_BYTES + (grp + u * DEQUANT_GROUPS) * UNIT_BYTES, dq);
                    ptx::mbar_arrive(BAR(B_RAW_EMPTY + slot));
                }
                ptx::fence_proxy_async_smem();
                ptx::mbar_arrive(BAR(B_V_FULL + b));
                LLATTN_TR(14, t);
                r += TILE_UNITS;
            }
            // ---- the run's last tile: fewer than four records and / or the query block's own K/V
#pragma unroll 1
            for (; i < ntiles && alive; ++i, ++t) {
                const int b = t & 1, nu = min(TILE_UNITS, U - TILE_UNITS * i);
                uint8_t* Kt = smem + SM_K + b * TILE_BYTES;
                uint8_t* Vt = smem + SM_V + b * VTILE_BYTES;
                // ---- K: the tile's K buffer is free once S of tile t-2 has been computed
                LLATTN_TR(10, t);
                if (t >= 2 && !ptx::mbar_wait(BAR(B_K_FREE + b), ((t >> 1) - 1) & 1, abort_flag)) { alive = false; errbits |= ERR_WAIT_DEQUANT; break; }
                LLATTN_TR(11, t);
#pragma unroll 1
                for (int u = grp; u < nu; u += DEQUANT_GROUPS) {
                    const int unit = TILE_UNITS * i + u;
                    if (unit < w.rec_count) {
                        const uint32_t rr = r + u, slot = rr % NRAW;
                        LLATTN_TR(15, t);
                        if (!ptx::mbar_wait(BAR(B_RAW_FULL + slot), (rr / NRAW) & 1, abort_flag)) { alive = false; errbits |= ERR_WAIT_DEQUANT; break; }
                        LLATTN_TR(16, t);
                        if (!(LLATTN_SKIP & 1)) dequant_k(smem + SM_RAW + slot * RAW_STRIDE, Kt + u * UNIT_BYTES, dq);
                    } else {          // the query block's own K, exact fp16
                        copy_fresh(p.Kf + f0, Kt + u * UNIT_BYTES, dt);
                    }
                }
                if (!alive) break;
                ptx::fence_proxy_async_smem();
                ptx::mbar_arrive(BAR(B_K_FULL + b));
                LLATTN_TR(12, t);
                // ---- V: free once PV of tile t-2 has been computed
                if (t >= 2 && !ptx::mbar_wait(BAR(B_PV_DONE + b), ((t >> 1) - 1) & 1, abort_flag)) { alive = false; errbits |= ERR_WAIT_DEQUANT; break; }
                LLATTN_TR(13, t);
#pragma unroll 1
                for (int u = grp; u < nu; u += DEQUANT_GROUPS) {
                    const int unit = TILE_UNITS * i + u;
                    if (unit < w.rec_count) {
                        const uint32_t slot = (r + u) % NRAW;       // landed: the K pass waited for it
                        if (!(LLATTN_SKIP & 1)) dequant_v(smem + SM_RAW + slot * RAW_STRIDE, Vt + u * UNIT_BYTES, dq);
                        ptx::mbar_arrive(BAR(B_RAW_EMPTY + slot));
                    } else {
                        copy_fresh(p.Vf + f0, Vt + u * UNIT_BYTES, dt);
                    }
                }
                ptx::fence_proxy_async_smem();
                ptx::mbar_arrive(BAR(B_V_FULL + b));
                LLATTN_TR(14, t);
                r += uint32_t(min(nu, max(0, w.rec_count - TILE_UNITS * i)));     // records of this tile (both groups count alike)
            }
        }
    } else if (warp >= WARP_PRODUCER) {
        // ================================================================== producers: bulk copies of records
        // producer k takes the records whose running number r is k modulo PRODUCERS
        const uint32_t pk = uint32_t(warp - WARP_PRODUCER);
        uint32_t r0 = 0, last = 0, issued = 0;        // records before this item; this producer's latest record
        bool alive = true;
#pragma unroll 1
        for (int ii = i0; ii < i1 && alive; ++ii) {
            WorkItem w; SeqDesc s;
            if (!fetch_item(p, ii, w, s, first_run, i0_any)) continue;
            const size_t hbase = size_t(w.kvh) * s.head_stride;
#pragma unroll 1
            for (uint32_t u = (pk - r0) % PRODUCERS; u < uint32_t(w.rec_count); u += PRODUCERS) {
                const uint32_t r = r0 + u, slot = r % NRAW;
                if (r >= NRAW && !ptx::mbar_wait(BAR(B_RAW_EMPTY + slot), ((r / NRAW) - 1) & 1, abort_flag)) { alive = false; errbits |= ERR_WAIT_PRODUCER; break; }
                if (lane == 0) {
                    const size_t ridx = s.pages ? size_t(s.pages[hbase + w.rec_begin + u]) : hbase + w.rec_begin + u;
                    ptx::mbar_arrive_expect_tx(BAR(B_RAW_FULL + slot), REC_BYTES);
                    ptx::bulk_g2s(ptx::smem_u32(smem + SM_RAW + slot * RAW_STRIDE), s.cache + ridx * REC_BYTES, REC_BYTES,
                                  BAR(B_RAW_FULL + slot));
                }
                __syncwarp();
                last = r; ++issued;
            }
            r0 += uint32_t(w.rec_count);
        }
        // copies still in flight must land before the shared memory is given back
        if (*abort_flag) {
            const uint32_t n = issued < NRAW / PRODUCERS ? issued : NRAW / PRODUCERS;
            for (uint32_t k = 0; k < n; ++k) {
                const uint32_t rr = last - PRODUCERS * k;
                volatile int never = 0;
                ptx::mbar_wait(BAR(B_RAW_FULL + rr % NRAW), (rr / NRAW) & 1, &never);
            }
        }
    } else if (warp == WARP_MMA) {
        // ================================================================== MMA issue (one elected lane issues, the warp stays together)
        // Loop bounds, tile counts and wait results are made visibly warp-uniform so that the operands of the MMAs can
        // live in uniform registers.
        uint32_t t = 0, itc = 0;
        bool alive = true;
        // one base descriptor per K buffer (K-major, 128-byte swizzle, 8-row groups 1024 B apart); the issue helper steps it
        const uint32_t k_s = ptx::smem_u32(smem + SM_K);
        const uint32_t klo0 = ptx::desc_lo(k_s, 16), klo1 = ptx::desc_lo(k_s + TILE_BYTES, 16), khi = ptx::desc_hi(1024) | (2u << 29);
        const uint32_t tmem = uniform_u32(tmem_any);
        const int i0 = uniform_i32(i0_any), i1 = uniform_i32(i1_any);
#if LLATTN_SINGLE_ISSUER
        // This warp issues everything, per tile t in the order PV(t), S(t+2). S(t+2) overwrites the buffer that holds P(t);
        // the tensor pipe executes the MMAs of one thread in issue order, so no wait for PV(t) to complete is needed.
        const uint32_t v_s = ptx::smem_u32(smem + SM_V);
        const uint32_t idO = ptx::idesc_f16(128, PV_N, false, true);
        const uint32_t vlo0 = ptx::desc_lo(v_s, KBLOCK), vlo1 = ptx::desc_lo(v_s + VTILE_BYTES, KBLOCK), vhi = ptx::desc_hi(1024) | (2u << 29);
        auto issue_s = [&](uint32_t tt, int nu) -> bool {
            const uint32_t b = tt & 1;
            if (!uniform_i32(ptx::mbar_wait(BAR(B_K_FULL + b), (tt >> 1) & 1, abort_flag))) return false;
            ptx::tc_fence_after();
            const uint32_t idS = ptx::idesc_f16(128, 32 * nu, false, false);
            ptx::mma_ts_s8_warp<KBLOCK / 16>(tmem + TM_S + b * 128, tmem + TM_Q, b ? klo1 : klo0, khi, idS, BAR(B_S_FULL + b), BAR(B_K_FREE + b));
            return true;
        };
#pragma unroll 1
        for (int ii = i0; ii < i1 && alive; ++ii) {
            WorkItem w; SeqDesc s;
            if (!uniform_i32(fetch_item(p, ii, w, s, first_run, i0_any))) continue;
            const int U = uniform_i32(w.rec_count + w.fresh), ntiles = (U + TILE_UNITS - 1) / TILE_UNITS;
            if (!uniform_i32(ptx::mbar_wait(BAR(B_Q_FULL), itc & 1, abort_flag))) { alive = false; errbits |= ERR_WAIT_MMA; break; }
            for (int j = 0; j < 2 && j < ntiles && alive; ++j)
                if (!issue_s(t + j, min(TILE_UNITS, U - TILE_UNITS * j))) { alive = false; errbits |= ERR_WAIT_MMA; }
#pragma unroll 1
            for (int i = 0; i < ntiles && alive; ++i, ++t) {
                const uint32_t b = t & 1;
                const int nu = min(TILE_UNITS, U - TILE_UNITS * i);
                LLATTN_TR(22, t);
                if (!uniform_i32(ptx::mbar_wait(BAR(B_V_FULL + b), (t >> 1) & 1, abort_flag))) { alive = false; errbits |= ERR_WAIT_MMA; break; }
                if (!uniform_i32(ptx::mbar_wait(BAR(B_P_FULL + b), (t >> 1) & 1, abort_flag))) { alive = false; errbits |= ERR_WAIT_MMA; break; }
                LLATTN_TR(24, t);
                // the previous item's epilogue must have read O before the first PV of this item overwrites it
                if (i == 0 && itc > 0 && !uniform_i32(ptx::mbar_wait(BAR(B_O_FREE), (itc - 1) & 1, abort_flag))) { alive = false; errbits |= ERR_WAIT_MMA; break; }
                ptx::tc_fence_after();
                {
                    const uint32_t pb = tmem + TM_S + b * 128, vlo = b ? vlo1 : vlo0;
                    if (nu == TILE_UNITS) {
                        if (PRECISE) {
                            ptx::mma_ts_pv8_warp<false>(tmem + TM_O, pb, vlo, vhi, idO, i == 0 ? 0u : 1u, 0u);
                            ptx::mma_ts_pv8_warp<true>(tmem + TM_O, pb + 16, vlo, vhi, idO, 1u, BAR(B_PV_DONE + b));     // the remainders of P
                        } else {
                            ptx::mma_ts_pv8_warp<true>(tmem + TM_O, pb, vlo, vhi, idO, i == 0 ? 0u : 1u, BAR(B_PV_DONE + b));
                        }
                    } else {
#pragma unroll
                        for (int u = 0; u < TILE_UNITS - 1; ++u)
                            if (u < nu) {
                                const uint64_t d0 = (uint64_t(vhi) << 32) | (vlo + 256u * u);
                                ptx::mma_ts_x2_warp(tmem + TM_O, pb + 32 * u, d0, d0 + 128, idO, (i == 0 && u == 0) ? 0u : 1u);
                                if (PRECISE) ptx::mma_ts_x2_warp(tmem + TM_O, pb + 32 * u + 16, d0, d0 + 128, idO, 1u);
                            }
                        ptx::mma_commit_warp(BAR(B_PV_DONE + b));
                    }
                }
                LLATTN_TR(26, t);
                if (i + 2 < ntiles && !issue_s(t + 2, min(TILE_UNITS, U - TILE_UNITS * (i + 2)))) { alive = false; errbits |= ERR_WAIT_MMA; break; }
                LLATTN_TR(25, t);
            }
            ++itc;
        }
#else
        // S = Q K^T issue; the PV warp below issues O += P V. Two issuing warps halve the per-tile instruction chain.
#pragma unroll 1
        for (int ii = i0; ii < i1 && alive; ++ii) {
            WorkItem w; SeqDesc s;
            if (!uniform_i32(fetch_item(p, ii, w, s, first_run, i0_any))) continue;
            const int U = uniform_i32(w.rec_count + w.fresh), ntiles = (U + TILE_UNITS - 1) / TILE_UNITS;
            if (!uniform_i32(ptx::mbar_wait(BAR(B_Q_FULL), itc & 1, abort_flag))) { alive = false; errbits |= ERR_WAIT_MMA; break; }
#pragma unroll 1
            for (int i = 0; i < ntiles; ++i, ++t) {
                const uint32_t b = t & 1;
                const int nu = min(TILE_UNITS, U - TILE_UNITS * i);
                LLATTN_TR(20, t);
                if (!uniform_i32(ptx::mbar_wait(BAR(B_K_FULL + b), (t >> 1) & 1, abort_flag))) { alive = false; errbits |= ERR_WAIT_MMA; break; }
                // S buffer b also holds P of tile t-2: PV of that tile must have consumed it
                if (t >= 2 && !uniform_i32(ptx::mbar_wait(BAR(B_PV_DONE + b), ((t >> 1) - 1) & 1, abort_flag))) { alive = false; errbits |= ERR_WAIT_MMA; break; }
                LLATTN_TR(21, t);
                ptx::tc_fence_after();
                {
                    const uint32_t idS = ptx::idesc_f16(128, 32 * nu, false, false), ds = tmem + TM_S + b * 128;
                    ptx::mma_ts_s8_warp<KBLOCK / 16>(ds, tmem + TM_Q, b ? klo1 : klo0, khi, idS, BAR(B_S_FULL + b), BAR(B_K_FREE + b));
                }
                LLATTN_TR(25, t);
            }
            ++itc;
        }
#endif
        // every MMA issued must have retired before tensor memory is released
        ptx::mma_commit_warp(BAR(B_SPARE));
        {
            volatile int never = 0;
            if (!ptx::mbar_wait(BAR(B_SPARE), 0, &never)) errbits |= ERR_WAIT_TEARDOWN;
        }
    } else {
#if !LLATTN_SINGLE_ISSUER
        // ================================================================== O += P V issue
        uint32_t t = 0, itc = 0;
        bool alive = true;
        const uint32_t v_s = ptx::smem_u32(smem + SM_V);
        const uint32_t idO = ptx::idesc_f16(128, PV_N, false, true);
        // one base descriptor per V buffer (MN-major, 128-byte swizzle: 8-key groups 1024 B apart, 64-dim blocks KBLOCK apart)
        const uint32_t vlo0 = ptx::desc_lo(v_s, KBLOCK), vlo1 = ptx::desc_lo(v_s + VTILE_BYTES, KBLOCK), vhi = ptx::desc_hi(1024) | (2u << 29);
        const uint32_t tmem = uniform_u32(tmem_any);
        const int i0 = uniform_i32(i0_any), i1 = uniform_i32(i1_any);
#pragma unroll 1
        for (int ii = i0; ii < i1 && alive; ++ii) {
            WorkItem w; SeqDesc s;
            if (!uniform_i32(fetch_item(p, ii, w, s, first_run, i0_any))) continue;
            const int U = uniform_i32(w.rec_count + w.fresh), ntiles = (U + TILE_UNITS - 1) / TILE_UNITS;
#pragma unroll 1
            for (int i = 0; i < ntiles; ++i, ++t) {
                const uint32_t b = t & 1;
                const int nu = min(TILE_UNITS, U - TILE_UNITS * i);
                LLATTN_TR(22, t);
                if (!uniform_i32(ptx::mbar_wait(BAR(B_V_FULL + b), (t >> 1) & 1, abort_flag))) { alive = false; errbits |= ERR_WAIT_MMA; break; }
                LLATTN_TR(23, t);
                if (!uniform_i32(ptx::mbar_wait(BAR(B_P_FULL + b), (t >> 1) & 1, abort_flag))) { alive = false; errbits |= ERR_WAIT_MMA; break; }
                LLATTN_TR(24, t);
                // the previous item's epilogue must have read O before the first PV of this item overwrites it
                if (i == 0 && itc > 0 && !uniform_i32(ptx::mbar_wait(BAR(B_O_FREE), (itc - 1) & 1, abort_flag))) { alive = false; errbits |= ERR_WAIT_MMA; break; }
                ptx::tc_fence_after();
                {
                    // unit u = keys 32u..32u+31 = K-steps 2u, 2u+1; its P sits at columns 32u .. 32u+15 of the S buffer
                    const uint32_t pb = tmem + TM_S + b * 128, vlo = b ? vlo1 : vlo0;
                    if (nu == TILE_UNITS) {
                        if (PRECISE) {
                            ptx::mma_ts_pv8_warp<false>(tmem + TM_O, pb, vlo, vhi, idO, i == 0 ? 0u : 1u, 0u);
                            ptx::mma_ts_pv8_warp<true>(tmem + TM_O, pb + 16, vlo, vhi, idO, 1u, BAR(B_PV_DONE + b));     // the remainders of P
                        } else {
                            ptx::mma_ts_pv8_warp<true>(tmem + TM_O, pb, vlo, vhi, idO, i == 0 ? 0u : 1u, BAR(B_PV_DONE + b));
                        }
                    } else {
#pragma unroll
                        for (int u = 0; u < TILE_UNITS - 1; ++u)
                            if (u < nu) {
                                const uint64_t d0 = (uint64_t(vhi) << 32) | (vlo + 256u * u);
                                ptx::mma_ts_x2_warp(tmem + TM_O, pb + 32 * u, d0, d0 + 128, idO, (i == 0 && u == 0) ? 0u : 1u);
                                if (PRECISE) ptx::mma_ts_x2_warp(tmem + TM_O, pb + 32 * u + 16, d0, d0 + 128, idO, 1u);
                            }
                        ptx::mma_commit_warp(BAR(B_PV_DONE + b));
                    }
                }
                LLATTN_TR(26, t);
            }
            ++itc;
        }
        ptx::mma_commit_warp(BAR(B_SPARE + 1));
        {
            volatile int never = 0;
            if (!ptx::mbar_wait(BAR(B_SPARE + 1), 0, &never)) errbits |= ERR_WAIT_TEARDOWN;
        }
#endif
    }

    // ---- split tiles. Every run of this CTA is stored and counted by now, so nothing this CTA waits for depends on
    // this CTA: for each of its runs that is part of a split tile, wait (bounded) until all of the tile's runs are
    // counted in, then all sixteen warps finish this run's share of the rows, a warp per row. The last warp to leave a
    // tile puts both of its counters back to zero for the next launch. Every thread of the CTA walks this loop the same
    // way (same runs, same outcome), so the CTA barrier inside it is reached by all.
    if (p.merge != nullptr) {
        int nsplit = 0;
#pragma unroll 1
        for (int ii = i0_any; ii < i1_any; ++ii) {
            WorkItem w; SeqDesc sq;
            if (!fetch_item(p, ii, w, sq, first_run, i0_any)) continue;
            const MergeDesc md = p.merge[w.tile];
            if (md.nslots <= 1) continue;
            int* counters = p.tile_counters + 4 * w.tile;
            // one warp polls the counter for the whole CTA (hundreds of finished CTAs polling with every warp would load
            // the L2 the slower CTAs still stream through); the others learn the outcome through shared memory
            volatile int* outcome = reinterpret_cast<volatile int*>(smem + SM_MISC + 8) + (nsplit & 1);
            if (warp == 0) {
                const bool ok = wait_count(counters, SOFTMAX_WARPS * md.nslots, abort_flag, ptx::WAIT_LIMIT_NS);
                if (lane == 0) *outcome = ok;
            }
            __syncthreads();
            ++nsplit;
            if (!*outcome) {
                errbits |= ERR_WAIT_FOLD;
                *abort_flag = 1;
                break;
            }
            constexpr int NW = ATTN_THREADS / 32;
            const int r0 = (w.slot - md.slot_begin) + md.nslots * warp, step = md.nslots * NW;
            if (md.nslots == 2) {
#pragma unroll 1
                for (int r = r0; r < QR; r += 4 * step) {
                    const int rows[4] = {r, r + step < QR ? r + step : -1, r + 2 * step < QR ? r + 2 * step : -1, r + 3 * step < QR ? r + 3 * step : -1};
                    fold_rows_few<4, 2>(p.Opart, p.Mpart, p.Lpart, md, rows, lane, p.out);
                }
            } else if (md.nslots <= 4) {
#pragma unroll 1
                for (int r = r0; r < QR; r += 2 * step) {
                    const int rows[2] = {r, r + step < QR ? r + step : -1};
                    fold_rows_few<2, 4>(p.Opart, p.Mpart, p.Lpart, md, rows, lane, p.out);
                }
            } else {
#pragma unroll 1
                for (int r = r0; r < QR; r += step) fold_row_warp(p.Opart, p.Mpart, p.Lpart, md, r, lane, p.out);
            }
            __syncwarp();
            if (lane == 0 && atomicAdd(counters + 1, 1) == (ATTN_THREADS / 32) * md.nslots - 1) { counters[0] = 0; counters[1] = 0; }
        }
    }

    if (errbits && p.err) atomicOr(p.err, errbits);
    ptx::tc_fence_before();
    __syncthreads();
    if (warp == WARP_MMA) ptx::tmem_dealloc(tmem, TMEM_COLS);
}

template <bool PRECISE>
__global__ void __launch_bounds__(ATTN_THREADS, 1) attn_tile_kernel(const __grid_constant__ KParams p) {
    attn_tile_body<PRECISE>(p, blockIdx.x);
}

}  // namespace llattn
