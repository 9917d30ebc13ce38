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
//   softmax warps : one thread per query row (TMEM lane); row max, lazy rescale (the reference maximum moves only
//                   when exceeded by more than 8 in log2 units, engine/attn.cu:237-255), p = 2^(s*scale*log2e - m),
//                   P stored back over S in TMEM as fp16 pairs (the 32 keys of chunk g at columns 32 g .. 32 g + 15, the
//                   first half of the S columns they were computed from: a softmax warp overwrites only S columns it
//                   has itself consumed)
// The run's un-normalised O (fp32), reference maximum (log2 units) and row sum go to a partial slot in the format of
// the reference's Opart/Mpart/Lpart (engine/attn.cu:291-305); merge_kernel.cuh folds the slots of a tile together.
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

namespace llattn {

// Timeline hooks for kernel tuning: compiled out unless LLATTN_TRACE is defined (the shipped library never defines it).
#ifdef LLATTN_TRACE
__device__ unsigned long long* g_trace_buf;      // [warps][LLATTN_TRACE_EVENTS] of (clock << 24 | tile << 8 | event)
constexpr int LLATTN_TRACE_EVENTS = 2048;
#define LLATTN_TR(ev, tile)                                                                                    \
    do {                                                                                                       \
        if (trace_ptr && trace_n < LLATTN_TRACE_EVENTS)                                                        \
            trace_ptr[trace_n++] =                                 \
                (static_cast<unsigned long long>(clock64()) << 24) | (static_cast<unsigned long long>((tile) & 0xffff) << 8) | (ev); \
    } while (0)
#else
#define LLATTN_TR(ev, tile) do {} while (0)
#endif
#ifndef LLATTN_SKIP
#define LLATTN_SKIP 0      // tuning builds only: bit 0 = no dequantisation, bit 1 = no softmax arithmetic (results are garbage)
#endif

constexpr int TILE_UNITS = 4;
constexpr int KBLOCK = 128 * 128;                  // 16384: 128 keys x 64 channels of fp16, one swizzled block
constexpr int TILE_BYTES = 2 * KBLOCK;             // K tile: channels 0-63, 64-127
constexpr int VTILE_BYTES = 3 * KBLOCK;            // V tile: dims 0-63, 64-127, then the block with the ones column
constexpr int UNIT_BYTES = 32 * 128;               // a unit's 32 keys inside a block
constexpr int PV_N = 144;                          // dims 0..127, column 128 = row sum, 129..143 unused
constexpr int NRAW = 8;                            // records in flight (two tiles' worth)
constexpr int RAW_STRIDE = 4864;                   // 4736 rounded up to a multiple of 128
constexpr int SM_K = 0;                            // two K tiles (every tile base is 1024-byte aligned)
constexpr int SM_V = SM_K + 2 * TILE_BYTES;        // two V tiles
constexpr int SM_RAW = SM_V + 2 * VTILE_BYTES;
constexpr int SM_BAR = SM_RAW + NRAW * RAW_STRIDE;
constexpr int SM_X = SM_BAR + 512;                 // row-max exchange between the two softmax warps of a lane quarter
constexpr int SM_MISC = SM_X + 2 * 4 * 128 * 4;
constexpr int ATTN_SMEM_BYTES = SM_MISC + 16;
// warps 0-7 softmax (warp w: TMEM lane quarter w % 4, key half w / 4), 8-15 dequant (four groups of two warps, group g
// takes unit g of every tile: a thread's scale / minimum words then serve eight passes over the record instead of four),
// then PV-MMA issue, S-MMA issue and two producers. The warp counts are the measured
// optimum: the kernel is bound by instruction issue, every warp pays a fixed number of hand-off instructions per tile,
// so fewer, busier dequantising warps win (16 of them: +4 % time), while a single group or four softmax warps leave too
// little latency hiding (+40 % / +12 %) and sixteen softmax warps pay too many hand-offs (+8 %).
#ifndef LLATTN_DEQUANT_WARPS
#define LLATTN_DEQUANT_WARPS 8
#endif
#ifndef LLATTN_GROUP_WARPS
#define LLATTN_GROUP_WARPS 2
#endif
#ifndef LLATTN_SOFTMAX_WARPS
#define LLATTN_SOFTMAX_WARPS 8
#endif
constexpr int SOFTMAX_WARPS = LLATTN_SOFTMAX_WARPS, KEY_PARTS = SOFTMAX_WARPS / 4, DEQUANT_WARPS = LLATTN_DEQUANT_WARPS, GROUP_WARPS = LLATTN_GROUP_WARPS, DEQUANT_GROUPS = DEQUANT_WARPS / GROUP_WARPS;
constexpr int GROUP_THREADS = 32 * GROUP_WARPS, DQ_PASSES = 16 / GROUP_WARPS;      // a group converts one record: 32 keys, two per warp and pass
constexpr int WARP_SERVICE = SOFTMAX_WARPS + DEQUANT_WARPS;
// Service warps, one per scheduler (a warp runs on scheduler warp % 4 and the softmax warps cannot move): PV issue, S
// issue and two copy producers that take alternate records, so that no scheduler carries much more than the others.
constexpr int WARP_MMA_PV = WARP_SERVICE, WARP_MMA = WARP_SERVICE + 1, WARP_PRODUCER = WARP_SERVICE + 2, PRODUCERS = 2;
constexpr int ATTN_THREADS = 32 * (WARP_SERVICE + 2 + PRODUCERS);  // 640
constexpr int TMEM_COLS = 512;
constexpr int TM_S = 0, TM_O = 256, TM_L = TM_O + 128, TM_Q = 400;   // S at columns 0 and 128, O at 256..383, row sum at 384, Q at 400..463
constexpr float RESCALE_SLACK = 8.f;

// barrier indices
enum { B_RAW_FULL = 0, B_RAW_EMPTY = B_RAW_FULL + NRAW, B_K_FULL = B_RAW_EMPTY + NRAW, B_V_FULL = B_K_FULL + 2,
       B_K_FREE = B_V_FULL + 2, B_PV_DONE = B_K_FREE + 2, B_S_FULL = B_PV_DONE + 2, B_P_FULL = B_S_FULL + 2,
       B_Q_FULL = B_P_FULL + 2, B_O_FREE, B_SPARE, B_XCHG = B_SPARE + 2, B_COUNT = B_XCHG + 4 };
static_assert(B_COUNT * 8 <= 512, "barrier area");
static_assert(ATTN_SMEM_BYTES <= 232448, "shared memory budget");
static_assert(SOFTMAX_WARPS == 4 || SOFTMAX_WARPS == 8 || SOFTMAX_WARPS == 16, "softmax warps: 1, 2 or 4 per TMEM lane quarter");
static_assert((GROUP_WARPS == 2 || GROUP_WARPS == 4) && DEQUANT_WARPS % GROUP_WARPS == 0 && DEQUANT_GROUPS >= 1 && TILE_UNITS % DEQUANT_GROUPS == 0,
              "dequant warps: groups of two or four, 1, 2 or 4 groups");

struct KParams {
    const SeqDesc* seqs;           // list mode
    const WorkItem* items;
    const int32_t* cta_first;      // [gridDim.x + 1]
    const half* Q;
    const half* Kf;
    const half* Vf;
    float* Opart;
    float* Mpart;
    float* Lpart;
    float sl2;                     // softmax scale * log2(e)
    int* err;
    // reference-grid mode (items == nullptr): CTA i is (kvh = i % 4, chunk = (i / 4) % ref_nchunks, jb = i / (4 * ref_nchunks))
    SeqDesc ref_seq;
    int ref_bpc;
    int ref_nchunks;
};

__device__ __forceinline__ bool fetch_item(const KParams& p, int idx, WorkItem& w, SeqDesc& s) {
    if (p.items) {
        w = p.items[idx];
        s = p.seqs[w.seq];
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
    w.pad = 0;
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
#pragma unroll
    for (int p = 0; p < DQ_PASSES; ++p) {
        half2 kh[4];
        unpack8(*reinterpret_cast<const uint32_t*>(raw + d.k_src + p * 128 * GROUP_WARPS), kh);
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
#pragma unroll
    for (int p = 0; p < DQ_PASSES; ++p) {
        const uint32_t vsu = __byte_perm(sw[p], sw[p], d.hsel), vmu = __byte_perm(mw[p], mw[p], d.hsel);
        const half2 vs = *reinterpret_cast<const half2*>(&vsu), vm = *reinterpret_cast<const half2*>(&vmu);
        half2 vh[4];
        unpack8(*reinterpret_cast<const uint32_t*>(raw + d.v_src + p * 128), vh);
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
            ptx::mbar_init(BAR(B_S_FULL + i), 1); ptx::mbar_init(BAR(B_P_FULL + i), 32 * SOFTMAX_WARPS);
        }
        ptx::mbar_init(BAR(B_Q_FULL), 32 * SOFTMAX_WARPS); ptx::mbar_init(BAR(B_O_FREE), 32 * SOFTMAX_WARPS);
        ptx::mbar_init(BAR(B_SPARE), 1);
        ptx::mbar_init(BAR(B_SPARE + 1), 1);
        for (int i = 0; i < 4; ++i) ptx::mbar_init(BAR(B_XCHG + i), 32 * KEY_PARTS);
        ptx::fence_mbar_init();
        *abort_flag = 0;
    }
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
        // thread = (query row, key part): the KEY_PARTS warps of a TMEM lane quarter split a tile's four 32-key chunks
        // (chunk g = S columns [32 g, 32 g + 32); its P goes to the first 16 of the same columns, so a warp only ever
        // overwrites S it has itself consumed), the channels of Q and the columns of O
        constexpr int CPW = 4 / KEY_PARTS;            // chunks per warp and tile = 32-column groups of O per warp
        const int q = warp & 3, kp = warp >> 2, row = q * 32 + lane;
        const uint32_t tlane = tmem + (uint32_t(q * 32) << 16);
        float* xb = reinterpret_cast<float*>(smem + SM_X);
        uint32_t t = 0;
        bool alive = true;
#pragma unroll 1
        for (int ii = i0; ii < i1 && alive; ++ii) {
            WorkItem w; SeqDesc s;
            if (!fetch_item(p, ii, w, s)) continue;
            const int U = w.rec_count + w.fresh, ntiles = (U + TILE_UNITS - 1) / TILE_UNITS;
            float mref = -INFINITY;
            {   // this thread's query row, channels [32 CPW kp, 32 CPW (kp + 1)), into tensor memory as fp16 pairs. Every S
                // MMA of the previous item has completed: this warp has seen the S of its last tile.
                const half* src = p.Q + ((size_t(s.q_first + w.qblk) * BLK + (row >> 2)) * NQH + 4 * w.kvh + (row & 3)) * D + 32 * CPW * kp;
#pragma unroll 1
                for (int c = 0; c < CPW; ++c) {
                    uint32_t r[16];
#pragma unroll
                    for (int g = 0; g < 4; ++g) {
                        const uint4 v = permute8(__ldg(reinterpret_cast<const uint4*>(src + 32 * c + 8 * g)));
                        r[4 * g] = v.x; r[4 * g + 1] = v.y; r[4 * g + 2] = v.z; r[4 * g + 3] = v.w;
                    }
                    ptx::tmem_st16(tlane + TM_Q + 16 * (CPW * kp + c), r);
                }
                ptx::tmem_wait_st();
                ptx::tc_fence_before();
                ptx::mbar_arrive(BAR(B_Q_FULL));
            }
#pragma unroll 1
            for (int i = 0; i < ntiles; ++i, ++t) {
                const int b = t & 1, nu = min(TILE_UNITS, U - TILE_UNITS * i);
                const int nc = max(0, min(CPW, nu - CPW * kp));          // 32-key chunks of this tile this warp owns
                LLATTN_TR(1, t);
                if (!ptx::mbar_wait(BAR(B_S_FULL + b), (t >> 1) & 1, abort_flag)) { alive = false; errbits |= ERR_WAIT_SOFTMAX; break; }
                LLATTN_TR(2, t);
                ptx::tc_fence_after();
                const uint32_t ts = tlane + TM_S + b * 128 + 32 * CPW * kp;
                float mx = -INFINITY;
#pragma unroll 1
                for (int c = 0; c < nc; ++c) {
                    uint32_t r[32];
                    ptx::tmem_ld32(ts + 32 * c, r);
                    ptx::tmem_wait_ld();
#pragma unroll
                    for (int j = 0; j < 32; j += 2) {
                        if (LLATTN_SKIP & 2) { if (j == 0) mx = fmaxf(mx, __uint_as_float(r[0])); }
                        else mx = max3(mx, __uint_as_float(r[j]), __uint_as_float(r[j + 1]));
                    }
                }
                // row max over all parts: exchange through shared memory with the other warps of the lane quarter
                // (double-buffered by tile parity; the quarter's mbarrier, one phase per tile, orders write -> read and
                // its wait is bounded)
                LLATTN_TR(5, t);
                if (KEY_PARTS > 1) {
                    xb[b * 512 + kp * 128 + row] = mx;
                    ptx::mbar_arrive(BAR(B_XCHG + q));
                    if (!ptx::mbar_wait(BAR(B_XCHG + q), t & 1, abort_flag)) { alive = false; errbits |= ERR_WAIT_SOFTMAX; break; }
#pragma unroll
                    for (int k = 1; k < KEY_PARTS; ++k) mx = fmaxf(mx, xb[b * 512 + ((kp + k) % KEY_PARTS) * 128 + row]);
                }
                LLATTN_TR(3, t);
                const float msc = mx * p.sl2;
                const bool moved = msc > mref + RESCALE_SLACK;
                if (i > 0 && __any_sync(0xffffffffu, moved)) {
                    // the accumulated O of these rows is rescaled to the new reference maximum (this warp's share of the
                    // columns); every PV issued so far must have landed first
                    if (!ptx::mbar_wait(BAR(B_PV_DONE + (b ^ 1)), ((t - 1) >> 1) & 1, abort_flag)) { alive = false; errbits |= ERR_WAIT_SOFTMAX; break; }
                    ptx::tc_fence_after();
                    const float corr = moved ? ex2(mref - msc) : 1.f;
#pragma unroll 1
                    for (int c = 0; c < CPW; ++c) {
                        uint32_t r[32];
                        ptx::tmem_ld32(tlane + TM_O + 32 * (CPW * kp + c), r);
                        ptx::tmem_wait_ld();
#pragma unroll
                        for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) * corr);
                        ptx::tmem_st32(tlane + TM_O + 32 * (CPW * kp + c), r);
                    }
                    if (kp == KEY_PARTS - 1) {
                        uint32_t r[16];
                        ptx::tmem_ld16(tlane + TM_L, r);
                        ptx::tmem_wait_ld();
                        r[0] = __float_as_uint(__uint_as_float(r[0]) * corr);
                        ptx::tmem_st16(tlane + TM_L, r);
                    }
                    ptx::tmem_wait_st();
                }
                if (moved) mref = msc;
                const unsigned long long sl2x2 = dup2(p.sl2), nmx2 = dup2(-mref);
#pragma unroll 1
                for (int c = 0; c < nc; ++c) {
                    uint32_t r[32], pk[16];
                    ptx::tmem_ld32(ts + 32 * c, r);
                    ptx::tmem_wait_ld();
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        if (LLATTN_SKIP & 2) { pk[j] = r[2 * j] & 0x03ff03ffu; continue; }
                        float x0, x1;
                        fma2(r[2 * j], r[2 * j + 1], sl2x2, nmx2, x0, x1);
                        const half2 h = __floats2half2_rn(ex2(x0), ex2(x1));
                        pk[j] = *reinterpret_cast<const uint32_t*>(&h);
                    }
                    ptx::tmem_st16(ts + 32 * c, pk);      // P chunk over the S columns it was computed from
                }
                ptx::tmem_wait_st();
                ptx::tc_fence_before();
                ptx::mbar_arrive(BAR(B_P_FULL + b));
                LLATTN_TR(4, t);
            }
            if (!alive) break;
            // ---- epilogue: un-normalised O (this warp's share of the columns), reference maximum and row sum of the run
            const uint32_t tl = t - 1;
            if (!ptx::mbar_wait(BAR(B_PV_DONE + (tl & 1)), (tl >> 1) & 1, abort_flag)) { alive = false; errbits |= ERR_WAIT_SOFTMAX; break; }
            ptx::tc_fence_after();
            float* orow = p.Opart + (size_t(w.slot) * QR + row) * D + 32 * CPW * kp;
#pragma unroll 1
            for (int c = 0; c < CPW; ++c) {
                uint32_t r[32];
                ptx::tmem_ld32(tlane + TM_O + 32 * (CPW * kp + c), r);
                ptx::tmem_wait_ld();
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
            if (kp == KEY_PARTS - 1) {
                uint32_t r[16];
                ptx::tmem_ld16(tlane + TM_L, r);
                ptx::tmem_wait_ld();
                p.Lpart[size_t(w.slot) * QR + row] = __uint_as_float(r[0]);
            }
            if (kp == 0) p.Mpart[size_t(w.slot) * QR + row] = mref;
            ptx::tc_fence_before();
            ptx::mbar_arrive(BAR(B_O_FREE));
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
            if (!fetch_item(p, ii, w, s)) continue;
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
            if (!fetch_item(p, ii, w, s)) continue;
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
        // ================================================================== S = Q K^T issue (one elected lane issues, the warp stays together)
        // Two issuing warps (this one and the PV one below) halve the per-tile instruction chain on the critical path.
        // Loop bounds, tile counts and wait results are made visibly warp-uniform so that the operands of the MMAs can
        // live in uniform registers.
        uint32_t t = 0, itc = 0;
        bool alive = true;
        // one base descriptor per K buffer (K-major, 128-byte swizzle, 8-row groups 1024 B apart); the issue helper steps it
        const uint32_t k_s = ptx::smem_u32(smem + SM_K);
        const uint32_t klo0 = ptx::desc_lo(k_s, 16), klo1 = ptx::desc_lo(k_s + TILE_BYTES, 16), khi = ptx::desc_hi(1024) | (2u << 29);
        const uint32_t tmem = uniform_u32(tmem_any);
        const int i0 = uniform_i32(i0_any), i1 = uniform_i32(i1_any);
#pragma unroll 1
        for (int ii = i0; ii < i1 && alive; ++ii) {
            WorkItem w; SeqDesc s;
            if (!uniform_i32(fetch_item(p, ii, w, s))) continue;
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
        // every MMA issued must have retired before tensor memory is released
        ptx::mma_commit_warp(BAR(B_SPARE));
        {
            volatile int never = 0;
            if (!ptx::mbar_wait(BAR(B_SPARE), 0, &never)) errbits |= ERR_WAIT_TEARDOWN;
        }
    } else {
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
            if (!uniform_i32(fetch_item(p, ii, w, s))) continue;
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
                        ptx::mma_ts_pv8_warp(tmem + TM_O, pb, vlo, vhi, idO, i == 0 ? 0u : 1u, BAR(B_PV_DONE + b));
                    } else {
#pragma unroll
                        for (int u = 0; u < TILE_UNITS - 1; ++u)
                            if (u < nu) {
                                const uint64_t d0 = (uint64_t(vhi) << 32) | (vlo + 256u * u);
                                ptx::mma_ts_x2_warp(tmem + TM_O, pb + 32 * u, d0, d0 + 128, idO, (i == 0 && u == 0) ? 0u : 1u);
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
    }

    if (errbits && p.err) atomicOr(p.err, errbits);
    ptx::tc_fence_before();
    __syncthreads();
    if (warp == WARP_MMA) ptx::tmem_dealloc(tmem, TMEM_COLS);
}

__global__ void __launch_bounds__(ATTN_THREADS, 1) attn_tile_kernel(const __grid_constant__ KParams p) {
    attn_tile_body(p, blockIdx.x);
}

}  // namespace llattn
