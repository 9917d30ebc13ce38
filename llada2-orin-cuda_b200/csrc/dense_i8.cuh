// Dense W4.A8 projection with residual add on tcgen05 tensor cores (kind::i8: u8 x s8 -> s32 in tensor memory).
//
// It consumes the int8 activations the merge kernel writes (values in fragment order inside every 128-group, one fp32
// scale and one int32 sum per token and group) and the reference's 4-bit weight strips as the engine holds them on the
// device, and computes what the reference's attention-output projection computes (engine/engine.cu:434,
// moe8::gemm<.., MODE 2>, engine/moe_i8.cu:295-400), for any number of tokens:
//     Y[n][r] += sum over 128-groups g, in order, of  (s_w[r][g] * s_x[n][g]) * float(P[r][n][g] - z[r][g] * Sxq[n][g])
// with P the exact integer dot product of the group. Every float operation is the reference's (one fp32 product of
// the two scales, one fused multiply-add per group, groups in ascending order, one add into Y), so results are
// bit-identical to the reference kernel.
//
// Weight strip (16 rows x K), device layout of the reference (engine/moe_i8.cu:34-41): the 1024-byte code tiles of
// the strip's K/128 groups, then their 48-byte metas. In a code tile lane l = 4 g + t of the reference's warp owns
// bytes 16 l .. 16 l + 15 and 512 + 16 l ..: eight words; word w (step j = w / 2, half h = w % 2) holds, for k = 32 j +
// 16 h + 4 t + e (e = byte index), the code of row g in the low nibble and of row g + 8 in the high nibble
// (engine/moe_i8.cu:127-160). A meta holds fp16 scale pairs (rows g | g + 8) at 4 g and zero-point pairs at 32 + 2 g.
//
// One CTA computes 128 weight rows x 64 tokens. Per 128-group: 128 threads unpack the eight strips' codes into a u8
// operand tile and copy the tokens' int8 rows (both K-major, 128-byte swizzle; the weights are stored at the
// activations' fragment positions, so the activations are copied as they are), a fifth warp issues four K = 32 MMAs
// into one of two 64-column accumulators, and the 128 threads (thread = weight row = tensor-memory lane) fold the
// previous group's integers into 64 fp32 accumulators while the next group's MMAs run.
#pragma once
#include <cuda_fp16.h>
#include "common.cuh"
#include "ptx.cuh"

namespace llattn {

constexpr int DN_ROWS = 128, DN_TOK = 64, DN_GROUP = 128;
constexpr int DN_TILE_BYTES = 1024, DN_META_BYTES = 48;
constexpr int DN_STAGES = 3;                                      // slots for data coming from global memory
constexpr int DN_A_BYTES = DN_ROWS * 128, DN_B_BYTES = DN_TOK * 128, DN_RAW_BYTES = 8 * DN_TILE_BYTES;
constexpr int DN_SM_A = 0;                                        // two unpacked weight tiles
constexpr int DN_SM_B = DN_SM_A + 2 * DN_A_BYTES;                 // DN_STAGES activation tiles, written by cp.async
constexpr int DN_SM_RAW = DN_SM_B + DN_STAGES * DN_B_BYTES;       // eight code tiles as they lie in memory (every thread copies and
                                                                  // unpacks its own 64 bytes, so one slot is enough)
// Token scales and sums are read by the folding threads themselves; a thread may be one group ahead of the slowest one
// when it refills a slot, so these have twice as many slots as there are stages.
constexpr int DN_SM_SX = DN_SM_RAW + DN_RAW_BYTES;                // [8][64] float token scales
constexpr int DN_SM_SQ = DN_SM_SX + 8 * DN_TOK * 4;               // [8][64] int token sums
constexpr int DN_SM_BAR = DN_SM_SQ + 8 * DN_TOK * 4;
constexpr int DN_SMEM_BYTES = DN_SM_BAR + 64;
constexpr int DN_THREADS = 160;
enum { DB_FULL = 0, DB_DONE = 2, DB_COUNT = 4 };

struct DenseParams {
    const uint8_t* W;      // strips
    const int8_t* q;       // [ntokens][K], fragment order inside every 128-group
    const float* s;        // [ntokens][K / 128]
    const int32_t* sum;    // [ntokens][K / 128]
    float* Y;              // [ntokens][rows], accumulated into
    int ntokens, rows, K;
    int* err;
};

__device__ __forceinline__ void mma_i8_ss(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}\n"
                 :: "r"(d), "l"(a), "l"(b), "r"(idesc), "r"(accumulate) : "memory");
}
// 16-byte and 4-byte asynchronous copies global -> shared (per-thread completion groups); `live` false writes zeros.
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool live) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(live ? 16 : 0) : "memory");
}
__device__ __forceinline__ void cp_async4(uint32_t dst, const void* src, bool live) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(dst), "l"(src), "r"(live ? 4 : 0) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int kPending> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(kPending) : "memory"); }

// kind::i8 instruction descriptor: s32 accumulator, A u8 (format 0), B s8 (format 1), both K-major.
__host__ __device__ constexpr uint32_t idesc_i8_u8s8(int M, int N) {
    return (2u << 4) | (0u << 7) | (1u << 10) | (uint32_t(N >> 3) << 17) | (uint32_t(M >> 4) << 24);
}

__global__ void __launch_bounds__(DN_THREADS) dense_i8_kernel(const DenseParams p) {
    extern __shared__ __align__(1024) uint8_t smem[];
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_flag_s;
    volatile int* abort_flag = &abort_flag_s;
    const int tid = threadIdx.x, warp = tid >> 5;
    const int row0 = blockIdx.x * DN_ROWS, n0 = blockIdx.y * DN_TOK;
    const int ktot = p.K / DN_GROUP;
    const uint32_t bar0 = ptx::smem_u32(smem + DN_SM_BAR);
    auto BAR = [&](int i) -> uint32_t { return bar0 + 8u * uint32_t(i); };
    if (ptx::smem_u32(smem) & 1023u) {
        if (tid == 0 && p.err) atomicOr(p.err, ERR_SMEM_ALIGN);
        return;
    }
    if (tid == 0) {
        for (int i = 0; i < 2; ++i) { ptx::mbar_init(BAR(DB_FULL + i), 128); ptx::mbar_init(BAR(DB_DONE + i), 1); }
        ptx::fence_mbar_init();
        abort_flag_s = 0;
    }
    if (warp == 4) { ptx::tmem_alloc(ptx::smem_u32(&tmem_slot), 128); ptx::tmem_relinquish(); }
    ptx::tc_fence_before();
    __syncthreads();
    ptx::tc_fence_after();
    const uint32_t tmem = tmem_slot;
    const size_t strip_bytes = size_t(ktot) * (DN_TILE_BYTES + DN_META_BYTES), meta_off = size_t(ktot) * DN_TILE_BYTES;
    int errbits = 0;

    if (warp < 4) {
        // ---- this thread's weight row: strip, row inside the strip, where its scale and zero point sit in a meta
        const int r = tid, strip = (row0 + r) >> 4, rr = r & 15, g8 = rr & 7, hi = rr >> 3;
        const uint8_t* my_meta = p.W + size_t(strip) * strip_bytes + meta_off + 4 * g8 + 2 * hi;
        const uint8_t* my_zero = p.W + size_t(strip) * strip_bytes + meta_off + 32 + 2 * g8 + hi;
        // what this thread brings in and stages per group: two (strip, reference lane) tasks of weight codes - it unpacks
        // exactly the bytes it copied itself - and half a token's 128-byte row, copied straight into the operand tile
        const int sl0 = tid >> 5, l = tid & 31, g = l >> 2, t = l & 3;       // task 0: strip sl0, task 1: strip sl0 + 4
        const uint8_t* code0 = p.W + size_t((row0 >> 4) + sl0) * strip_bytes + 16 * l;
        const uint8_t* code1 = code0 + 4 * strip_bytes;
        const int tn = tid >> 1, hf = tid & 1;
        const bool tlive = n0 + tn < p.ntokens;
        const int8_t* arow = p.q + size_t(tlive ? n0 + tn : 0) * p.K + 64 * hf;
        const bool slive = tid < DN_TOK && n0 + tid < p.ntokens;
        const size_t srow = size_t(slive ? n0 + tid : 0) * ktot;
        const uint32_t sm0 = ptx::smem_u32(smem);
        const uint32_t raw_mine = sm0 + DN_SM_RAW + 64 * tid;             // 4 x 16 bytes per stage
        const uint32_t b_mine = sm0 + DN_SM_B + tn * 128;
        auto fetch = [&](int i) {          // asynchronous copies of group i (always one commit, so groups count uniformly)
            if (i < ktot) {
                const int sg = i % DN_STAGES;
                const size_t co = size_t(i) * DN_TILE_BYTES;
                cp_async16(raw_mine, code0 + co, true);
                cp_async16(raw_mine + 16, code0 + co + 512, true);
                cp_async16(raw_mine + 32, code1 + co, true);
                cp_async16(raw_mine + 48, code1 + co + 512, true);
                const int8_t* src = arow + size_t(i) * DN_GROUP;
#pragma unroll
                for (int k = 0; k < 4; ++k)
                    cp_async16(b_mine + sg * DN_B_BYTES + (((4 * hf + k) ^ (tn & 7)) << 4), src + 16 * k, tlive);
                if (tid < DN_TOK) {
                    cp_async4(sm0 + DN_SM_SX + ((i & 7) * DN_TOK + tid) * 4, p.s + srow + i, slive);
                    cp_async4(sm0 + DN_SM_SQ + ((i & 7) * DN_TOK + tid) * 4, p.sum + srow + i, slive);
                }
            }
            cp_async_commit();
        };
        float c[DN_TOK];
#pragma unroll
        for (int n = 0; n < DN_TOK; ++n) c[n] = 0.f;
        const bool second_half = p.ntokens - n0 > 32;
        bool alive = true;
        uint16_t sw_next = 0;
        int z_next = 0;
        fetch(0);
#pragma unroll 1
        for (int i = 0; i <= ktot && alive; ++i) {
            // scale and zero point of the group folded in this iteration (loaded one iteration ago, behind the proxy fence:
            // a fence with loads in flight waits for them)
            const uint16_t sw_bits = sw_next;
            const int z = z_next;
            if (i < ktot) {
                const int st = i & 1;
                // group i has landed (this thread's copies; nothing else is in flight: a proxy fence with copies in flight
                // would wait for them). The A tile's previous MMAs (group i - 2) were seen complete when this thread folded
                // that group.
                cp_async_wait<0>();
                uint8_t* As = smem + DN_SM_A + st * DN_A_BYTES;
                const uint4* raw = reinterpret_cast<const uint4*>(smem + DN_SM_RAW + 64 * tid);
                // weights: each task yields 8 words for row g of its strip and 8 for row g + 8, stored at the codes'
                // fragment positions
#pragma unroll
                for (int task = 0; task < 2; ++task) {
                    const uint4 lo = raw[2 * task], h4 = raw[2 * task + 1];
                    const uint32_t w[8] = {lo.x, lo.y, lo.z, lo.w, h4.x, h4.y, h4.z, h4.w};
                    const int ra = (sl0 + 4 * task) * 16 + g, rb = ra + 8;            // rows inside the CTA tile
                    // word k holds the codes at fragment positions 32 t + 8 (k / 2) + 4 (k % 2): words 0-3 are the 16-byte chunk
                    // 2 t of the row, words 4-7 chunk 2 t + 1. Two 16-byte stores per row; a quarter warp covers eight
                    // different chunk positions, so they are conflict-free.
                    const uint32_t m = 0x0F0F0F0Fu;
                    *reinterpret_cast<uint4*>(As + ra * 128 + (((2 * t) ^ (ra & 7)) << 4)) = make_uint4(w[0] & m, w[1] & m, w[2] & m, w[3] & m);
                    *reinterpret_cast<uint4*>(As + ra * 128 + (((2 * t + 1) ^ (ra & 7)) << 4)) = make_uint4(w[4] & m, w[5] & m, w[6] & m, w[7] & m);
                    *reinterpret_cast<uint4*>(As + rb * 128 + (((2 * t) ^ (rb & 7)) << 4)) =
                        make_uint4((w[0] >> 4) & m, (w[1] >> 4) & m, (w[2] >> 4) & m, (w[3] >> 4) & m);
                    *reinterpret_cast<uint4*>(As + rb * 128 + (((2 * t + 1) ^ (rb & 7)) << 4)) =
                        make_uint4((w[4] >> 4) & m, (w[5] >> 4) & m, (w[6] >> 4) & m, (w[7] >> 4) & m);
                }
                ptx::fence_proxy_async_smem();         // the A tile, and the activation tile the copies wrote, for the tensor core
                ptx::mbar_arrive(BAR(DB_FULL + st));
                // group i + 1 comes in while group i - 1 is folded; its slots were last read by the MMAs of group i - 2
                fetch(i + 1);
                sw_next = __ldg(reinterpret_cast<const uint16_t*>(my_meta + size_t(i) * DN_META_BYTES));
                z_next = int(__ldg(my_zero + size_t(i) * DN_META_BYTES));
            }
            if (i >= 1) {
                // ---- fold group i - 1: its integers are complete in accumulator (i - 1) % 2. The token scales were
                // written by other threads' copies: their arrivals on db_full order them before this read.
                const int gi = i - 1, st = gi & 1;
                if (!ptx::mbar_wait(BAR(DB_FULL + st), (gi >> 1) & 1, abort_flag)) { alive = false; errbits |= ERR_WAIT_DEQUANT; break; }
                if (!ptx::mbar_wait(BAR(DB_DONE + st), (gi >> 1) & 1, abort_flag)) { alive = false; errbits |= ERR_WAIT_DEQUANT; break; }
                ptx::tc_fence_after();
                const float sw = __half2float(__ushort_as_half(sw_bits));
                const float* sx = reinterpret_cast<const float*>(smem + DN_SM_SX) + (gi & 7) * DN_TOK;
                const int* sq = reinterpret_cast<const int*>(smem + DN_SM_SQ) + (gi & 7) * DN_TOK;
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    if (h == 1 && !second_half) break;       // a tile with at most 32 live tokens (the reference's decode shape)
                    uint32_t d[32];
                    ptx::tmem_ld32(tmem + (uint32_t(warp * 32) << 16) + st * DN_TOK + 32 * h, d);
                    ptx::tmem_wait_ld();
#pragma unroll
                    for (int n4 = 0; n4 < 32; n4 += 4) {
                        const float4 sx4 = *reinterpret_cast<const float4*>(sx + 32 * h + n4);      // broadcast 16-byte loads
                        const int4 sq4 = *reinterpret_cast<const int4*>(sq + 32 * h + n4);
                        const float sxv[4] = {sx4.x, sx4.y, sx4.z, sx4.w};
                        const int sqv[4] = {sq4.x, sq4.y, sq4.z, sq4.w};
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            // int -> float through the float whose bits are 1.5 * 2^23 + v: exact for |v| < 2^22 (here
                            // |v| <= 255 * 127 * 128), integer adds and one float subtract at full rate
                            const int n = n4 + e;
                            const int v = int(d[n]) - z * sqv[e];
                            const float vf = __int_as_float(v + 0x4B400000) - 12582912.0f;
                            c[32 * h + n] = __fmaf_rn(__fmul_rn(sw, sxv[e]), vf, c[32 * h + n]);
                        }
                    }
                }
                ptx::tc_fence_before();
            }
        }
        cp_async_wait<0>();
        if (alive) {
            // Y += c, sixteen tokens at a time: all loads of a batch are issued before the first add, so the round trips
            // to memory overlap instead of queueing behind one another (one coalesced 128-byte line per warp and token)
            float* ybase = p.Y + size_t(n0) * p.rows + row0 + r;
#pragma unroll
            for (int nb = 0; nb < DN_TOK; nb += 16) {
                float y[16];
#pragma unroll
                for (int j = 0; j < 16; ++j) y[j] = n0 + nb + j < p.ntokens ? __ldcg(ybase + size_t(nb + j) * p.rows) : 0.f;
#pragma unroll
                for (int j = 0; j < 16; ++j)
                    if (n0 + nb + j < p.ntokens) __stcg(ybase + size_t(nb + j) * p.rows, y[j] + c[nb + j]);
            }
        }
    } else {
        // ---- MMA issue: group i = four K-steps of 32 into accumulator i % 2, overwriting it
        const uint32_t id = idesc_i8_u8s8(DN_ROWS, DN_TOK);
        bool alive = true;
#pragma unroll 1
        for (int i = 0; i < ktot && alive; ++i) {
            const int st = i & 1;
            if (!ptx::mbar_wait(BAR(DB_FULL + st), (i >> 1) & 1, abort_flag)) { alive = false; errbits |= ERR_WAIT_MMA; break; }
            ptx::tc_fence_after();
            if (ptx::elect_one()) {
                const uint32_t a_s = ptx::smem_u32(smem + DN_SM_A + st * DN_A_BYTES);
                const uint32_t b_s = ptx::smem_u32(smem + DN_SM_B + (i % DN_STAGES) * DN_B_BYTES);
#pragma unroll
                for (int k = 0; k < 4; ++k)
                    mma_i8_ss(tmem + st * DN_TOK, ptx::smem_desc_sw128(a_s + 32 * k, 16, 1024), ptx::smem_desc_sw128(b_s + 32 * k, 16, 1024), id, k > 0);
                ptx::mma_commit(BAR(DB_DONE + st));
            }
            __syncwarp();
        }
    }
    if (errbits && p.err) atomicOr(p.err, errbits);
    ptx::tc_fence_before();
    __syncthreads();
    if (warp == 4) ptx::tmem_dealloc(tmem, 128);
}

}  // namespace llattn
