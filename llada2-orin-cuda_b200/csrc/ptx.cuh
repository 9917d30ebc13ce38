// Thin inline-PTX wrappers for the sm_100a features the attention kernel is built from: mbarriers, bulk
// asynchronous global->shared copies, tensor memory (TMEM) allocation, tcgen05 MMA / load / store / commit, and
// the shared-memory matrix descriptors the MMA reads its operands through.
//
// Every wait in here is bounded: a wait that does not complete within WAIT_LIMIT_NS returns false so the caller can
// record an error and leave instead of hanging the GPU.
#pragma once
#include <cstdint>
#include <cuda_fp16.h>

namespace llattn {
namespace ptx {

constexpr unsigned long long WAIT_LIMIT_NS = 2000000000ull;   // 2 s: far above any kernel's whole runtime
constexpr uint32_t SUSPEND_HINT_NS = 20000;                   // a waiting thread may sleep this long in hardware; it is woken
                                                              // when the phase completes, so polling costs no issue slots

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ unsigned long long globaltimer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile(
        "{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.b32 %0, 1, 0, p;\n\t}\n" : "=r"(pred));
    return pred != 0;
}

// ---------------------------------------------------------------------------------------------- mbarrier
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\tmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.b32 %0, 1, 0, p;\n\t}\n"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}

// Bounded wait for the phase with the given parity. `abort_flag` (shared memory) lets one role's time-out release
// every other role that is waiting. Returns false on time-out or abort. A phase that is already complete costs one
// non-blocking test; otherwise the hardware suspends the thread inside try_wait until the phase completes (the loop
// body runs about once per wait), and the clock is read every 64 rounds.
// `limit_ns` is the kernels' WAIT_LIMIT_NS everywhere except in the wait self-test, which passes a millisecond.
__device__ __forceinline__ bool mbar_wait_limit(uint32_t bar, uint32_t parity, volatile int* abort_flag, unsigned long long limit_ns) {
    if (mbar_try_wait(bar, parity)) return true;
    uint32_t ok;
    unsigned long long t0 = 0;
    for (uint32_t it = 0;; ++it) {
        asm volatile(
            "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\tselp.b32 %0, 1, 0, p;\n\t}\n"
            : "=r"(ok) : "r"(bar), "r"(parity), "r"(SUSPEND_HINT_NS) : "memory");
        if (ok) return true;
        if ((it & 63u) == 63u || limit_ns < WAIT_LIMIT_NS) {
            if (*abort_flag) return false;
            const unsigned long long t = globaltimer_ns();
            if (t0 == 0) t0 = t;
            else if (t - t0 > limit_ns) { *abort_flag = 1; return false; }
        }
    }
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
    return mbar_wait_limit(bar, parity, abort_flag, WAIT_LIMIT_NS);
}

// Generic-proxy writes to shared memory (st.shared by threads) must be made visible to the async proxy (the
// tensor core reading operands through descriptors) before the consumer is signalled.
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// ---------------------------------------------------------------------------------------------- bulk async copy
// global -> shared, completion counted in bytes on an mbarrier. dst, src 16-byte aligned, bytes a multiple of 16.
__device__ __forceinline__ void bulk_g2s(uint32_t dst_smem, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst_smem), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

// ---------------------------------------------------------------------------------------------- tensor memory
// One warp allocates `ncols` (power of two, 32..512) columns; the base address is written to shared memory.
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
// The same wait, naming the registers a tcgen05.ld filled as in/out operands: the compiler then cannot schedule a use
// of those registers above the wait (a plain register operation has no ordering against a volatile asm otherwise).
__device__ __forceinline__ void tmem_wait_ld_tied(uint32_t (&r)[32]) {
    asm volatile("tcgen05.wait::ld.sync.aligned;" : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]), "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15]), "+r"(r[16]), "+r"(r[17]), "+r"(r[18]), "+r"(r[19]), "+r"(r[20]), "+r"(r[21]), "+r"(r[22]), "+r"(r[23]), "+r"(r[24]), "+r"(r[25]), "+r"(r[26]), "+r"(r[27]), "+r"(r[28]), "+r"(r[29]), "+r"(r[30]), "+r"(r[31]) :: "memory");
}
__device__ __forceinline__ void tmem_wait_ld_tied(uint32_t (&r)[16]) {
    asm volatile("tcgen05.wait::ld.sync.aligned;" : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]), "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15]) :: "memory");
}
__device__ __forceinline__ void tmem_wait_ld_tied(uint32_t (&a)[16], uint32_t (&b)[16]) {
    asm volatile("tcgen05.wait::ld.sync.aligned;" : "+r"(a[0]), "+r"(a[1]), "+r"(a[2]), "+r"(a[3]), "+r"(a[4]), "+r"(a[5]), "+r"(a[6]), "+r"(a[7]), "+r"(a[8]), "+r"(a[9]), "+r"(a[10]), "+r"(a[11]), "+r"(a[12]), "+r"(a[13]), "+r"(a[14]), "+r"(a[15]), "+r"(b[0]), "+r"(b[1]), "+r"(b[2]), "+r"(b[3]), "+r"(b[4]), "+r"(b[5]), "+r"(b[6]), "+r"(b[7]), "+r"(b[8]), "+r"(b[9]), "+r"(b[10]), "+r"(b[11]), "+r"(b[12]), "+r"(b[13]), "+r"(b[14]), "+r"(b[15]) :: "memory");
}
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// 32 lanes x 32 columns of 32-bit cells: thread t of the warp gets lane (warp%4)*32 + t, columns c .. c+31.
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        :: "r"(taddr),
           "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
           "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
           "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
           "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
        :: "r"(taddr),
           "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
           "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}

__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t* r) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
                 :: "r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]) : "memory");
}

// ---------------------------------------------------------------------------------------------- tcgen05 MMA
// Shared-memory matrix descriptor, no swizzle ("interleaved" canonical layout): the operand is made of 8x16-byte
// core matrices, each stored as 128 contiguous bytes.
//   K-major operand (rows = M or N index, 16 bytes = 8 consecutive K elements):
//       lbo = byte distance between the two core matrices adjacent in K, sbo = between 8-row groups.
//   MN-major operand (16 bytes = 8 consecutive M/N elements, the 8 rows of a core matrix are 8 K indices):
//       lbo = byte distance between core matrices adjacent in K, sbo = between groups of 8 in M/N.
__device__ __forceinline__ uint64_t smem_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    return uint64_t((saddr & 0x3ffffu) >> 4) | (uint64_t(lbo_bytes >> 4) << 16) | (uint64_t(sbo_bytes >> 4) << 32) |
           (uint64_t(1) << 46);
}
// The same with the 128-byte swizzle: rows of 128 bytes, the 16-byte chunk c of row r stored at chunk position
// c ^ (r % 8), tile base 1024-byte aligned. K-major operand (row = M/N index, 64 fp16 of K per row): sbo = 1024 (next
// 8 rows), lbo unused, a K-step of 16 elements advances the start address by 32 bytes. MN-major operand (row = K index,
// 64 fp16 of N per row): sbo = 1024 (next 8 K rows), lbo = distance between 64-element column blocks of N, a K-step
// advances by 16 rows. Both conventions were checked against a CPU product on the device.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    return smem_desc(saddr, lbo_bytes, sbo_bytes) | (uint64_t(2) << 61);
}
// Instruction descriptor for kind::f16 with fp16 A and B, fp32 accumulate, M x N tile, no negate, dense.
__host__ __device__ constexpr uint32_t idesc_f16(int M, int N, bool a_mn_major, bool b_mn_major) {
    return (1u << 4) | (uint32_t(a_mn_major) << 15) | (uint32_t(b_mn_major) << 16) | (uint32_t(N >> 3) << 17) |
           (uint32_t(M >> 4) << 24);
}
// D[tmem] (+)= A[smem] * B[smem]; issued by one thread.
__device__ __forceinline__ void mma_ss(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}\n"
        :: "r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]; A is K-major fp16 pairs packed in 32-bit cells, row i in lane i.
__device__ __forceinline__ void mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}\n"
        :: "r"(d_tmem), "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// Descriptor words for the fused issue helpers below: the low word carries the start address and LBO, the high word
// SBO and the version bit; stepping an operand through shared memory is an add on the low word (16-byte units).
__device__ __forceinline__ uint32_t desc_lo(uint32_t saddr, uint32_t lbo_bytes) {
    return ((saddr & 0x3ffffu) >> 4) | ((lbo_bytes >> 4) << 16);
}
__host__ __device__ constexpr uint32_t desc_hi(uint32_t sbo_bytes) { return (sbo_bytes >> 4) | (1u << 14); }

// Whole-warp issue helpers: every lane executes them (uniform control flow, so the operands can live in uniform
// registers); one elected lane issues. Each works from one base descriptor and steps its address field, so the issuing
// warp carries two words per operand tile, not eight descriptors (its instructions sit on the kernel's critical cycle).
//
// S = Q K^T, eight K-steps of 16 channels: A advances 8 TMEM columns per step; step j reads block j / 4 of the K tile,
// 32 bytes (2 units of 16) further along the 128-byte rows per step (kBlock16 = block size / 16). Two commits.
template <uint32_t kBlock16>
__device__ __forceinline__ void mma_ts_s8_warp(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo, uint32_t b_hi, uint32_t idesc,
                                               uint32_t bar1, uint32_t bar2) {
    asm volatile(
        "{\n\t.reg .pred pe, pf, pt;\n\t.reg .b32 a, l;\n\t.reg .b64 db;\n\t"
        "elect.sync _|pe, 0xffffffff;\n\t"
        "setp.ne.b32 pf, 0, 0;\n\t setp.eq.b32 pt, 0, 0;\n\t"
        "mov.b64 db, {%3, %4};\n\t"
        "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], [%2], db, %1, pf;\n\t"
        "add.u32 a, %2, 8;\n\t add.u32 l, %3, 2;\n\t mov.b64 db, {l, %4};\n\t"
        "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], [a], db, %1, pt;\n\t"
        "add.u32 a, %2, 16;\n\t add.u32 l, %3, 4;\n\t mov.b64 db, {l, %4};\n\t"
        "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], [a], db, %1, pt;\n\t"
        "add.u32 a, %2, 24;\n\t add.u32 l, %3, 6;\n\t mov.b64 db, {l, %4};\n\t"
        "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], [a], db, %1, pt;\n\t"
        "add.u32 a, %2, 32;\n\t add.u32 l, %3, %7;\n\t mov.b64 db, {l, %4};\n\t"
        "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], [a], db, %1, pt;\n\t"
        "add.u32 a, %2, 40;\n\t add.u32 l, %3, %8;\n\t mov.b64 db, {l, %4};\n\t"
        "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], [a], db, %1, pt;\n\t"
        "add.u32 a, %2, 48;\n\t add.u32 l, %3, %9;\n\t mov.b64 db, {l, %4};\n\t"
        "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], [a], db, %1, pt;\n\t"
        "add.u32 a, %2, 56;\n\t add.u32 l, %3, %10;\n\t mov.b64 db, {l, %4};\n\t"
        "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], [a], db, %1, pt;\n\t"
        "@pe tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%5];\n\t"
        "@pe tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%6];\n\t"
        "}\n"
        :: "r"(d_tmem), "r"(idesc), "r"(a_tmem), "r"(b_lo), "r"(b_hi), "r"(bar1), "r"(bar2),
           "n"(kBlock16), "n"(kBlock16 + 2), "n"(kBlock16 + 4), "n"(kBlock16 + 6)
        : "memory");
}
// O (+)= P V over a full tile of four 32-key units from one base descriptor: K-step j (16 keys) adds 128 16-byte units;
// the P of unit u sits at columns 32u .. 32u+15 of the S buffer, 8 columns per K-step. One commit (COMMIT), or none.
template <bool COMMIT>
__device__ __forceinline__ void mma_ts_pv8_warp(uint32_t d_tmem, uint32_t p_tmem, uint32_t b_lo, uint32_t b_hi, uint32_t idesc,
                                                uint32_t accumulate_first, uint32_t bar) {
    asm volatile(
        "{\n\t.reg .pred pe, pa, pt;\n\t.reg .b32 a, l;\n\t.reg .b64 db;\n\t"
        "elect.sync _|pe, 0xffffffff;\n\t"
        "setp.ne.b32 pa, %5, 0;\n\t setp.eq.b32 pt, 0, 0;\n\t"
        "mov.b64 db, {%2, %3};\n\t"
        "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %4, pa;\n\t"
        "add.u32 a, %1, 8;\n\t add.u32 l, %2, 128;\n\t mov.b64 db, {l, %3};\n\t"
        "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], [a], db, %4, pt;\n\t"
        "add.u32 a, %1, 32;\n\t add.u32 l, %2, 256;\n\t mov.b64 db, {l, %3};\n\t"
        "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], [a], db, %4, pt;\n\t"
        "add.u32 a, %1, 40;\n\t add.u32 l, %2, 384;\n\t mov.b64 db, {l, %3};\n\t"
        "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], [a], db, %4, pt;\n\t"
        "add.u32 a, %1, 64;\n\t add.u32 l, %2, 512;\n\t mov.b64 db, {l, %3};\n\t"
        "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], [a], db, %4, pt;\n\t"
        "add.u32 a, %1, 72;\n\t add.u32 l, %2, 640;\n\t mov.b64 db, {l, %3};\n\t"
        "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], [a], db, %4, pt;\n\t"
        "add.u32 a, %1, 96;\n\t add.u32 l, %2, 768;\n\t mov.b64 db, {l, %3};\n\t"
        "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], [a], db, %4, pt;\n\t"
        "add.u32 a, %1, 104;\n\t add.u32 l, %2, 896;\n\t mov.b64 db, {l, %3};\n\t"
        "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], [a], db, %4, pt;\n\t"
        "setp.ne.b32 pt, %7, 0;\n\t and.pred pt, pt, pe;\n\t"
        "@pt tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%6];\n\t"
        "}\n"
        :: "r"(d_tmem), "r"(p_tmem), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate_first), "r"(bar), "n"(COMMIT ? 1 : 0)
        : "memory");
}
// Two K-steps (one 32-key unit) of D (+)= A[tmem] * B[smem]; A advances 8 TMEM columns.
__device__ __forceinline__ void mma_ts_x2_warp(uint32_t d_tmem, uint32_t a_tmem, uint64_t b0, uint64_t b1, uint32_t idesc,
                                               uint32_t accumulate_first) {
    asm volatile(
        "{\n\t.reg .pred pe, pa, pt;\n\t.reg .b32 at;\n\t"
        "elect.sync _|pe, 0xffffffff;\n\t"
        "setp.ne.b32 pa, %5, 0;\n\t setp.eq.b32 pt, 0, 0;\n\t"
        "add.u32 at, %1, 8;\n\t"
        "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %4, pa;\n\t"
        "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], [at], %3, %4, pt;\n\t"
        "}\n"
        :: "r"(d_tmem), "r"(a_tmem), "l"(b0), "l"(b1), "r"(idesc), "r"(accumulate_first) : "memory");
}
__device__ __forceinline__ void mma_commit_warp(uint32_t bar) {
    asm volatile("{\n\t.reg .pred pe;\n\telect.sync _|pe, 0xffffffff;\n\t"
                 "@pe tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t}\n" ::"r"(bar) : "memory");
}
// Arrive once on `bar` when every MMA issued so far by this thread has completed.
__device__ __forceinline__ void mma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

}  // namespace ptx
}  // namespace llattn
