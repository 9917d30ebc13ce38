// C ABI of libllattn.so (see include/llattn.h): argument checking, the host-side work planner and the kernel
// launches. No torch types, no exit(): every failure comes back as a status code plus a thread-local message.
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <algorithm>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <cstdlib>
#include <cmath>
#include <mutex>
#include <new>
#include <vector>

#include "llattn.h"
#include "common.cuh"
#include "kv_commit.cuh"
#include "attn_kernel.cuh"
#include "merge_kernel.cuh"
#include "qkv_prepare.cuh"
#include "dense_i8.cuh"

namespace {

thread_local char g_err[512] = "";

int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}

#define CU(call)                                                                                  \
    do {                                                                                          \
        cudaError_t e_ = (call);                                                                  \
        if (e_ != cudaSuccess) return fail(LLATTN_ECUDA, "%s: %s", #call, cudaGetErrorString(e_)); \
    } while (0)

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
inline cudaStream_t as_stream(void* s) { return static_cast<cudaStream_t>(s); }

}  // namespace

// ====================================================================================================== context

struct llattn_ctx {
    int device = 0;
    int num_sms = 0;
    int* err_word = nullptr;          // device
    void* workspace = nullptr;        // device: partial results (grow-only)
    size_t workspace_bytes = 0;
    void* stage = nullptr;            // device staging for the host-buffer entry point: two slots (grow-only)
    size_t stage_bytes = 0, stage_slot_bytes = 0;
    bool host_ready = false;          // copy streams and events of the host-buffer path exist
    int host_slot = 0;
    cudaStream_t s_in = nullptr, s_out = nullptr;
    cudaEvent_t ev_in[2] = {}, ev_comp[2] = {}, ev_out[2] = {};
    std::mutex mu;
};

struct llattn_plan {
    llattn_ctx* ctx = nullptr;
    llattn_plan_stats stats{};
    void* dev_blob = nullptr;         // seq descriptors, work items, per-CTA ranges, tile descriptors (fixed section offsets)
    void* host_blob = nullptr;        // pinned mirror: llattn_plan_update fills it and copies it up asynchronously
    size_t blob_bytes = 0, off_seqs = 0, off_items = 0, off_cta = 0, off_merge = 0;
    size_t cap_seqs = 0, cap_items = 0, cap_tiles = 0;
    int launch_ctas = 0;              // grid of every launch of this plan (CTAs beyond the used ones find no items)
    cudaEvent_t ev_upload = nullptr;
    bool upload_pending = false;
    const llattn::SeqDesc* d_seqs = nullptr;
    const llattn::RunDesc* d_items = nullptr;
    const int32_t* d_cta_first = nullptr;
    const llattn::MergeDesc* d_merge = nullptr;
};

namespace {

struct DeviceGuard {
    int prev = -1;
    bool ok = true;
    explicit DeviceGuard(int dev) {
        if (cudaGetDevice(&prev) != cudaSuccess) { ok = false; return; }
        if (prev != dev && cudaSetDevice(dev) != cudaSuccess) ok = false;
    }
    ~DeviceGuard() { if (prev >= 0) cudaSetDevice(prev); }
};

int ensure_kernel_attrs() {
    static std::mutex mu;
    static bool done[64] = {};
    int dev = 0;
    CU(cudaGetDevice(&dev));
    std::lock_guard<std::mutex> lk(mu);
    if (dev < 64 && done[dev]) return LLATTN_OK;
    CU(cudaFuncSetAttribute(llattn::attn_tile_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, llattn::ATTN_SMEM_BYTES));
    CU(cudaFuncSetAttribute(llattn::attn_tile_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, llattn::ATTN_SMEM_BYTES));
    if (dev < 64) done[dev] = true;
    return LLATTN_OK;
}

int grow(void** p, size_t* have, size_t need) {
    if (need <= *have) return LLATTN_OK;
    if (*p) { CU(cudaFree(*p)); *p = nullptr; *have = 0; }
    const size_t want = need + need / 4;
    if (cudaMalloc(p, want) != cudaSuccess) {
        cudaGetLastError();
        return fail(LLATTN_ENOMEM, "cudaMalloc of %zu bytes failed", want);
    }
    *have = want;
    return LLATTN_OK;
}

}  // namespace

extern "C" {

const char* llattn_version(void) { return "llattn 0.1 (sm_100a)"; }
const char* llattn_last_error(void) { return g_err; }

int llattn_pick_bpc(int nblocks, int nbatch) {
    if (nbatch < 1) nbatch = 1;
    const int want = nbatch >= 4 ? 1 : 4 / nbatch;
    return std::max(1, (nblocks + want - 1) / want);
}
int llattn_chunks_for(int nblocks, int bpc) { return nblocks <= 0 ? 1 : (nblocks + bpc - 1) / bpc; }
int llattn_tile_units(void) { return llattn::TILE_UNITS; }

// ------------------------------------------------------------------------------------------------------ commit

int llattn_kv_commit(const void* Kf, const void* Vf, void* cache, int max_blocks, int blk, int nb, void* stream) {
    if (!Kf || !Vf || !cache) return fail(LLATTN_EINVAL, "kv_commit: null pointer");
    if (nb < 0 || blk < 0 || max_blocks <= 0 || blk + nb > max_blocks)
        return fail(LLATTN_EINVAL, "kv_commit: blocks [%d, %d) outside a cache of %d blocks", blk, blk + nb, max_blocks);
    if (!aligned16(Kf) || !aligned16(Vf) || !aligned16(cache)) return fail(LLATTN_EINVAL, "kv_commit: pointers must be 16-byte aligned");
    if (nb == 0) return LLATTN_OK;
    if (nb > 65535) return fail(LLATTN_EINVAL, "kv_commit: at most 65535 blocks per call");
    llattn::kv_commit_kernel<<<dim3(llattn::NKV, nb), llattn::COMMIT_THREADS, 0, as_stream(stream)>>>(
        static_cast<const half*>(Kf), static_cast<const half*>(Vf), static_cast<uint8_t*>(cache), nullptr, max_blocks, blk);
    CU(cudaGetLastError());
    return LLATTN_OK;
}

int llattn_kv_commit_paged(const void* Kf, const void* Vf, void* pool, const int32_t* pages, int nb, void* stream) {
    if (!Kf || !Vf || !pool || !pages) return fail(LLATTN_EINVAL, "kv_commit_paged: null pointer");
    if (nb < 0 || nb > 65535) return fail(LLATTN_EINVAL, "kv_commit_paged: nb must be in [0, 65535]");
    if (!aligned16(Kf) || !aligned16(Vf) || !aligned16(pool)) return fail(LLATTN_EINVAL, "kv_commit_paged: pointers must be 16-byte aligned");
    if (nb == 0) return LLATTN_OK;
    llattn::kv_commit_kernel<<<dim3(llattn::NKV, nb), llattn::COMMIT_THREADS, 0, as_stream(stream)>>>(
        static_cast<const half*>(Kf), static_cast<const half*>(Vf), static_cast<uint8_t*>(pool), pages, 0, 0);
    CU(cudaGetLastError());
    return LLATTN_OK;
}

// ------------------------------------------------------------------------------------------------------ producer

namespace {
int launch_prepare(const float* qkv, const int32_t* pos, const float* gq, const float* gk, float eps, const float* inv_freq,
                   void* q, void* k, void* v, int T, void* records, const int32_t* pages, int max_blocks, int blk, void* stream) {
    llattn::PrepArgs a{qkv, pos, gq, gk, inv_freq, eps, static_cast<half*>(q), static_cast<half*>(k), static_cast<half*>(v), T,
                       static_cast<uint8_t*>(records), pages, max_blocks, blk};
    llattn::qkv_prepare_kernel<<<dim3((T + llattn::BLK - 1) / llattn::BLK, 8), llattn::PREP_THREADS, 0, as_stream(stream)>>>(a);
    CU(cudaGetLastError());
    return LLATTN_OK;
}
}  // namespace

int llattn_qk_norm_rope(const float* qkv, const int32_t* pos, const float* gq, const float* gk, float eps,
                        const float* inv_freq, void* q, void* k, void* v, int T, void* stream) {
    if (!qkv || !pos || !gq || !gk || !inv_freq || !q || !k || !v) return fail(LLATTN_EINVAL, "qk_norm_rope: null pointer");
    if (T < 0 || T > 1 << 24) return fail(LLATTN_EINVAL, "qk_norm_rope: T = %d", T);
    if (!aligned16(k) || !aligned16(v)) return fail(LLATTN_EINVAL, "qk_norm_rope: k and v must be 16-byte aligned");
    if (T == 0) return LLATTN_OK;
    return launch_prepare(qkv, pos, gq, gk, eps, inv_freq, q, k, v, T, nullptr, nullptr, 0, 0, stream);
}

int llattn_qkv_prepare_commit(const float* qkv, const int32_t* pos, const float* gq, const float* gk, float eps,
                              const float* inv_freq, void* q, void* k, void* v, int nb, void* cache, const int32_t* pages,
                              int max_blocks, int blk, void* stream) {
    if (!qkv || !pos || !gq || !gk || !inv_freq || !q || !k || !v || !cache) return fail(LLATTN_EINVAL, "qkv_prepare_commit: null pointer");
    if (nb < 0 || nb > 65535) return fail(LLATTN_EINVAL, "qkv_prepare_commit: nb must be in [0, 65535]");
    if (!pages && (blk < 0 || max_blocks <= 0 || blk + nb > max_blocks))
        return fail(LLATTN_EINVAL, "qkv_prepare_commit: blocks [%d, %d) outside a cache of %d blocks", blk, blk + nb, max_blocks);
    if (!aligned16(k) || !aligned16(v) || !aligned16(cache)) return fail(LLATTN_EINVAL, "qkv_prepare_commit: k, v and cache must be 16-byte aligned");
    if (nb == 0) return LLATTN_OK;
    return launch_prepare(qkv, pos, gq, gk, eps, inv_freq, q, k, v, nb * llattn::BLK, cache, pages, max_blocks, blk, stream);
}

// ------------------------------------------------------------------------------------------------------ consumer
// The attention-output projection on the int8 activations the merge kernel writes.

int llattn_dense_w4a8(const void* W, const int8_t* q, const float* s, const int32_t* sum, float* Y, int ntokens, int rows, int K,
                      int* err_word, void* stream) {
    if (!W || !q || !s || !sum || !Y) return fail(LLATTN_EINVAL, "dense_w4a8: null pointer");
    if (ntokens < 0 || ntokens > 1 << 22) return fail(LLATTN_EINVAL, "dense_w4a8: ntokens = %d", ntokens);
    if (rows <= 0 || rows % llattn::DN_ROWS || K <= 0 || K % llattn::DN_GROUP || K > 1 << 20 || rows > 1 << 20)
        return fail(LLATTN_EINVAL, "dense_w4a8: rows = %d, K = %d (both multiples of 128)", rows, K);
    if (ntokens == 0) return LLATTN_OK;
    static std::once_flag once[64];
    int dev = 0;
    CU(cudaGetDevice(&dev));
    if (dev >= 0 && dev < 64)
        std::call_once(once[dev], [] {
            cudaFuncSetAttribute(llattn::dense_i8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, llattn::DN_SMEM_BYTES);
        });
    llattn::DenseParams p{static_cast<const uint8_t*>(W), q, s, sum, Y, ntokens, rows, K, err_word};
    const dim3 grid(rows / llattn::DN_ROWS, (ntokens + llattn::DN_TOK - 1) / llattn::DN_TOK);
    llattn::dense_i8_kernel<<<grid, llattn::DN_THREADS, llattn::DN_SMEM_BYTES, as_stream(stream)>>>(p);
    CU(cudaGetLastError());
    return LLATTN_OK;
}

}  // extern "C"

#include "llattn_attention.inl"
#include "kvpool.inl"

// ====================================================================================================== no-allocation entry point
// Scratch for llattn_attention_static: partial results (un-normalised O, reference maximum, row sum) of up to
// STATIC_MAX_SLOTS runs. It lives in the library image, so every GPU that loads the library holds these bytes until the
// process exits, and every call on a device shares them.
namespace {
constexpr int STATIC_MAX_SLOTS = 160;                                  // 148 SMs worth of runs for one query block, rounded up
constexpr int STATIC_MAX_QBLOCKS = 16;                                 // a prefill pass of the reference engine
constexpr size_t STATIC_SLOT_FLOATS = size_t(llattn::QR) * llattn::D + 2 * llattn::QR;   // 16640 floats = 66560 B
}  // namespace
static __device__ __align__(256) float g_static_scratch[STATIC_MAX_SLOTS * STATIC_SLOT_FLOATS];   // 10.16 MiB

namespace {
struct StaticSetup { float* scratch = nullptr; int num_sms = 0; bool ready = false; };
StaticSetup g_static[64];
std::mutex g_static_mu;

// Once per device, with that device current: resolve the DEVICE address of the scratch array. In host code the
// array's name is only a stand-in symbol; handing it to a kernel would make the kernel dereference a host address.
int static_setup(int dev, StaticSetup** out) {
    if (dev < 0 || dev >= 64) return fail(LLATTN_EINVAL, "attention_static: device index %d not supported", dev);
    std::lock_guard<std::mutex> lk(g_static_mu);
    StaticSetup& st = g_static[dev];
    if (!st.ready) {
        float* ptr = nullptr;
        cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_static_scratch);
        if (e != cudaSuccess || !ptr) return fail(LLATTN_ECUDA, "attention_static: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
        e = cudaDeviceGetAttribute(&st.num_sms, cudaDevAttrMultiProcessorCount, dev);
        if (e != cudaSuccess) return fail(LLATTN_ECUDA, "attention_static: cudaDeviceGetAttribute: %s", cudaGetErrorString(e));
        st.scratch = ptr;
        st.ready = true;
    }
    *out = &st;
    return LLATTN_OK;
}
}  // namespace

extern "C" int llattn_attention_static(const void* Q, const void* Kf, const void* Vf, const void* cache, int max_blocks,
                                       int nblocks, int nb, float scale, void* O16, float* O32, float* LSE, int8_t* q8,
                                       float* s8, int32_t* sum8, int* err_word, void* stream) {
    using namespace llattn;
    if (!Q || !Kf || !Vf) return fail(LLATTN_EINVAL, "attention_static: Q, Kf and Vf are required");
    if (!O16 && !O32 && !LSE && !q8) return fail(LLATTN_EINVAL, "attention_static: no output requested");
    if (q8 && (!s8 || !sum8)) return fail(LLATTN_EINVAL, "attention_static: q8 needs s8 and sum8");
    if (nb < 1 || nb > STATIC_MAX_QBLOCKS)
        return fail(LLATTN_EINVAL, "attention_static: %d query blocks; the built-in scratch serves 1..%d per call", nb, STATIC_MAX_QBLOCKS);
    if (nblocks < 0 || max_blocks < 0 || nblocks + nb - 1 > max_blocks)
        return fail(LLATTN_EINVAL, "attention_static: %d blocks visible, cache holds %d", nblocks + nb - 1, max_blocks);
    if (nblocks + nb - 1 > 0 && !cache) return fail(LLATTN_EINVAL, "attention_static: null cache with committed blocks");
    if (!aligned16(Q) || !aligned16(Kf) || !aligned16(Vf) || !aligned16(cache) || !aligned16(O16) || !aligned16(O32))
        return fail(LLATTN_EINVAL, "attention_static: pointers must be 16-byte aligned");
    int dev = -1;
    CU(cudaGetDevice(&dev));
    StaticSetup* st = nullptr;
    if (int rc = static_setup(dev, &st)) return rc;
    if (int rc = ensure_kernel_attrs()) return rc;
    // split each (query block, kv head) into runs so that about one run lands on every SM, within the scratch's slots
    const int nbl = nblocks + nb - 1;
    const int want = std::max(1, std::min(STATIC_MAX_SLOTS / (NKV * nb), (st->num_sms + NKV * nb - 1) / (NKV * nb)));
    int bpc = std::max(1, (nbl + want - 1) / want);
    bpc = std::max(bpc, std::min(nbl, 8));                       // at least two 128-key tiles per run when there are that many
    bpc = (bpc + TILE_UNITS - 1) / TILE_UNITS * TILE_UNITS;      // cuts on tile boundaries
    const int nchunks = llattn_chunks_for(nbl, bpc);
    if (NKV * nchunks * nb > STATIC_MAX_SLOTS)
        return fail(LLATTN_ENOMEM, "attention_static: %d partial slots needed, the built-in scratch holds %d", NKV * nchunks * nb, STATIC_MAX_SLOTS);
    const size_t ns = size_t(NKV) * nchunks * nb;
    float* Opart = st->scratch;
    float* Mpart = Opart + ns * QR * D;
    float* Lpart = Mpart + ns * QR;
    KParams p{};
    p.Q = static_cast<const half*>(Q); p.Kf = static_cast<const half*>(Kf); p.Vf = static_cast<const half*>(Vf);
    p.Opart = Opart; p.Mpart = Mpart; p.Lpart = Lpart;
    p.sl2 = (scale > 0.f ? scale : 0.08838834764831845f) * 1.4426950408889634f;
    p.err = err_word;
    p.ref_seq = SeqDesc{static_cast<const uint8_t*>(cache), nullptr, max_blocks, nblocks, nb, 0};
    p.ref_bpc = bpc;
    p.ref_nchunks = nchunks;
    attn_tile_kernel<false><<<NKV * nchunks * nb, ATTN_THREADS, ATTN_SMEM_BYTES, as_stream(stream)>>>(p);
    CU(cudaGetLastError());
    MergeOut o{static_cast<half*>(O16), O32, LSE, q8, s8, sum8};
    combine_ref_kernel<<<dim3(NKV, QR / MERGE_ROWS, nb), MERGE_THREADS, 0, as_stream(stream)>>>(Opart, Mpart, Lpart, nchunks, nblocks, bpc, o);
    CU(cudaGetLastError());
    return LLATTN_OK;
}

// ====================================================================================================== wait self-test
// What a kernel of this library does when a wait can never complete, shown without making any real kernel fail: four
// warps wait on barriers nobody will ever arrive on, a fifth on a counter nobody counts into (the wait a CTA does for
// the other runs of a split tile). Warp 0 has `limit_ns` (a millisecond in the test); when its wait runs out it raises
// the CTA's abort flag, as every role of the attention kernel does, and the other warps - whose own limit is the
// kernels' two seconds - see the flag at their next poll and leave too. Then the fifth warp waits on its counter once
// more, alone and with the short limit, to show that wait running out by itself. Every warp reports through the error
// word, the kernel returns normally and the context stays usable.
namespace llattn {
__device__ int selftest_counter;       // nothing ever counts in here

__global__ void __launch_bounds__(160) wait_selftest_kernel(unsigned long long limit_ns, int* err, unsigned long long* waited_ns) {
    __shared__ uint64_t bars[4];
    __shared__ int abort_flag;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int i = 0; i < 4; ++i) ptx::mbar_init(ptx::smem_u32(&bars[i]), 1);
        ptx::fence_mbar_init();
        abort_flag = 0;
    }
    __syncthreads();
    const unsigned long long t0 = ptx::globaltimer_ns();
    bool ok;
    if (warp < 4) ok = ptx::mbar_wait_limit(ptx::smem_u32(&bars[warp]), 0, &abort_flag, warp == 0 ? limit_ns : ptx::WAIT_LIMIT_NS);
    else ok = wait_count(&selftest_counter, 1, &abort_flag, ptx::WAIT_LIMIT_NS);      // the wait of the tile folding: released by the flag
    const unsigned long long t1 = ptx::globaltimer_ns();
    if (!ok && lane == 0) {
        atomicOr(err, warp == 0 ? ERR_WAIT_PRODUCER : warp == 1 ? ERR_WAIT_DEQUANT : warp == 2 ? ERR_WAIT_MMA : warp == 3 ? ERR_WAIT_SOFTMAX : ERR_WAIT_FOLD);
        waited_ns[warp] = t1 - t0;
    }
    __syncthreads();
    // and the counter wait running out by itself, with the short limit
    if (warp == 4) {
        abort_flag = 0;
        __syncwarp();
        const unsigned long long t2 = ptx::globaltimer_ns();
        const bool ok2 = wait_count(&selftest_counter, 1, &abort_flag, limit_ns);
        if (!ok2 && lane == 0) waited_ns[5] = ptx::globaltimer_ns() - t2;
    }
}
}  // namespace llattn

extern "C" int llattn_wait_selftest(unsigned long long limit_ns, int* err_word, unsigned long long* waited_ns6, void* stream) {
    if (!err_word || !waited_ns6) return fail(LLATTN_EINVAL, "wait_selftest: null pointer");
    if (limit_ns == 0 || limit_ns > 100000000ull) return fail(LLATTN_EINVAL, "wait_selftest: limit of %llu ns; 1 ns .. 100 ms", limit_ns);
    llattn::wait_selftest_kernel<<<1, 160, 0, as_stream(stream)>>>(limit_ns, err_word, waited_ns6);
    CU(cudaGetLastError());
    return LLATTN_OK;
}

#ifdef LLATTN_TRACE
// Tuning builds only: points the kernel's timeline hooks at a device buffer of 18 * 2048 64-bit words.
extern "C" int llattn_debug_set_trace(void* dev_ptr) {
    CU(cudaMemcpyToSymbol(llattn::g_trace_buf, &dev_ptr, sizeof(dev_ptr)));
    return LLATTN_OK;
}
#endif
