// C ABI of libllattn.so (see include/llattn.h): argument checking, the host-side work planner and the kernel
// launches. No torch types, no exit(): every failure comes back as a status code plus a thread-local message.
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <algorithm>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <new>
#include <vector>

#include "llattn.h"
#include "common.cuh"
#include "kv_commit.cuh"
#include "attn_kernel.cuh"
#include "merge_kernel.cuh"

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
    void* stage = nullptr;            // device staging for the host-buffer entry point (grow-only)
    size_t stage_bytes = 0;
    std::mutex mu;
};

struct llattn_plan {
    llattn_ctx* ctx = nullptr;
    llattn_plan_stats stats{};
    void* dev_blob = nullptr;         // seq descriptors, work items, per-CTA ranges, merge descriptors
    const llattn::SeqDesc* d_seqs = nullptr;
    const llattn::WorkItem* d_items = nullptr;
    const int32_t* d_cta_first = nullptr;
    const llattn::MergeDesc* d_merge = nullptr;
    int ntiles_out = 0;               // output tiles = nq_total * 4
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
    CU(cudaFuncSetAttribute(llattn::attn_tile_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, llattn::ATTN_SMEM_BYTES));
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

}  // extern "C"

#include "llattn_attention.inl"
