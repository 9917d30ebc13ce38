// C entry point around the reference's own W.A8 GEMM (engine/moe_i8.cu:408-442), launched the way the engine launches its
// attention-output projection (engine/engine.cu:346-358 with gemm<4, 2>(Ly.dense, items_dense, nullptr, 1, nullptr, oA.a,
// ones, HID, HID, nullptr, h, 1, 2)): 4 warps, NT = 4 (32 tokens per work item), 2 strips per warp, MODE 2, one K split.
// Compiled for sm_100a from the reference checkout (-I<reference>/engine). TEST INFRASTRUCTURE ONLY.
#include "moe_i8.cu"

// W: strips in device layout (already relaid), one matrix (expert 0, 4-bit). Tokens in items of 32 (the reference's
// block); `work` and the expert table are device buffers the caller provides: work [nitems] of {0, 32 i, 32},
// off [1] = {0}, bits [1] = {4}.
extern "C" int ref_dense_w4a8(const uint8_t* W, const int8_t* q, const float* s, const int* sum, float* Y, int ntokens, int rows,
                              int K, const void* work, const uint64_t* off, const int8_t* bits, const float* ones, int groups,
                              void* stream) {
    constexpr int GW = 4, GMS = 2, NT = 4;
    if (ntokens % 32 || (rows / 16) % (GW * GMS * groups) || (K / 128) % 4) return -1;
    moe8::ExpertTable tab{W, off, off, bits};
    moe8::Act X{q, s, sum};
    moe8::GemmArgs g{tab, static_cast<const moe8::Work*>(work), nullptr, nullptr, X, ones, rows, K, nullptr, Y, groups, 0};
    const int smem = moe8::smem_bytes(NT, K);
    cudaFuncSetAttribute(moe8::gemm<GW, NT, GMS, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    const dim3 grid(rows / 16 / (GW * GMS * groups), ntokens / 32, 1);
    moe8::gemm<GW, NT, GMS, 2><<<grid, GW * 32, smem, static_cast<cudaStream_t>(stream)>>>(g);
    return int(cudaGetLastError());
}
