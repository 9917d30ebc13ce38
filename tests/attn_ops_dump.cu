// The attention operators exactly as the reference engine launches them (engine/engine.cu:427-432 for a decode step,
// :589-598 for a batched prefill pass), run on seeded inputs for a list of (committed blocks, batch blocks) cases, with
// both output forms of attn_combine: fp16 O, and the int8 activation (codes in fragment order, group scale, code sum)
// the dense projection reads. Compiled twice from this one file: against the reference's engine/attn.cu and, with
// -DUSE_SHIM, against include/attn_shim.cuh; tests/test_gpu_engine_ops.py compares the two dumps.
//   attn_ops_dump <output file>
#include <cstdio>
#include <cstdlib>
#include <random>
#include <vector>
#include <cuda_runtime.h>
#ifdef USE_SHIM
#include "attn_shim.cuh"
#else
#include "attn.cu"
#endif

#define CK(x) do { cudaError_t e_ = (x); if (e_ != cudaSuccess) { printf("FAIL: CUDA error %s at line %d\n", cudaGetErrorString(e_), __LINE__); return 1; } } while (0)

int main(int argc, char** argv) {
    if (argc < 2) { printf("usage: attn_ops_dump <output file>\n"); return 2; }
    const int cases[][2] = {{0, 1}, {1, 1}, {3, 1}, {40, 1}, {101, 1}, {0, 3}, {5, 16}, {30, 12}, {2, 4}};
    const int MAXB = 160, PB = 16, T = 32;
    std::mt19937 rng(5);
    std::normal_distribution<float> nd(0.f, 1.f);
    auto fill = [&](std::vector<half>& v, bool outlier) {
        for (size_t i = 0; i < v.size(); ++i) v[i] = __float2half(nd(rng) * (outlier && i % 128 == 77 ? 6.f : 1.f));
    };
    std::vector<half> hK(size_t(MAXB) * T * 4 * 128), hV(hK.size());
    fill(hK, true); fill(hV, false);
    half *dK, *dV, *dQ, *dKf, *dVf, *dO;
    uint8_t* cache;
    float *Op, *Mp, *Lp, *s8;
    int8_t* q8;
    int* sum8;
    const size_t rows = size_t(PB) * T;
    CK(cudaMalloc(&dK, hK.size() * 2)); CK(cudaMalloc(&dV, hV.size() * 2));
    CK(cudaMalloc(&dQ, rows * 16 * 128 * 2)); CK(cudaMalloc(&dKf, rows * 4 * 128 * 2)); CK(cudaMalloc(&dVf, rows * 4 * 128 * 2));
    CK(cudaMalloc(&dO, rows * 16 * 128 * 2)); CK(cudaMalloc(&q8, rows * 2048)); CK(cudaMalloc(&s8, rows * 16 * 4)); CK(cudaMalloc(&sum8, rows * 16 * 4));
    CK(cudaMalloc(&cache, size_t(4) * MAXB * attn::KV_BLOCK_BYTES));
    const size_t slots = size_t(PB) * 4 * 4;                 // engine/engine.cu:301-304
    CK(cudaMalloc(&Op, slots * 128 * 128 * 4)); CK(cudaMalloc(&Mp, slots * 128 * 4)); CK(cudaMalloc(&Lp, slots * 128 * 4));
    CK(cudaMemcpy(dK, hK.data(), hK.size() * 2, cudaMemcpyHostToDevice)); CK(cudaMemcpy(dV, hV.data(), hV.size() * 2, cudaMemcpyHostToDevice));
    CK(cudaFuncSetAttribute(attn::attn_partial, cudaFuncAttributeMaxDynamicSharedMemorySize, attn::SMEM_BYTES));
    FILE* f = fopen(argv[1], "wb");
    if (!f) { printf("FAIL: cannot write %s\n", argv[1]); return 1; }
    for (const auto& c : cases) {
        const int ctx0 = c[0], nb = c[1], TT = nb * T;
        std::vector<half> hQ(size_t(TT) * 16 * 128), hKf(size_t(TT) * 4 * 128), hVf(hKf.size());
        fill(hQ, false); fill(hKf, true); fill(hVf, false);
        CK(cudaMemcpy(dQ, hQ.data(), hQ.size() * 2, cudaMemcpyHostToDevice)); CK(cudaMemcpy(dKf, hKf.data(), hKf.size() * 2, cudaMemcpyHostToDevice));
        CK(cudaMemcpy(dVf, hVf.data(), hVf.size() * 2, cudaMemcpyHostToDevice));
        CK(cudaMemset(cache, 0, size_t(4) * MAXB * attn::KV_BLOCK_BYTES));
        if (ctx0) attn::kv_commit<<<dim3(4, ctx0), 128>>>(dK, dV, cache, MAXB, 0);
        if (nb > 1) attn::kv_commit<<<dim3(4, nb), 128>>>(dKf, dVf, cache, MAXB, ctx0);      // a prefill pass commits first
        const int last = nb > 1 ? ctx0 + nb - 1 : ctx0;
        const int bpc = attn::pick_bpc(last, nb), nchunks = attn::chunks_for(last, bpc);
        attn::Args aa{dQ, dKf, dVf, cache, MAXB, ctx0, bpc, nchunks, 0.08838834764831845f, Op, Mp, Lp};
        CK(cudaMemset(dO, 0, rows * 16 * 128 * 2)); CK(cudaMemset(q8, 0, rows * 2048));
        attn::attn_partial<<<dim3(4, nchunks, nb), attn::ATT_NTH, attn::SMEM_BYTES>>>(aa);
        attn::attn_combine<<<dim3(4, 128 / attn::COMB_ROWS, nb), 32 * attn::COMB_ROWS>>>(Op, Mp, Lp, nchunks, ctx0, bpc, dO, nullptr, nullptr, nullptr);
        attn::attn_combine<<<dim3(4, 128 / attn::COMB_ROWS, nb), 32 * attn::COMB_ROWS>>>(Op, Mp, Lp, nchunks, ctx0, bpc, dO, q8, s8, sum8);
        CK(cudaDeviceSynchronize());
        std::vector<half> hO(size_t(TT) * 16 * 128);
        std::vector<int8_t> hq(size_t(TT) * 2048);
        std::vector<float> hs(size_t(TT) * 16);
        std::vector<int> hsum(size_t(TT) * 16);
        CK(cudaMemcpy(hO.data(), dO, hO.size() * 2, cudaMemcpyDeviceToHost)); CK(cudaMemcpy(hq.data(), q8, hq.size(), cudaMemcpyDeviceToHost));
        CK(cudaMemcpy(hs.data(), s8, hs.size() * 4, cudaMemcpyDeviceToHost)); CK(cudaMemcpy(hsum.data(), sum8, hsum.size() * 4, cudaMemcpyDeviceToHost));
        const int head[4] = {ctx0, nb, bpc, nchunks};
        fwrite(head, 4, 4, f);
        fwrite(hO.data(), 2, hO.size(), f); fwrite(hq.data(), 1, hq.size(), f);
        fwrite(hs.data(), 4, hs.size(), f); fwrite(hsum.data(), 4, hsum.size(), f);
        printf("case ctx %d nb %d: bpc %d nchunks %d\n", ctx0, nb, bpc, nchunks);
    }
    fclose(f);
    printf("DONE\n");
    return 0;
}
