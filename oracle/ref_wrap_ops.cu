// C entry point around the reference's own qk_norm_rope kernel (engine/ops.cu:429-453), compiled for sm_100a from
// the reference checkout (found through -I<reference>/engine at build time). TEST INFRASTRUCTURE ONLY.
#include "ops.cu"

extern "C" int ref_qk_norm_rope(const float* qkv, const int* pos, const float* gq, const float* gk, float eps,
                                const float* inv_freq, void* q, void* k, void* v, int T, void* stream) {
    ops::qk_norm_rope<<<dim3(T, 3), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        qkv, pos, gq, gk, eps, inv_freq, static_cast<half*>(q), static_cast<half*>(k), static_cast<half*>(v));
    return int(cudaGetLastError());
}
