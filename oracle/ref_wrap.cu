// C entry points around the reference's own attention kernels, compiled for sm_100a from the reference checkout
// (found through -I<reference>/engine at build time; no reference source is kept in this repository).
// TEST INFRASTRUCTURE ONLY: the GPU parity tests use it as the reference-kernel oracle and the bench reports it
// beside the new kernels. It launches engine/attn.cu's kv_commit (:369), attn_partial (:145) and attn_combine
// (:319) exactly as engine/engine.cu:429-432,591-598,654-657 do.
#include "attn.cu"

extern "C" {

int ref_pick_bpc(int nblocks, int nbatch) { return attn::pick_bpc(nblocks, nbatch); }
int ref_chunks_for(int nblocks, int bpc) { return attn::chunks_for(nblocks, bpc); }
int ref_smem_bytes() { return attn::SMEM_BYTES; }

int ref_kv_commit(const void* Kf, const void* Vf, void* cache, int max_blocks, int blk, int nb, void* stream) {
    attn::kv_commit<<<dim3(4, nb), 128, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const half*>(Kf), static_cast<const half*>(Vf), static_cast<uint8_t*>(cache), max_blocks, blk);
    return int(cudaGetLastError());
}

// One sequence, nb query blocks (block j sees nblocks + j records + its fresh block). bpc <= 0: the engine's policy.
// Opart/Mpart/Lpart sized for nb * 4 * nchunks slots by the caller (nchunks = ref_chunks_for(nblocks + nb - 1, bpc)).
// O16 non-null -> fp16 output; q8 non-null -> int8 activation output instead (as attn_combine does).
int ref_attention(const void* Q, const void* Kf, const void* Vf, const void* cache, int max_blocks, int nblocks, int nb,
                  int bpc, float* Opart, float* Mpart, float* Lpart, void* O16, int8_t* q8, float* s8, int* sum8,
                  void* stream) {
    static bool attr_set = false;
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(attn::attn_partial, cudaFuncAttributeMaxDynamicSharedMemorySize, attn::SMEM_BYTES);
        if (e != cudaSuccess) return int(e);
        attr_set = true;
    }
    if (bpc <= 0) bpc = attn::pick_bpc(nblocks + nb - 1, nb);
    const int nchunks = attn::chunks_for(nblocks + nb - 1, bpc);
    attn::Args a{static_cast<const half*>(Q), static_cast<const half*>(Kf), static_cast<const half*>(Vf),
                 static_cast<const uint8_t*>(cache), max_blocks, nblocks, bpc, nchunks, 0.08838834764831845f,
                 Opart, Mpart, Lpart};
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    attn::attn_partial<<<dim3(4, nchunks, nb), attn::ATT_NTH, attn::SMEM_BYTES, st>>>(a);
    attn::attn_combine<<<dim3(4, 128 / attn::COMB_ROWS, nb), 32 * attn::COMB_ROWS, 0, st>>>(
        Opart, Mpart, Lpart, nchunks, nblocks, bpc, static_cast<half*>(O16), q8, s8, sum8);
    return int(cudaGetLastError());
}

}
