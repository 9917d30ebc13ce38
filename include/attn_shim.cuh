// Source-level stand-in for the reference's engine/attn.cu: namespace `attn` with the names, signatures and launch
// shapes the reference's engine.cu, decode.cu and tests use, bodies from this repository's sm_100a kernels.
//
// Use: in the reference tree replace `#include "attn.cu"` (engine/engine.cu:27, engine/tests/test_attn.cu:9) by
// `#include "attn_shim.cuh"` and compile with
//   nvcc -std=c++17 -gencode arch=compute_100a,code=sm_100a -I<this repo>/include -I<this repo>/llada2-orin-cuda_b200/csrc
// Everything the callers do keeps working unchanged: `attn::Args{...}` aggregate initialisation
// (engine/engine.cu:430,595), `<<<dim3(4, nchunks, nb), attn::ATT_NTH, attn::SMEM_BYTES, st>>>` launches (:431,:596),
// `cudaFuncSetAttribute(attn::attn_partial, ...)` (:342), taking the kernels' addresses and patching their graph
// nodes (:524-552), `attn::kv_commit<<<dim3(4, nb), 128>>>` (:591,:656).
//
// What differs from the file it replaces (all visible through the constants below):
//   ATT_NTH is 512 and SMEM_BYTES about 203 KB (one CTA per SM; the reference ran 128 threads, 79 KB, two per SM);
//   a CTA's chunk should hold a multiple of 4 blocks (128-key MMA tiles) — any blocks_per_chunk is correct, multiples
//   of 4 are faster; and B200 wants about one chunk per SM and kv head quarter, so a caller after speed sizes its
//   partial buffers for MAX_CHUNKS_HINT chunks (engine/engine.cu:301 sizes them for 4) and calls pick_bpc below,
//   which spreads a single block's context over the whole GPU instead of over 4 chunks.
#pragma once
#include <cuda_fp16.h>
#include <cstdint>
#include <algorithm>
#include "common.cuh"
#include "kv_commit.cuh"
#include "attn_kernel.cuh"
#include "merge_kernel.cuh"

namespace attn {

constexpr int D = llattn::D, BLK = llattn::BLK, QR = llattn::QR;
constexpr int KV_BLOCK_BYTES = llattn::REC_BYTES;
constexpr int KOFF_META = llattn::KOFF_META, VOFF = llattn::VOFF, VOFF_META = llattn::VOFF_META;
constexpr int ATT_NTH = llattn::ATTN_THREADS;
constexpr int SMEM_BYTES = llattn::ATTN_SMEM_BYTES;
constexpr int COMB_ROWS = 8;                              // engine/attn.cu:318; the callers size the launch with it
constexpr int MAX_CHUNKS_HINT = 37;                       // 148 SMs / 4 kv heads

struct Args {                                             // engine/attn.cu:51-64, field for field
    const half* Q;
    const half* Kf;
    const half* Vf;
    const uint8_t* cache;
    int max_blocks;
    int nblocks;
    int blocks_per_chunk;
    int nchunks;
    float scale;
    float* Opart;
    float* Mpart;
    float* Lpart;
};

__host__ __device__ inline int chunks_for(int nblocks, int bpc) { return nblocks <= 0 ? 1 : (nblocks + bpc - 1) / bpc; }

// engine/attn.cu:361-364 asked for ~4 chunks per head (8 SMs). Here: about one chunk per SM over the 4 kv heads and
// nbatch query blocks, at least 8 blocks per chunk, on a multiple of 4. With max_chunks the caller caps the count to
// what its partial buffers hold (pass 4 to reproduce the reference's buffer sizing).
//
// Buffer bound for an UNMODIFIED engine. The reference sizes Opart/Mpart/Lpart for PB x 4 heads x 4 chunks = 256 slots
// (PB = 16, engine/engine.cu:301-304) and calls pick_bpc(nblocks, nb) with two arguments (engine.cu:429,535,594). A
// launch writes slot indices below nb x 4 x nchunks, and nchunks never exceeds the cap below. With the default cap that
// is 1 x 4 x 37 = 148 slots for a decode step and at most 192 for a prefill pass (nb = 12: 4 chunks, nb = 16: 3 chunks),
// under 256 for every nb in 1..16; the static_assert keeps it so if either constant changes. An engine with a smaller
// PB must pass max_chunks = 4.
constexpr int cmax(int a, int b) { return a > b ? a : b; }
constexpr int cmin(int a, int b) { return a < b ? a : b; }
constexpr int chunk_cap(int nbatch, int max_chunks) { return cmax(1, cmin(max_chunks, (148 + 4 * nbatch - 1) / (4 * nbatch))); }
inline int pick_bpc(int nblocks, int nbatch, int max_chunks = MAX_CHUNKS_HINT) {
    const int want = chunk_cap(nbatch, max_chunks);
    int bpc = std::max(1, (nblocks + want - 1) / want);
    bpc = std::max(bpc, std::min(nblocks, 8));
    return (bpc + 3) / 4 * 4;
}
// chunks never exceed the cap (bpc >= ceil(nblocks / cap)), so nb x 4 x cap bounds the slots a launch touches
constexpr int REFERENCE_PARTIAL_SLOTS = 16 * 4 * 4;       // PB x kv heads x chunks, engine/engine.cu:301-304
constexpr bool slots_fit_reference(int nb) { return nb > 16 || (nb * 4 * chunk_cap(nb, MAX_CHUNKS_HINT) <= REFERENCE_PARTIAL_SLOTS && slots_fit_reference(nb + 1)); }
static_assert(slots_fit_reference(1), "the default chunk cap overflows the partial buffers an unmodified engine allocates");

__global__ void __launch_bounds__(ATT_NTH, 1) attn_partial(Args a) {
    llattn::KParams p{};
    p.Q = a.Q; p.Kf = a.Kf; p.Vf = a.Vf;
    p.Opart = a.Opart; p.Mpart = a.Mpart; p.Lpart = a.Lpart;
    p.sl2 = a.scale * 1.4426950408889634f;
    p.err = nullptr;
    p.ref_seq = llattn::SeqDesc{a.cache, nullptr, a.max_blocks, a.nblocks, int(gridDim.z), 0};
    p.ref_bpc = a.blocks_per_chunk;
    p.ref_nchunks = a.nchunks;
    // reference grid (kv head, chunk, query block); gridDim.y may be smaller than nchunks after a graph patch
    if (int(blockIdx.y) >= a.nchunks) return;
    llattn::attn_tile_body<false>(p, (int(blockIdx.z) * a.nchunks + int(blockIdx.y)) * 4 + int(blockIdx.x));
}

// The reference's launch shape is kept (grid (4, 128 / COMB_ROWS, nb), a warp per query row); the warp folds its row with
// the routine the attention kernel's own folding uses (merge_kernel.cuh: lane = 4 dims, the slots' reference exponents
// and row sums fetched by the lanes in parallel, up to twelve slots' rows in flight).
__global__ void __launch_bounds__(32 * COMB_ROWS)
attn_combine(const float* Opart, const float* Mpart, const float* Lpart, int nchunks, int nblocks, int bpc, half* O,
             int8_t* q8, float* s8, int* sum8) {
    llattn::MergeOut o{};
    if (q8) { o.q8 = q8; o.s8 = s8; o.sum8 = sum8; }      // as engine/attn.cu:340-357: the int8 form replaces fp16 O
    else o.O16 = O;
    const int kvh = blockIdx.x, jb = blockIdx.z;
    const int r = blockIdx.y * COMB_ROWS + (threadIdx.x >> 5);
    const llattn::MergeDesc md{jb, kvh, (jb * 4 + kvh) * nchunks, chunks_for(nblocks + jb, bpc)};
    llattn::fold_row_warp(Opart, Mpart, Lpart, md, r, int(threadIdx.x & 31), o);
}

__global__ void __launch_bounds__(llattn::COMMIT_THREADS)
kv_commit(const half* Kf, const half* Vf, uint8_t* cache, int max_blocks, int blk) {
    llattn::kv_commit_body(Kf, Vf, cache, nullptr, max_blocks, blk);
}

}  // namespace attn
