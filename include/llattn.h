/*
 * llattn — block-diffusion attention over the int4 "4c/4" KV cache and its block-commit quantiser, for sm_100a.
 *
 * C ABI of libllattn.so. Plain pointers and sizes only. Every function returns an llattn_status (0 = ok) and never
 * exits the process; llattn_last_error() gives the message of the last failure on the calling thread. Unless a
 * parameter says "host", data pointers are DEVICE pointers owned by the caller. `stream` is a cudaStream_t passed
 * as void* (NULL = the default stream). A context may be used from any thread, one call at a time.
 *
 * Each entry point names the interface of the reference engine (patrickbdevaney/llada2-orin-cuda) it stands in
 * for, as file:line of that project.
 *
 * Layouts (engine/attn.cu:51-64 and :3-7,22-25):
 *   Q        [nq_total][32 tok][16 heads][128] fp16, after q-norm and RoPE
 *   Kf, Vf   [nq_total][32 tok][4 heads][128]  fp16, the fresh K/V of the query blocks
 *   record   4736 bytes per (kv head, 32-token block): K codes [32][64], K scale fp16[128], K min fp16[128],
 *            V codes [32][64], V scale fp16[32], V min fp16[32]; value = code * scale + min
 *   cache    one layer of one sequence, [4 heads][max_blocks][4736]
 */
#ifndef LLATTN_H
#define LLATTN_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define LLATTN_HEAD_DIM 128
#define LLATTN_BLOCK_TOKENS 32
#define LLATTN_KV_HEADS 4
#define LLATTN_Q_HEADS 16
#define LLATTN_RECORD_BYTES 4736 /* attn::KV_BLOCK_BYTES, engine/attn.cu:23 */
#define LLATTN_KOFF_META 2048    /* attn::KOFF_META */
#define LLATTN_VOFF 2560         /* attn::VOFF */
#define LLATTN_VOFF_META 4608    /* attn::VOFF_META */

typedef enum llattn_status {
    LLATTN_OK = 0,
    LLATTN_EINVAL = 1,  /* bad argument (null pointer, negative count, misaligned pointer, index out of range) */
    LLATTN_ECUDA = 2,   /* a CUDA runtime call failed */
    LLATTN_ENOMEM = 3,  /* an allocation failed, or a caller-provided buffer is too small */
    LLATTN_EDEVICE = 4  /* a kernel reported a wait that ran out (see llattn_device_status) */
} llattn_status;

const char* llattn_version(void);
const char* llattn_last_error(void);

/* ---- split policy of the reference, kept for callers that size buffers with it.
 * attn::pick_bpc (engine/attn.cu:361-364) and attn::chunks_for (engine/attn.cu:67). */
int llattn_pick_bpc(int nblocks, int nbatch);
int llattn_chunks_for(int nblocks, int blocks_per_chunk);

/* 32-token blocks per MMA tile of this build (3 or 4). Runs of blocks that start on a multiple of it keep tiles full;
 * any split is correct. No counterpart in the reference. */
int llattn_tile_units(void);

/* ---- block commit.
 * Stands in for attn::kv_commit<<<dim3(4, nb), 128, 0, st>>>(Kf, Vf, cache, max_blocks, blk)
 * (engine/attn.cu:369; call sites engine/engine.cu:591 and :656): block j of Kf/Vf becomes record blk + j of every
 * kv head of `cache`. Output bytes are identical to the reference kernel's. */
int llattn_kv_commit(const void* Kf, const void* Vf, void* cache, int max_blocks, int blk, int nb, void* stream);

/* Same quantiser into a record pool: block j, head h goes to record pages[j * 4 + h] of `pool`
 * (`pages` is a device array of nb * 4 indices). No counterpart in the reference, whose cache is contiguous. */
int llattn_kv_commit_paged(const void* Kf, const void* Vf, void* pool, const int32_t* pages, int nb, void* stream);

/* ---- producer of the attention inputs.
 * Stands in for ops::qk_norm_rope<<<dim3(T, 3), 256, 0, st>>>(qkv, pos, gq, gk, eps, inv_freq, q, k, v)
 * (engine/ops.cu:429-453; call sites engine/engine.cu:427 and :589): per-head RMSNorm of q and k with weights gq/gk
 * [128], RoPE on the first 64 dims at position pos[t] with inv_freq [32] and bf16-rounded cos/sin, v converted;
 * qkv [T][3072] fp32 in; q [T][16][128], k and v [T][4][128] fp16 out. Same arithmetic, same order: bit-identical. */
int llattn_qk_norm_rope(const float* qkv, const int32_t* pos, const float* gq, const float* gk, float eps,
                        const float* inv_freq, void* q, void* k, void* v, int T, void* stream);

/* The same producer for a prefill pass of `nb` whole 32-token blocks (T = 32 nb), fused with their commit: stands in
 * for the pair ops::qk_norm_rope + attn::kv_commit at engine/engine.cu:589-591. q, k, v are written as above (the
 * attention step reads the fresh fp16 K/V), and block j, kv head h also becomes record blk + j of head h of `cache`
 * (pages == NULL), or record pages[j * 4 + h] of the pool `cache` (pages: device array of nb * 4 indices) - quantised
 * from the fp16 values still in shared memory, without reading K/V back. Bytes are identical to running the two
 * reference kernels one after the other. */
int llattn_qkv_prepare_commit(const float* qkv, const int32_t* pos, const float* gq, const float* gk, float eps,
                              const float* inv_freq, void* q, void* k, void* v, int nb, void* cache, const int32_t* pages,
                              int max_blocks, int blk, void* stream);

/* ---- consumer of the attention output: the dense projection on the int8 `Act` the attention epilogue writes.
 * Stands in for Engine::gemm<4, 2>(Ly.dense, items_dense, ..., oA.a, ones, HID, HID, nullptr, h, 1, 2)
 * (engine/engine.cu:434 -> moe8::gemm<4, 4, 2, 2>, engine/moe_i8.cu:295-442) for any number of tokens:
 *   Y[n][r] += sum over the K/128 groups g, ascending, of (s_w[r][g] * s[n][g]) * float(P - z[r][g] * sum[n][g]),
 * P the exact integer dot product of the group's 4-bit weight codes and int8 activations. W: `rows / 16` strips in the
 * reference's device layout (per strip the K/128 code tiles of 1024 bytes, then the K/128 metas of 48 bytes,
 * engine/moe_i8.cu:34-41 after relayout_strips); q [ntokens][K] int8 in fragment order inside every 128-group,
 * s and sum [ntokens][K/128] (the moe8::Act triple, engine/moe_i8.cu:55-66); Y [ntokens][rows] fp32. rows and K are
 * multiples of 128. Same float operations in the same order as the reference kernel: bit-identical results.
 * err_word: device int for a wait that ran out, or NULL. */
int llattn_dense_w4a8(const void* W, const int8_t* q, const float* s, const int32_t* sum, float* Y, int ntokens, int rows, int K,
                      int* err_word, void* stream);

/* ---- the reference operator pair on caller-owned buffers.
 * llattn_args mirrors attn::Args (engine/attn.cu:51-64) field for field. */
typedef struct llattn_args {
    const void* Q;
    const void* Kf;
    const void* Vf;
    const void* cache;
    int max_blocks;
    int nblocks;          /* committed blocks visible to query block 0; block j sees nblocks + j */
    int blocks_per_chunk;
    int nchunks;          /* chunk slots per (query block, kv head) in the partial buffers */
    float scale;          /* 1/sqrt(128) */
    float* Opart;         /* [nb][4][nchunks][128][128] un-normalised */
    float* Mpart;         /* [nb][4][nchunks][128] reference maximum, log2 units */
    float* Lpart;         /* [nb][4][nchunks][128] */
} llattn_args;

/* Stands in for attn::attn_partial<<<dim3(4, nchunks, nb), ATT_NTH, SMEM_BYTES, st>>>(args)
 * (engine/attn.cu:145; call sites engine/engine.cu:431 and :596). `err_word` is a device int the kernel ORs an
 * error code into when a bounded wait runs out (may be NULL). */
int llattn_attn_partial(const llattn_args* args, int nb, int* err_word, void* stream);

/* Stands in for attn::attn_combine<<<dim3(4, 16, nb), 256, 0, st>>>(Opart, Mpart, Lpart, nchunks, nblocks, bpc,
 * O, q8, s8, sum8) (engine/attn.cu:319; call sites engine/engine.cu:432 and :598). With q8 non-null the int8
 * activation form (fragment order, per-head scale, integer sum) is written and O is not, as in the reference. */
int llattn_attn_combine(const float* Opart, const float* Mpart, const float* Lpart, int nchunks, int nblocks,
                        int blocks_per_chunk, void* O, int8_t* q8, float* s8, int32_t* sum8, int nb, void* stream);

/* ---- batched path: many independent sequences, ragged lengths, contiguous or paged caches.
 * No counterpart in the reference (it serves one sequence); each sequence gets exactly what
 * attn_partial + attn_combine give it at engine/engine.cu:429-432 (decode) or :594-598 (prefill). */
typedef struct llattn_ctx llattn_ctx;
typedef struct llattn_plan llattn_plan;

typedef struct llattn_seq {
    const void* cache;     /* device: this layer's cache of the sequence, or the record pool when pages != NULL */
    const int32_t* pages;  /* device: NULL, or [4][head_stride] record indices into the pool */
    int32_t head_stride;   /* contiguous: max_blocks; paged: entries per kv head in `pages` */
    int32_t nblocks;       /* committed blocks visible to the sequence's first query block */
    int32_t nq;            /* query blocks in this call: 1 for a denoising step, up to 16 for a prefill pass */
    int32_t q_first;       /* index of its first query block in Q / Kf / Vf and in the outputs */
} llattn_seq;

typedef struct llattn_io {
    const void* Q;
    const void* Kf;
    const void* Vf;
    void* O16;      /* [nq_total*32][16][128] fp16, or NULL */
    float* O32;     /* same shape fp32, or NULL */
    float* LSE;     /* [nq_total*32][16] natural-log sum of exponentials of the scaled scores, or NULL */
    int8_t* q8;     /* [nq_total*32][2048] int8 activations in fragment order, or NULL (engine/attn.cu:346-357) */
    float* s8;      /* [nq_total*32][16] */
    int32_t* sum8;  /* [nq_total*32][16] */
    float scale;    /* 0 -> 1/sqrt(128) */
    uint32_t flags; /* 0, or LLATTN_IO_PRECISE_P */
    int64_t cache_offset; /* bytes added to every sequence's `cache` pointer in this call (multiple of 16). The layers of a
                             model keep their caches (or record pools) a fixed distance apart (engine/engine.cu:233 allocates
                             one cache per layer, all of one size): one plan then serves all layers of a step, layer l
                             being called with cache_offset = l * (bytes between two layers' caches). 0 for a plan whose
                             `cache` pointers already name the layer. */
} llattn_io;

/* llattn_io.flags. Default (0): the softmax probabilities enter the P.V product as fp16, like the reference kernel's
 * (engine/attn.cu:261-263); a query row that one key partly dominates then carries that key's fp16 rounding (2^-12
 * relative), which at long contexts exceeds 2e-3 of the output RMS on a few elements. LLATTN_IO_PRECISE_P carries every
 * probability as an fp16 value plus an fp16 remainder (two P.V chains per tile): max-abs error against the fp64 oracle
 * stays within 2e-3 of the output RMS at 32 K tokens, at about two thirds of the throughput. No counterpart in the
 * reference. */
#define LLATTN_IO_PRECISE_P 1u

typedef struct llattn_plan_stats {
    int32_t nseq, nq_total, nitems, nslots, nctas;   /* nctas: CTAs that got work (the launch may have more) */
    int64_t total_units;       /* records + fresh blocks over all (query block, kv head) pairs */
    int64_t max_cta_units;     /* units of the busiest CTA */
    size_t workspace_bytes;    /* partial-result scratch the plan needs (owned by the context) */
} llattn_plan_stats;

int llattn_create(int device, llattn_ctx** out);
void llattn_destroy(llattn_ctx* ctx);

/* Builds the work list for `nseq` sequences (host array) and uploads it; allocates, so not for use inside stream
 * capture. `nctas` <= 0, or more than the device has SMs, means one CTA per SM (the CTAs of a launch wait for one
 * another's partial results, so all of them must be resident: one fits on an SM). Every launch of the plan has exactly
 * that many CTAs. With fewer (query block, kv head) tiles than CTAs, each tile is cut into equal runs on CTAs of their
 * own; otherwise the CTAs get contiguous, near-equal shares of the whole unit sequence. A plan that needs
 * more scratch than any earlier plan of the context makes the context reallocate its scratch: CUDA graphs captured with
 * earlier plans then hold stale addresses and must be captured again (create the largest plan first to avoid that). */
int llattn_plan_create(llattn_ctx* ctx, const llattn_seq* seqs_host, int nseq, int nctas, llattn_plan** out);
void llattn_plan_destroy(llattn_plan* plan);
int llattn_plan_get_stats(const llattn_plan* plan, llattn_plan_stats* out);

/* New lengths (and cache / page-table pointers) for an existing plan, without allocation or device synchronisation:
 * the work list is rebuilt on the host into the plan's pinned mirror and copied over the plan's device blob with one
 * cudaMemcpyAsync on `stream`; launches ordered after it on that stream see the new plan. The sequences keep their
 * number and their query-block counts (nq, q_first); contexts may grow or shrink freely. A CUDA graph that captured
 * llattn_attention with this plan stays valid: the kernel reads lengths, work items and tile descriptors from the
 * plan's device memory and its grid does not change, so a committed block needs this one call and no node patching
 * (the reference rewrites the parameters of 40 graph nodes instead, engine/engine.cu:533-562). The only wait is for the
 * previous update's copy to have left the pinned mirror. Not for use inside stream capture (it issues a copy). */
int llattn_plan_update(llattn_plan* plan, const llattn_seq* seqs_host, int nseq, void* stream);

/* The planner alone, on the host (no CUDA call): statistics of the plan llattn_plan_create would build and, when the
 * arrays are given, its work items (8 int32 each: sequence, query block, kv head, first record, record count, fresh
 * flag, partial slot, output tile) and the per-CTA item ranges (nctas + 1 bounds, nctas = the CTAs that got work). For
 * sizing and for host-side tests. */
int llattn_plan_preview(const llattn_seq* seqs_host, int nseq, int nctas, llattn_plan_stats* stats, int32_t* items_out,
                        int max_items, int32_t* cta_first_out, int max_ctas);

/* One attention pass over every sequence of the plan: ONE kernel launch (a cooperative one), no allocation, no host
 * sync. A (query block, kv head) tile that one CTA handles alone is normalised and written by that CTA; a tile spread
 * over n CTAs is folded together by those n CTAs once each has finished all of its own runs: each waits (bounded) for
 * the tile's other partial results in the context's scratch and finishes every n-th row, adding the partial results in
 * a fixed order, so results do not depend on timing. Calls that share a context must not overlap on the GPU. */
int llattn_attention(llattn_ctx* ctx, const llattn_plan* plan, const llattn_io* io, void* stream);

/* Same, with Q/Kf/Vf and the requested outputs in HOST memory (pinned, so the copies are asynchronous). The KV cache
 * stays on the device, as in the reference engine. Consecutive calls are pipelined: a call's inputs go up on the
 * context's own copy stream, its kernels run on `stream`, its outputs come down on a second copy stream, so the upload
 * of one call and the download of the previous one overlap the kernels in between. Host inputs must stay unchanged,
 * and host outputs are complete, only once llattn_host_flush has been ordered on a stream and that stream has reached
 * it. Not for use inside stream capture. */
int llattn_attention_host(llattn_ctx* ctx, const llattn_plan* plan, const llattn_io* io_host, void* stream);

/* Makes `stream` wait for every download llattn_attention_host has issued so far. */
int llattn_host_flush(llattn_ctx* ctx, void* stream);

/* ---- attention without any allocation, for callers that cannot allocate device memory.
 * No counterpart in the reference. Some hosts of this library may not call cudaMalloc at the point where they need
 * attention: an engine whose memory plan is fixed at start-up and audited (every device byte accounted for before the
 * first request), a plugin running inside another runtime's allocator, or code that has already entered a region
 * where allocation is forbidden. This entry point serves them: it takes one sequence (the shape of the reference
 * engine's layer step, engine/engine.cu:429-432 and :594-598: nb query blocks, block j seeing nblocks + j records of
 * `cache` plus its own fresh K/V) and keeps its partial results in an array built into the library image instead of
 * in allocated memory. It creates no context and no plan and calls no allocating routine.
 *   Limits: nb <= 16 query blocks per call; the built-in array is 160 partial slots = 10.16 MiB, held by every GPU
 *   that loads the library until the process exits. Larger requests are refused with LLATTN_EINVAL / LLATTN_ENOMEM.
 *   First call on a device: resolves the array's device address and raises the kernel's shared-memory limit; make
 *   that first call before any stream capture begins.
 *   Sharing: every call on a device uses the same array. Calls whose kernels can overlap on the GPU (different
 *   streams, or concurrent host threads) race on it; issue them on one stream or order them yourself.
 * Outputs as in llattn_io (any of O16, O32, LSE, q8+s8+sum8; at least one). scale 0 means 1/sqrt(128). err_word: device
 * int the kernel ORs an error code into if a bounded wait runs out (may be NULL). */
int llattn_attention_static(const void* Q, const void* Kf, const void* Vf, const void* cache, int max_blocks, int nblocks,
                            int nb, float scale, void* O16, float* O32, float* LSE, int8_t* q8, float* s8, int32_t* sum8,
                            int* err_word, void* stream);

/* ---- page manager with prefix reuse for the record pools of the batched path (host only, no CUDA call).
 * Generalises the reference's single-sequence prefix cache (engine/decode.cu:469-481: committed blocks whose token ids
 * equal the new prompt's leading full blocks are kept) to many sequences over one pool. A page is one committed
 * 32-token block; its record for kv head h of any layer is record `page * 4 + h` of that layer's pool. Sequences that
 * share a prefix of token blocks share its pages; pages of closed sequences stay reusable until their slot is needed
 * (least recently used first). The caller owns the pools, commits the pages reported as not reused and then tells the
 * manager so (llattn_kvpool_mark_committed): only marked pages are ever reported as reused or kept after their last
 * holder closes, so a failed open or a sequence closed before its commit leaves nothing behind that looks committed. */
typedef struct llattn_kvpool llattn_kvpool;
int llattn_kvpool_create(int npages, llattn_kvpool** out);
void llattn_kvpool_destroy(llattn_kvpool* pool);
/* Opens a sequence on a prompt: its ntokens / 32 full blocks get pages (pages_out, in block order, may be NULL);
 * *reused_blocks leading blocks were found committed already and need no prefill. */
int llattn_kvpool_open(llattn_kvpool* pool, const int32_t* tokens, int ntokens, int32_t* seq_id, int32_t* reused_blocks,
                       int32_t* pages_out, int pages_cap);
/* A decoded block of 32 final token ids becomes the sequence's next page (*reused = 1 if an identical continuation
 * was already committed by another sequence). */
int llattn_kvpool_append(llattn_kvpool* pool, int32_t seq_id, const int32_t* block_tokens, int32_t* page_out, int32_t* reused);
/* The records of the sequence's first `nblocks` pages (all of them if nblocks < 0) have been written: from now on
 * other sequences with the same leading blocks get them as reused. Call it once the commit has been ordered on the
 * stream that later readers use. */
int llattn_kvpool_mark_committed(llattn_kvpool* pool, int32_t seq_id, int nblocks);
int llattn_kvpool_pages(llattn_kvpool* pool, int32_t seq_id, int32_t* pages_out, int cap, int32_t* nblocks);
int llattn_kvpool_close(llattn_kvpool* pool, int32_t seq_id);
/* out6 = pages, free, cached (reusable, unreferenced), block hits, block misses, evictions */
int llattn_kvpool_stats(llattn_kvpool* pool, int64_t* out6);

/* Self-test of the bounded waits every kernel here is built on, with nothing made to fail: one CTA whose first four
 * warps wait on barriers that nothing will ever complete and whose fifth waits on a counter nothing counts into (the
 * wait of a CTA for the other runs of a split tile). Warp 0's limit is `limit_ns` (1 ns .. 100 ms); when it runs out
 * the warp raises the CTA's abort flag and the other warps, whose own limit is the kernels' two seconds, leave at their
 * next poll; the fifth warp then waits on its counter once more with `limit_ns` and lets that run out too. The kernel
 * returns normally; `err_word` (device int, zeroed by the caller) then holds bits 1|2|4|8|128 (one per warp: the
 * producer / dequant / MMA / softmax / fold codes of llattn_device_status) and waited_ns6 (device, 6 x uint64) how long
 * each of the five warps waited, then how long the counter wait took to run out alone. No counterpart in the
 * reference, whose kernels have no waits that can fail. */
int llattn_wait_selftest(unsigned long long limit_ns, int* err_word, unsigned long long* waited_ns6, void* stream);

/* Reads (and clears) the context's device error word; synchronises `stream`. 0 = no kernel wait ran out. Bits: 1, 2, 4,
 * 8 a producer / dequant / MMA-issue / softmax warp's wait inside a CTA, 16 the wait for the last MMA at the end of a CTA,
 * 32 a malformed work item, 64 a misaligned shared-memory base, 128 a CTA's wait for the other runs of a tile it shares. */
int llattn_device_status(llattn_ctx* ctx, void* stream, int* code);

#ifdef __cplusplus
}
#endif
#endif /* LLATTN_H */
