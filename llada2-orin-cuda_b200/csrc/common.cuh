// Constants of the "4c/4" KV record (engine/attn.cu:3-7,22-25 of the reference) and the plain structs the host
// planner and the kernels share.
#pragma once
#include <cstdint>

namespace llattn {

constexpr int D = 128;            // head dim
constexpr int BLK = 32;           // tokens per block
constexpr int NKV = 4;            // kv heads
constexpr int NQH = 16;           // query heads
constexpr int QR = 128;           // query rows per kv head: 32 tokens x 4 GQA heads, row r = token r/4, head 4*kvh + r%4
constexpr int REC_BYTES = 4736;   // one record = one (kv head, 32-token block)
constexpr int KOFF_META = 2048;   // K scale fp16[128], then K min fp16[128]
constexpr int VOFF = 2560;        // V codes
constexpr int VOFF_META = 4608;   // V scale fp16[32], then V min fp16[32]

// One sequence as the kernels see it (device memory).
struct SeqDesc {
    const uint8_t* cache;     // contiguous: this layer's [4][head_stride][4736]; paged: the record pool
    const int32_t* pages;     // null, or [4][head_stride] record indices into the pool
    int32_t head_stride;      // records (or page-table entries) per kv head
    int32_t nblocks;          // committed blocks visible to query block 0; query block j sees nblocks + j
    int32_t nq;               // query blocks of this sequence in this call
    int32_t q_first;          // index of its first query block in the Q / Kf / Vf / output arrays
};

// One contiguous run of KV units (records, then optionally the fresh block) of one (sequence, query block, kv head).
struct WorkItem {
    int32_t seq;
    int32_t qblk;             // query block within the sequence
    int32_t kvh;
    int32_t rec_begin;        // first record of the run
    int32_t rec_count;        // records in the run
    int32_t fresh;            // 1: the query block's own fp16 K/V follow the records
    int32_t slot;             // partial-result slot this run writes
    int32_t tile;             // output tile (query block x kv head) the run belongs to: index of its MergeDesc
};

// What the kernel reads per run: the run and its sequence side by side, 64 bytes, so that a CTA reaches everything about
// its first run with two dependent loads (its item range, then this) instead of three.
struct alignas(16) RunDesc {
    WorkItem w;
    SeqDesc s;
};
static_assert(sizeof(RunDesc) == 64, "RunDesc layout");

// One output tile (query block x kv head) and the partial slots that make it up.
struct MergeDesc {
    int32_t q_index;          // global query block index (q_first + qblk)
    int32_t kvh;
    int32_t slot_begin;
    int32_t nslots;
};

// Device error word bits (set by a kernel whose bounded wait ran out, or whose shared-memory base is not aligned).
enum : int {
    ERR_WAIT_PRODUCER = 1, ERR_WAIT_DEQUANT = 2, ERR_WAIT_MMA = 4, ERR_WAIT_SOFTMAX = 8, ERR_WAIT_TEARDOWN = 16,
    ERR_BAD_ITEM = 32, ERR_SMEM_ALIGN = 64, ERR_WAIT_FOLD = 128
};

}  // namespace llattn
