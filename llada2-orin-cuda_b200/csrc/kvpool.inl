// Host-side page manager for the record pools of the batched path, with prefix reuse (included by llattn.cu).
//
// The reference keeps one sequence's cache and, between requests, the committed blocks whose token ids equal the new
// prompt's leading full blocks (engine/decode.cu:469-481). This generalises that rule to many sequences over one pool:
// a page is one committed 32-token block of one sequence (its records in every layer and kv head sit at record index
// page * 4 + head of each layer's pool); a page is identified by the chain of token blocks that leads to it, so two
// requests that share a prefix share its pages. Pages of closed sequences stay cached until their slot is needed
// (least recently used first). No CUDA call is made here: the caller owns the pools and runs the commits.
//
// A page counts as reusable only once its records exist: the caller says so with llattn_kvpool_mark_committed after the
// commit kernel has been ordered. Until then a second sequence with the same prefix gets the same page index (it would
// write the same bytes) but is told the block is NOT reused, so it prefills it too; and a page that loses its last
// holder before it was marked goes back to the free list instead of the cache.

#include <list>
#include <unordered_map>

namespace {

struct KvPage {
    uint64_t key = 0;                 // hash of (parent key, 32 token ids); 0 = not registered
    int32_t parent = -1;              // page of the previous block in the chain (-1 for block 0)
    int32_t refs = 0;                 // open sequences that hold it
    int32_t tokens[32];
    bool committed = false;           // its records have been written (llattn_kvpool_mark_committed)
    bool cached = false;              // refs == 0, committed and still registered: in the LRU list
    std::list<int32_t>::iterator lru;
};

inline uint64_t kv_mix(uint64_t h, uint64_t v) {
    h ^= v + 0x9e3779b97f4a7c15ull + (h << 6) + (h >> 2);
    h *= 0xff51afd7ed558ccdull;
    return h ^ (h >> 33);
}
inline uint64_t kv_block_key(uint64_t parent_key, const int32_t* tok) {
    uint64_t h = kv_mix(0x243f6a8885a308d3ull, parent_key);
    for (int i = 0; i < 32; ++i) h = kv_mix(h, uint64_t(uint32_t(tok[i])) + 1);
    return h ? h : 1;
}

}  // namespace

struct llattn_kvpool {
    std::vector<KvPage> pages;
    std::vector<int32_t> free_list;
    std::list<int32_t> lru;                                   // front = least recently used cached page
    std::unordered_multimap<uint64_t, int32_t> by_key;
    std::unordered_map<int32_t, std::vector<int32_t>> seqs;   // open sequence -> its pages in block order
    int32_t next_seq = 1;
    int64_t hits = 0, misses = 0, evictions = 0;
    std::mutex mu;

    int32_t find(uint64_t key, int32_t parent, const int32_t* tok) {
        auto r = by_key.equal_range(key);
        for (auto it = r.first; it != r.second; ++it) {
            const KvPage& pg = pages[it->second];
            if (pg.parent == parent && memcmp(pg.tokens, tok, sizeof(pg.tokens)) == 0) return it->second;
        }
        return -1;
    }
    void unregister(int32_t p) {
        KvPage& pg = pages[p];
        auto r = by_key.equal_range(pg.key);
        for (auto it = r.first; it != r.second; ++it)
            if (it->second == p) { by_key.erase(it); break; }
        pg.key = 0;
    }
    void take(int32_t p) {                                    // a sequence starts holding page p
        KvPage& pg = pages[p];
        if (pg.cached) { lru.erase(pg.lru); pg.cached = false; }
        ++pg.refs;
    }
    void drop(int32_t p) {
        KvPage& pg = pages[p];
        if (--pg.refs == 0) {
            if (pg.key && pg.committed) { pg.lru = lru.insert(lru.end(), p); pg.cached = true; }
            else {                                            // never committed: nothing worth keeping
                if (pg.key) unregister(p);
                pg.committed = false;
                free_list.push_back(p);
            }
        }
    }
    // A page nobody holds: a free one, else the least recently used cached one. A cached page whose children are
    // still registered leaves them unreachable (their parent link no longer matches), which is what eviction means.
    int32_t grab() {
        if (!free_list.empty()) { const int32_t p = free_list.back(); free_list.pop_back(); return p; }
        if (lru.empty()) return -1;
        const int32_t p = lru.front();
        lru.pop_front();
        pages[p].cached = false;
        pages[p].committed = false;
        unregister(p);
        ++evictions;
        return p;
    }
    int32_t add_block(uint64_t parent_key, int32_t parent, const int32_t* tok, bool* reused) {
        const uint64_t key = kv_block_key(parent_key, tok);
        int32_t p = find(key, parent, tok);
        if (p >= 0) {                                         // same chain of blocks: same page; reused only if its records exist
            *reused = pages[p].committed;
            take(p);
            if (*reused) ++hits; else ++misses;
            return p;
        }
        *reused = false;
        p = grab();
        if (p < 0) return -1;
        KvPage& pg = pages[p];
        pg.key = key; pg.parent = parent; pg.refs = 0; pg.committed = false;
        memcpy(pg.tokens, tok, sizeof(pg.tokens));
        by_key.emplace(key, p);
        take(p);
        ++misses;
        return p;
    }
};

extern "C" {

int llattn_kvpool_create(int npages, llattn_kvpool** out) {
    if (!out) return fail(LLATTN_EINVAL, "kvpool_create: null out pointer");
    *out = nullptr;
    if (npages < 1 || npages > (1 << 28)) return fail(LLATTN_EINVAL, "kvpool_create: npages = %d", npages);
    llattn_kvpool* kp = new (std::nothrow) llattn_kvpool();
    if (!kp) return fail(LLATTN_ENOMEM, "kvpool_create: out of host memory");
    kp->pages.resize(size_t(npages));
    kp->free_list.reserve(size_t(npages));
    for (int p = npages - 1; p >= 0; --p) kp->free_list.push_back(p);     // page 0 is handed out first
    *out = kp;
    return LLATTN_OK;
}

void llattn_kvpool_destroy(llattn_kvpool* kp) { delete kp; }

int llattn_kvpool_open(llattn_kvpool* kp, const int32_t* tokens, int ntokens, int32_t* seq_id, int32_t* reused_blocks,
                       int32_t* pages_out, int pages_cap) {
    if (!kp || !seq_id || (ntokens > 0 && !tokens)) return fail(LLATTN_EINVAL, "kvpool_open: null pointer");
    if (ntokens < 0) return fail(LLATTN_EINVAL, "kvpool_open: ntokens = %d", ntokens);
    const int full = ntokens / 32;
    if (pages_out && pages_cap < full) return fail(LLATTN_ENOMEM, "kvpool_open: %d pages, room for %d", full, pages_cap);
    std::lock_guard<std::mutex> lk(kp->mu);
    std::vector<int32_t> mine;
    mine.reserve(size_t(full) + 8);
    uint64_t pkey = 0;
    int32_t parent = -1, reused = 0;
    bool prefix = true;
    for (int b = 0; b < full; ++b) {
        bool hit = false;
        const int32_t p = kp->add_block(pkey, parent, tokens + size_t(b) * 32, &hit);
        if (p < 0) {
            for (int32_t q : mine) kp->drop(q);
            return fail(LLATTN_ENOMEM, "kvpool_open: pool exhausted at block %d of %d (every page is held by an open sequence)", b, full);
        }
        if (hit && prefix) ++reused; else prefix = false;
        mine.push_back(p);
        pkey = kp->pages[p].key;
        parent = p;
    }
    *seq_id = kp->next_seq++;
    if (reused_blocks) *reused_blocks = reused;
    if (pages_out) memcpy(pages_out, mine.data(), mine.size() * sizeof(int32_t));
    kp->seqs.emplace(*seq_id, std::move(mine));
    return LLATTN_OK;
}

int llattn_kvpool_append(llattn_kvpool* kp, int32_t seq_id, const int32_t* block_tokens, int32_t* page_out, int32_t* reused) {
    if (!kp || !block_tokens || !page_out) return fail(LLATTN_EINVAL, "kvpool_append: null pointer");
    std::lock_guard<std::mutex> lk(kp->mu);
    auto it = kp->seqs.find(seq_id);
    if (it == kp->seqs.end()) return fail(LLATTN_EINVAL, "kvpool_append: sequence %d is not open", seq_id);
    std::vector<int32_t>& mine = it->second;
    const int32_t parent = mine.empty() ? -1 : mine.back();
    const uint64_t pkey = parent < 0 ? 0 : kp->pages[parent].key;
    bool hit = false;
    const int32_t p = kp->add_block(pkey, parent, block_tokens, &hit);
    if (p < 0) return fail(LLATTN_ENOMEM, "kvpool_append: pool exhausted (every page is held by an open sequence)");
    mine.push_back(p);
    *page_out = p;
    if (reused) *reused = hit ? 1 : 0;
    return LLATTN_OK;
}

int llattn_kvpool_mark_committed(llattn_kvpool* kp, int32_t seq_id, int nblocks) {
    if (!kp) return fail(LLATTN_EINVAL, "kvpool_mark_committed: null pool");
    std::lock_guard<std::mutex> lk(kp->mu);
    auto it = kp->seqs.find(seq_id);
    if (it == kp->seqs.end()) return fail(LLATTN_EINVAL, "kvpool_mark_committed: sequence %d is not open", seq_id);
    const int have = int(it->second.size());
    if (nblocks > have) return fail(LLATTN_EINVAL, "kvpool_mark_committed: %d blocks, the sequence has %d", nblocks, have);
    const int n = nblocks < 0 ? have : nblocks;
    for (int b = 0; b < n; ++b) kp->pages[it->second[b]].committed = true;
    return LLATTN_OK;
}

int llattn_kvpool_pages(llattn_kvpool* kp, int32_t seq_id, int32_t* pages_out, int cap, int32_t* nblocks) {
    if (!kp || !nblocks) return fail(LLATTN_EINVAL, "kvpool_pages: null pointer");
    std::lock_guard<std::mutex> lk(kp->mu);
    auto it = kp->seqs.find(seq_id);
    if (it == kp->seqs.end()) return fail(LLATTN_EINVAL, "kvpool_pages: sequence %d is not open", seq_id);
    *nblocks = int32_t(it->second.size());
    if (pages_out) {
        if (cap < *nblocks) return fail(LLATTN_ENOMEM, "kvpool_pages: %d pages, room for %d", *nblocks, cap);
        memcpy(pages_out, it->second.data(), it->second.size() * sizeof(int32_t));
    }
    return LLATTN_OK;
}

int llattn_kvpool_close(llattn_kvpool* kp, int32_t seq_id) {
    if (!kp) return fail(LLATTN_EINVAL, "kvpool_close: null pool");
    std::lock_guard<std::mutex> lk(kp->mu);
    auto it = kp->seqs.find(seq_id);
    if (it == kp->seqs.end()) return fail(LLATTN_EINVAL, "kvpool_close: sequence %d is not open", seq_id);
    // children first, so that the least recently used end of the list holds the deepest blocks
    for (auto p = it->second.rbegin(); p != it->second.rend(); ++p) kp->drop(*p);
    kp->seqs.erase(it);
    return LLATTN_OK;
}

int llattn_kvpool_stats(llattn_kvpool* kp, int64_t* out6) {
    if (!kp || !out6) return fail(LLATTN_EINVAL, "kvpool_stats: null pointer");
    std::lock_guard<std::mutex> lk(kp->mu);
    out6[0] = int64_t(kp->pages.size());
    out6[1] = int64_t(kp->free_list.size());
    out6[2] = int64_t(kp->lru.size());
    out6[3] = kp->hits;
    out6[4] = kp->misses;
    out6[5] = kp->evictions;
    return LLATTN_OK;
}

}  // extern "C"
