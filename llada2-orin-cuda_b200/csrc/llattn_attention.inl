// Attention entry points of the C ABI (included at the end of llattn.cu): the reference-shaped operator pair, the
// context, the host-side work planner and the batched launches.

namespace {

constexpr size_t SLOT_O_BYTES = size_t(llattn::QR) * llattn::D * sizeof(float);   // 64 KiB
constexpr size_t SLOT_ML_BYTES = size_t(llattn::QR) * sizeof(float);
// The scratch starts with the arrival counters of the fused merge (4 per output tile, all zero between launches: the run
// that completes a tile puts its counter back), then the partial slots.
constexpr int COUNTER_TILES = 16384;
constexpr size_t COUNTER_BYTES = size_t(COUNTER_TILES) * 4 * sizeof(int);

int grow_workspace(llattn_ctx* c, size_t need) {
    if (need <= c->workspace_bytes) return LLATTN_OK;
    if (int rc = grow(&c->workspace, &c->workspace_bytes, need)) return rc;
    CU(cudaMemset(c->workspace, 0, COUNTER_BYTES));
    return LLATTN_OK;
}

// Splits the flattened unit sequence (every (sequence, query block, kv head) tile contributes nblocks + j records and
// one fresh block, in that order) into `nctas` contiguous shares of near-equal size. A share boundary inside a tile
// falls on a multiple of 4 units from the tile's start so that 128-key MMA tiles stay full, and a run is never
// shorter than `min_units` unless the tile itself is. Every run gets its own partial slot; the slots of one tile are
// consecutive. When there are no more output tiles than CTAs the tiles are cut one by one instead (see build_plan).
struct HostPlan {
    std::vector<llattn::SeqDesc> seqs;
    std::vector<llattn::WorkItem> items;
    std::vector<int32_t> cta_first;
    std::vector<llattn::MergeDesc> merge;
    int64_t total_units = 0, max_cta_units = 0, max_cta_cost = 0;
    int nq_total = 0, used_ctas = 0;
};

// What a CTA's list costs, in the time of a unit (about a third of a microsecond): its units, a start-up charge per run
// (query load, first records, the pipeline filling up, the epilogue), and for a run of a split tile the partial result's
// round trip through the L2 and its share of the folding.
constexpr int64_t RUN_STARTUP_UNITS = 20, RUN_SPLIT_UNITS = 4;
// A piece of a tile shorter than this is not worth a run of its own: the cut moves to the tile's end (or start) instead.
constexpr int SHORTEST_PIECE = 12;

void finish_plan(HostPlan& hp, int nctas) {
    if (hp.cta_first.back() != int32_t(hp.items.size())) hp.cta_first.push_back(int32_t(hp.items.size()));
    hp.used_ctas = int(hp.cta_first.size()) - 1;
    // the launch always has `nctas` CTAs (a captured graph keeps its grid when the plan is updated): the rest get no items
    while (int(hp.cta_first.size()) < nctas + 1) hp.cta_first.push_back(int32_t(hp.items.size()));
    hp.max_cta_units = hp.max_cta_cost = 0;
    for (size_t c = 0; c + 1 < hp.cta_first.size(); ++c) {
        int64_t u = 0;
        for (int i = hp.cta_first[c]; i < hp.cta_first[c + 1]; ++i) u += hp.items[i].rec_count + hp.items[i].fresh;
        hp.max_cta_units = std::max(hp.max_cta_units, u);
        int64_t cost = u;
        for (int i = hp.cta_first[c]; i < hp.cta_first[c + 1]; ++i)
            cost += RUN_STARTUP_UNITS + (hp.merge[hp.items[i].tile].nslots > 1 ? RUN_SPLIT_UNITS : 0);
        hp.max_cta_cost = std::max(hp.max_cta_cost, cost);
    }
}

// Contiguous shares of the flattened unit sequence (see above).
void cut_contiguous(const llattn_seq* seqs, int nseq, int nctas, int64_t total, int64_t MIN_UNITS, HostPlan& hp) {
    using namespace llattn;
    // The share of the CTA being filled is re-derived from what is left (units and CTAs), so rounding a cut down to a
    // tile boundary never pushes work into an extra CTA: the plan uses at most `nctas` CTAs.
    int64_t left = total;
    int ctas_left = nctas;
    auto new_share = [&]() -> int64_t {
        int64_t sh = ctas_left > 1 ? (left + ctas_left - 1) / ctas_left : left;
        sh = std::max<int64_t>(sh, MIN_UNITS);
        return (sh + TILE_UNITS - 1) / TILE_UNITS * TILE_UNITS;
    };
    hp.cta_first.assign(1, 0);
    int64_t room = new_share();      // units the current CTA can still take
    int slot = 0;
    auto next_cta = [&]() {
        hp.cta_first.push_back(int32_t(hp.items.size()));
        if (ctas_left > 1) --ctas_left;
        room = new_share();
    };
    for (int s = 0; s < nseq; ++s)
        for (int j = 0; j < seqs[s].nq; ++j)
            for (int h = 0; h < NKV; ++h) {
                const int nrec = seqs[s].nblocks + j;
                const int U = nrec + 1;
                int done = 0;
                const int slot0 = slot, tile = int(hp.merge.size());
                while (done < U) {
                    int take = int(std::min<int64_t>(room, U - done));
                    if (take < U - done) {
                        take = take / TILE_UNITS * TILE_UNITS;                      // keep the cut on a tile boundary
                        if (U - done - take < SHORTEST_PIECE) take = U - done;      // no short tail for the next CTA
                        else if (take < SHORTEST_PIECE && int(hp.items.size()) > hp.cta_first.back()) take = 0;   // no short head here
                    }
                    if (take == 0) { next_cta(); continue; }
                    const int rec_cnt = std::min(take, nrec - done);
                    hp.items.push_back(WorkItem{s, j, h, done, std::max(rec_cnt, 0), done + take == U ? 1 : 0, slot++, tile});
                    done += take;
                    room -= take;
                    left -= take;
                    if (room <= 0 && left > 0) next_cta();
                }
                hp.merge.push_back(MergeDesc{seqs[s].q_first + j, h, slot0, slot - slot0});
            }
    finish_plan(hp, nctas);
}

// Every run on a CTA of its own: each output tile is cut into equal runs, their number in proportion to the tile's
// length (and no run shorter than about 0.75 sqrt(units of the tile)). Possible when there are no more output tiles than CTAs; better
// than contiguous shares when the step is a latency problem (a handful of sequences), because no CTA then pays the
// start-up of two runs one after the other.
void cut_per_tile(const llattn_seq* seqs, int nseq, int nctas, int64_t total, HostPlan& hp) {
    using namespace llattn;
    std::vector<int> runs;
    int64_t given = 0;
    for (int s = 0; s < nseq; ++s)
        for (int j = 0; j < seqs[s].nq; ++j)
            for (int h = 0; h < NKV; ++h) {
                const int64_t U = seqs[s].nblocks + j + 1;
                // a run costs about a unit's time per unit plus a bit over half a unit per run of its tile (its partial
                // result is written, waited for and read back): the sum is smallest near 0.75 sqrt(U) units per run
                // (measured: 8 units at 2 K tokens, 12 at 8 K)
                const int64_t shortest = std::max<int64_t>(2 * TILE_UNITS, int64_t(0.75 * std::sqrt(double(U)) + 0.5));
                const int64_t by_share = U * nctas / total, by_length = (U + shortest - 1) / shortest;
                runs.push_back(int(std::max<int64_t>(1, std::min(by_share, by_length))));
                given += runs.back();
            }
    while (given > nctas) {                       // only when many tiles were rounded up to one run
        auto it = std::max_element(runs.begin(), runs.end());
        --*it; --given;
    }
    hp.cta_first.assign(1, 0);
    int slot = 0, t = 0;
    for (int s = 0; s < nseq; ++s)
        for (int j = 0; j < seqs[s].nq; ++j)
            for (int h = 0; h < NKV; ++h, ++t) {
                const int nrec = seqs[s].nblocks + j, U = nrec + 1, slot0 = slot;
                const int per = std::max(TILE_UNITS, ((U + runs[t] - 1) / runs[t] + TILE_UNITS - 1) / TILE_UNITS * TILE_UNITS);
                for (int done = 0; done < U; done += per) {
                    const int take = std::min(per, U - done);
                    hp.items.push_back(WorkItem{s, j, h, done, std::max(std::min(take, nrec - done), 0), done + take == U ? 1 : 0, slot++, t});
                    hp.cta_first.push_back(int32_t(hp.items.size()));
                }
                hp.merge.push_back(MergeDesc{seqs[s].q_first + j, h, slot0, slot - slot0});
            }
    finish_plan(hp, nctas);
}

int build_plan(const llattn_seq* seqs, int nseq, int nctas, HostPlan& hp) {
    using namespace llattn;
    hp.seqs.resize(nseq);
    int64_t total = 0, ntile_out = 0;
    int nq_total = 0;
    for (int s = 0; s < nseq; ++s) {
        const llattn_seq& q = seqs[s];
        if (!q.cache && q.nblocks + q.nq - 1 > 0) return fail(LLATTN_EINVAL, "plan: sequence %d has a null cache", s);
        if (q.nblocks < 0 || q.nq < 1 || q.q_first < 0 || q.head_stride < 0)
            return fail(LLATTN_EINVAL, "plan: sequence %d has a negative count (nblocks %d, nq %d, q_first %d)", s, q.nblocks, q.nq, q.q_first);
        if (q.nblocks + q.nq - 1 > q.head_stride)
            return fail(LLATTN_EINVAL, "plan: sequence %d reads %d blocks but head_stride is %d", s, q.nblocks + q.nq - 1, q.head_stride);
        if (q.cache && !aligned16(q.cache)) return fail(LLATTN_EINVAL, "plan: sequence %d cache is not 16-byte aligned", s);
        hp.seqs[s] = SeqDesc{static_cast<const uint8_t*>(q.cache), q.pages, q.head_stride, q.nblocks, q.nq, q.q_first};
        for (int j = 0; j < q.nq; ++j) total += int64_t(NKV) * (q.nblocks + j + 1);
        ntile_out += int64_t(NKV) * q.nq;
        nq_total = std::max(nq_total, q.q_first + q.nq);
    }
    hp.total_units = total;
    hp.nq_total = nq_total;
    auto take_if_cheaper = [&](HostPlan& alt) {
        if (alt.max_cta_cost < hp.max_cta_cost) {
            hp.items.swap(alt.items); hp.cta_first.swap(alt.cta_first); hp.merge.swap(alt.merge);
            hp.used_ctas = alt.used_ctas; hp.max_cta_units = alt.max_cta_units; hp.max_cta_cost = alt.max_cta_cost;
        }
    };
    cut_contiguous(seqs, nseq, nctas, total, 16, hp);
    if (total < 16 * int64_t(nctas)) {       // little work: shorter shares on more CTAs may beat several runs per CTA
        HostPlan alt;
        cut_contiguous(seqs, nseq, nctas, total, TILE_UNITS, alt);
        take_if_cheaper(alt);
    }
    if (ntile_out <= nctas) {
        HostPlan alt;
        cut_per_tile(seqs, nseq, nctas, total, alt);
        take_if_cheaper(alt);
    }
    return LLATTN_OK;
}

int check_io(const llattn_io* io, const char* who) {
    if (!io || !io->Q || !io->Kf || !io->Vf) return fail(LLATTN_EINVAL, "%s: Q, Kf and Vf are required", who);
    if (!io->O16 && !io->O32 && !io->q8 && !io->LSE) return fail(LLATTN_EINVAL, "%s: no output requested", who);
    if (io->q8 && (!io->s8 || !io->sum8)) return fail(LLATTN_EINVAL, "%s: q8 needs s8 and sum8", who);
    if (io->flags & ~uint32_t(LLATTN_IO_PRECISE_P)) return fail(LLATTN_EINVAL, "%s: unknown flag bits 0x%x", who, io->flags);
    return LLATTN_OK;
}

}  // namespace

extern "C" {

// ----------------------------------------------------------------------------- the reference operator pair

int llattn_attn_partial(const llattn_args* a, int nb, int* err_word, void* stream) {
    using namespace llattn;
    if (!a || !a->Q || !a->Kf || !a->Vf || !a->Opart || !a->Mpart || !a->Lpart) return fail(LLATTN_EINVAL, "attn_partial: null pointer");
    if (nb < 1 || a->nblocks < 0 || a->blocks_per_chunk < 1 || a->nchunks < 1)
        return fail(LLATTN_EINVAL, "attn_partial: bad shape (nb %d, nblocks %d, bpc %d, nchunks %d)", nb, a->nblocks, a->blocks_per_chunk, a->nchunks);
    if (a->nblocks + nb - 1 > 0 && !a->cache) return fail(LLATTN_EINVAL, "attn_partial: null cache with committed blocks");
    if (a->nblocks + nb - 1 > a->max_blocks) return fail(LLATTN_EINVAL, "attn_partial: %d blocks visible, cache holds %d", a->nblocks + nb - 1, a->max_blocks);
    if (llattn_chunks_for(a->nblocks + nb - 1, a->blocks_per_chunk) > a->nchunks)
        return fail(LLATTN_EINVAL, "attn_partial: %d chunks needed, %d slots given", llattn_chunks_for(a->nblocks + nb - 1, a->blocks_per_chunk), a->nchunks);
    if (!aligned16(a->Q) || !aligned16(a->Kf) || !aligned16(a->Vf) || !aligned16(a->cache) || !aligned16(a->Opart))
        return fail(LLATTN_EINVAL, "attn_partial: pointers must be 16-byte aligned");
    if (int rc = ensure_kernel_attrs()) return rc;
    KParams p{};
    p.Q = static_cast<const half*>(a->Q); p.Kf = static_cast<const half*>(a->Kf); p.Vf = static_cast<const half*>(a->Vf);
    p.Opart = a->Opart; p.Mpart = a->Mpart; p.Lpart = a->Lpart;
    p.sl2 = a->scale * 1.4426950408889634f;
    p.err = err_word;
    p.ref_seq = SeqDesc{static_cast<const uint8_t*>(a->cache), nullptr, a->max_blocks, a->nblocks, nb, 0};
    p.ref_bpc = a->blocks_per_chunk;
    p.ref_nchunks = a->nchunks;
    attn_tile_kernel<false><<<NKV * a->nchunks * nb, ATTN_THREADS, ATTN_SMEM_BYTES, as_stream(stream)>>>(p);
    CU(cudaGetLastError());
    return LLATTN_OK;
}

int llattn_attn_combine(const float* Opart, const float* Mpart, const float* Lpart, int nchunks, int nblocks, int bpc,
                        void* O, int8_t* q8, float* s8, int32_t* sum8, int nb, void* stream) {
    using namespace llattn;
    if (!Opart || !Mpart || !Lpart) return fail(LLATTN_EINVAL, "attn_combine: null partial buffer");
    if (!O && !q8) return fail(LLATTN_EINVAL, "attn_combine: neither O nor q8 given");
    if (q8 && (!s8 || !sum8)) return fail(LLATTN_EINVAL, "attn_combine: q8 needs s8 and sum8");
    if (nb < 1 || nchunks < 1 || bpc < 1 || nblocks < 0) return fail(LLATTN_EINVAL, "attn_combine: bad shape");
    MergeOut o{};
    if (q8) { o.q8 = q8; o.s8 = s8; o.sum8 = sum8; }       // as the reference: int8 form replaces the fp16 output
    else o.O16 = static_cast<half*>(O);
    combine_ref_kernel<<<dim3(NKV, QR / MERGE_ROWS, nb), MERGE_THREADS, 0, as_stream(stream)>>>(Opart, Mpart, Lpart, nchunks, nblocks, bpc, o);
    CU(cudaGetLastError());
    return LLATTN_OK;
}

// ----------------------------------------------------------------------------- context

int llattn_create(int device, llattn_ctx** out) {
    if (!out) return fail(LLATTN_EINVAL, "create: null out pointer");
    *out = nullptr;
    int ndev = 0;
    CU(cudaGetDeviceCount(&ndev));
    if (device < 0 || device >= ndev) return fail(LLATTN_EINVAL, "create: device %d of %d", device, ndev);
    DeviceGuard g(device);
    if (!g.ok) return fail(LLATTN_ECUDA, "create: cannot select device %d", device);
    cudaDeviceProp prop;
    CU(cudaGetDeviceProperties(&prop, device));
    if (prop.major != 10) return fail(LLATTN_ECUDA, "create: device %d is sm_%d%d; this library holds sm_100a code only", device, prop.major, prop.minor);
    llattn_ctx* c = new (std::nothrow) llattn_ctx();
    if (!c) return fail(LLATTN_ENOMEM, "create: out of host memory");
    c->device = device;
    c->num_sms = prop.multiProcessorCount;
    if (cudaMalloc(&c->err_word, sizeof(int)) != cudaSuccess || cudaMemset(c->err_word, 0, sizeof(int)) != cudaSuccess) {
        cudaGetLastError();
        delete c;
        return fail(LLATTN_ENOMEM, "create: cannot allocate the device error word");
    }
    if (int rc = ensure_kernel_attrs()) { cudaFree(c->err_word); delete c; return rc; }
    // the largest grid a cooperative launch of the attention kernel accepts here: what fits on the device at once (fewer
    // than one CTA per SM when the process was given only a part of the GPU)
    int per_sm = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, llattn::attn_tile_kernel<true>, llattn::ATTN_THREADS, llattn::ATTN_SMEM_BYTES) != cudaSuccess || per_sm < 1) {
        cudaGetLastError();
        cudaFree(c->err_word);
        delete c;
        return fail(LLATTN_ECUDA, "create: the attention kernel does not fit on an SM of device %d", device);
    }
    *out = c;
    return LLATTN_OK;
}

void llattn_destroy(llattn_ctx* c) {
    if (!c) return;
    DeviceGuard g(c->device);
    cudaFree(c->err_word);
    cudaFree(c->workspace);
    cudaFree(c->stage);
    if (c->host_ready) {
        cudaStreamDestroy(c->s_in);
        cudaStreamDestroy(c->s_out);
        for (int i = 0; i < 2; ++i) { cudaEventDestroy(c->ev_in[i]); cudaEventDestroy(c->ev_comp[i]); cudaEventDestroy(c->ev_out[i]); }
    }
    delete c;
}

namespace {

inline size_t up256(size_t x) { return (x + 255) / 256 * 256; }

void fill_stats(llattn_plan* pl, const HostPlan& hp, int nseq) {
    pl->stats.nseq = nseq;
    pl->stats.nq_total = hp.nq_total;
    pl->stats.nitems = int32_t(hp.items.size());
    pl->stats.nslots = int32_t(hp.items.size());
    pl->stats.nctas = hp.used_ctas;
    pl->stats.total_units = hp.total_units;
    pl->stats.max_cta_units = hp.max_cta_units;
}

// Lays the host plan out in the plan's pinned mirror (section offsets are fixed by the capacities chosen at creation).
int stage_plan(llattn_plan* pl, const HostPlan& hp) {
    if (hp.seqs.size() > pl->cap_seqs || hp.items.size() > pl->cap_items || hp.merge.size() > pl->cap_tiles ||
        hp.cta_first.size() != size_t(pl->launch_ctas) + 1)
        return fail(LLATTN_ENOMEM, "plan: %zu sequences, %zu runs, %zu tiles; the plan was created for %zu, %zu, %zu",
                    hp.seqs.size(), hp.items.size(), hp.merge.size(), pl->cap_seqs, pl->cap_items, pl->cap_tiles);
    uint8_t* h = static_cast<uint8_t*>(pl->host_blob);
    memcpy(h + pl->off_seqs, hp.seqs.data(), hp.seqs.size() * sizeof(llattn::SeqDesc));
    llattn::RunDesc* runs = reinterpret_cast<llattn::RunDesc*>(h + pl->off_items);
    for (size_t i = 0; i < hp.items.size(); ++i) runs[i] = llattn::RunDesc{hp.items[i], hp.seqs[hp.items[i].seq]};
    memcpy(h + pl->off_cta, hp.cta_first.data(), hp.cta_first.size() * sizeof(int32_t));
    memcpy(h + pl->off_merge, hp.merge.data(), hp.merge.size() * sizeof(llattn::MergeDesc));
    return LLATTN_OK;
}

}  // namespace

int llattn_plan_create(llattn_ctx* c, const llattn_seq* seqs, int nseq, int nctas, llattn_plan** out) {
    using namespace llattn;
    if (!c || !seqs || !out) return fail(LLATTN_EINVAL, "plan_create: null pointer");
    *out = nullptr;
    if (nseq < 1) return fail(LLATTN_EINVAL, "plan_create: nseq must be positive");
    // One CTA fits on an SM, and a CTA waits (bounded) for the other runs of the tiles it shares: every CTA of the launch
    // must be on an SM at the same time, so the grid never exceeds the SM count (the launch is a cooperative one).
    if (nctas <= 0 || nctas > c->num_sms) nctas = c->num_sms;
    nctas = std::min(nctas, llattn::FOLD_MAX_SLOTS);       // a tile has at most one run per CTA, and the folding holds that many
    HostPlan hp;
    if (int rc = build_plan(seqs, nseq, nctas, hp)) return rc;
    if (hp.merge.size() > COUNTER_TILES) return fail(LLATTN_EINVAL, "plan_create: %zu output tiles, at most %d per call", hp.merge.size(), COUNTER_TILES);
    std::lock_guard<std::mutex> lk(c->mu);
    DeviceGuard g(c->device);
    if (!g.ok) return fail(LLATTN_ECUDA, "plan_create: cannot select device %d", c->device);
    llattn_plan* pl = new (std::nothrow) llattn_plan();
    if (!pl) return fail(LLATTN_ENOMEM, "plan_create: out of host memory");
    pl->ctx = c;
    pl->launch_ctas = nctas;
    // Capacities: a later llattn_plan_update may change every length, as long as the sequences keep their number and
    // their query-block counts. A tile is cut at most once per CTA boundary, so tiles + CTAs bounds the runs.
    pl->cap_seqs = hp.seqs.size();
    pl->cap_tiles = hp.merge.size();
    pl->cap_items = hp.merge.size() + size_t(nctas);
    pl->off_seqs = 0;
    pl->off_items = pl->off_seqs + up256(pl->cap_seqs * sizeof(SeqDesc));
    pl->off_cta = pl->off_items + up256(pl->cap_items * sizeof(RunDesc));
    pl->off_merge = pl->off_cta + up256((size_t(nctas) + 1) * sizeof(int32_t));
    pl->blob_bytes = pl->off_merge + up256(pl->cap_tiles * sizeof(MergeDesc));
    auto bail = [&](int code, const char* what) {
        if (pl->dev_blob) cudaFree(pl->dev_blob);
        if (pl->host_blob) cudaFreeHost(pl->host_blob);
        if (pl->ev_upload) cudaEventDestroy(pl->ev_upload);
        cudaGetLastError();
        delete pl;
        return fail(code, "plan_create: %s", what);
    };
    if (cudaMalloc(&pl->dev_blob, pl->blob_bytes) != cudaSuccess) return bail(LLATTN_ENOMEM, "cudaMalloc of the plan failed");
    if (cudaMallocHost(&pl->host_blob, pl->blob_bytes) != cudaSuccess) return bail(LLATTN_ENOMEM, "cudaMallocHost of the plan mirror failed");
    if (cudaEventCreateWithFlags(&pl->ev_upload, cudaEventDisableTiming) != cudaSuccess) return bail(LLATTN_ECUDA, "cudaEventCreate failed");
    memset(pl->host_blob, 0, pl->blob_bytes);
    if (int rc = stage_plan(pl, hp)) { bail(rc, "internal"); return rc; }
    if (cudaMemcpy(pl->dev_blob, pl->host_blob, pl->blob_bytes, cudaMemcpyHostToDevice) != cudaSuccess) return bail(LLATTN_ECUDA, "upload failed");
    const uint8_t* d = static_cast<const uint8_t*>(pl->dev_blob);
    pl->d_seqs = reinterpret_cast<const SeqDesc*>(d + pl->off_seqs);
    pl->d_items = reinterpret_cast<const RunDesc*>(d + pl->off_items);
    pl->d_cta_first = reinterpret_cast<const int32_t*>(d + pl->off_cta);
    pl->d_merge = reinterpret_cast<const MergeDesc*>(d + pl->off_merge);
    fill_stats(pl, hp, nseq);
    // the scratch is sized for the most runs any update can bring, so that an update never allocates
    pl->stats.workspace_bytes = COUNTER_BYTES + pl->cap_items * (SLOT_O_BYTES + 2 * SLOT_ML_BYTES);
    if (int rc = grow_workspace(c, pl->stats.workspace_bytes)) { bail(rc, "workspace"); return rc; }
    *out = pl;
    return LLATTN_OK;
}

int llattn_plan_update(llattn_plan* pl, const llattn_seq* seqs, int nseq, void* stream) {
    using namespace llattn;
    if (!pl || !seqs) return fail(LLATTN_EINVAL, "plan_update: null pointer");
    if (size_t(nseq) != pl->cap_seqs) return fail(LLATTN_EINVAL, "plan_update: %d sequences, the plan was created for %zu", nseq, pl->cap_seqs);
    HostPlan hp;
    if (int rc = build_plan(seqs, nseq, pl->launch_ctas, hp)) return rc;
    // the pinned mirror is reused: the previous update's copy must have left it (a wait on a finished copy, not on kernels)
    if (pl->upload_pending) { CU(cudaEventSynchronize(pl->ev_upload)); pl->upload_pending = false; }
    if (int rc = stage_plan(pl, hp)) return rc;
    CU(cudaMemcpyAsync(pl->dev_blob, pl->host_blob, pl->blob_bytes, cudaMemcpyHostToDevice, as_stream(stream)));
    CU(cudaEventRecord(pl->ev_upload, as_stream(stream)));
    pl->upload_pending = true;
    const size_t ws = pl->stats.workspace_bytes;
    fill_stats(pl, hp, nseq);
    pl->stats.workspace_bytes = ws;
    return LLATTN_OK;
}

int llattn_plan_preview(const llattn_seq* seqs, int nseq, int nctas, llattn_plan_stats* stats, int32_t* items_out,
                        int max_items, int32_t* cta_first_out, int max_ctas) {
    using namespace llattn;
    if (!seqs || !stats) return fail(LLATTN_EINVAL, "plan_preview: null pointer");
    if (nseq < 1 || nctas < 1) return fail(LLATTN_EINVAL, "plan_preview: nseq and nctas must be positive");
    HostPlan hp;
    if (int rc = build_plan(seqs, nseq, nctas, hp)) return rc;
    memset(stats, 0, sizeof(*stats));
    stats->nseq = nseq;
    stats->nq_total = hp.nq_total;
    stats->nitems = stats->nslots = int32_t(hp.items.size());
    stats->nctas = hp.used_ctas;
    stats->total_units = hp.total_units;
    stats->max_cta_units = hp.max_cta_units;
    stats->workspace_bytes = COUNTER_BYTES + (hp.merge.size() + size_t(nctas)) * (SLOT_O_BYTES + 2 * SLOT_ML_BYTES);
    if (items_out) {
        if (max_items < int(hp.items.size())) return fail(LLATTN_ENOMEM, "plan_preview: %zu items, room for %d", hp.items.size(), max_items);
        memcpy(items_out, hp.items.data(), hp.items.size() * sizeof(WorkItem));
    }
    if (cta_first_out) {
        if (max_ctas < hp.used_ctas) return fail(LLATTN_ENOMEM, "plan_preview: %d CTAs, room for %d", hp.used_ctas, max_ctas);
        memcpy(cta_first_out, hp.cta_first.data(), (size_t(hp.used_ctas) + 1) * sizeof(int32_t));
    }
    return LLATTN_OK;
}

void llattn_plan_destroy(llattn_plan* pl) {
    if (!pl) return;
    DeviceGuard g(pl->ctx->device);
    if (pl->upload_pending) cudaEventSynchronize(pl->ev_upload);
    cudaFree(pl->dev_blob);
    cudaFreeHost(pl->host_blob);
    cudaEventDestroy(pl->ev_upload);
    delete pl;
}

int llattn_plan_get_stats(const llattn_plan* pl, llattn_plan_stats* out) {
    if (!pl || !out) return fail(LLATTN_EINVAL, "plan_get_stats: null pointer");
    *out = pl->stats;
    return LLATTN_OK;
}

int llattn_attention(llattn_ctx* c, const llattn_plan* pl, const llattn_io* io, void* stream) {
    using namespace llattn;
    if (!c || !pl || pl->ctx != c) return fail(LLATTN_EINVAL, "attention: plan does not belong to this context");
    if (int rc = check_io(io, "attention")) return rc;
    if (!aligned16(io->Q) || !aligned16(io->Kf) || !aligned16(io->Vf) || !aligned16(io->O16) || !aligned16(io->O32))
        return fail(LLATTN_EINVAL, "attention: pointers must be 16-byte aligned");
    if (io->cache_offset & 15) return fail(LLATTN_EINVAL, "attention: cache_offset must be a multiple of 16 bytes");
    if (c->workspace_bytes < pl->stats.workspace_bytes) return fail(LLATTN_ENOMEM, "attention: workspace smaller than the plan needs");
    int dev = -1;
    CU(cudaGetDevice(&dev));
    if (dev != c->device) return fail(LLATTN_EINVAL, "attention: current device %d, context device %d", dev, c->device);
    const size_t ns = pl->cap_items;
    float* Opart = reinterpret_cast<float*>(static_cast<uint8_t*>(c->workspace) + COUNTER_BYTES);
    float* Mpart = Opart + ns * QR * D;
    float* Lpart = Mpart + ns * QR;
    KParams p{};
    p.items = pl->d_items; p.cta_first = pl->d_cta_first;
    p.Q = static_cast<const half*>(io->Q); p.Kf = static_cast<const half*>(io->Kf); p.Vf = static_cast<const half*>(io->Vf);
    p.Opart = Opart; p.Mpart = Mpart; p.Lpart = Lpart;
    p.sl2 = (io->scale > 0.f ? io->scale : 0.08838834764831845f) * 1.4426950408889634f;
    p.err = c->err_word;
    p.merge = pl->d_merge;
    p.tile_counters = static_cast<int*>(c->workspace);
    p.out = MergeOut{static_cast<half*>(io->O16), io->O32, io->LSE, io->q8, io->s8, io->sum8};
    p.cache_offset = io->cache_offset;
    // cooperative: the driver starts the grid only when all of its CTAs can be resident together (see plan_create)
    void* args[] = {&p};
    const void* fn = (io->flags & LLATTN_IO_PRECISE_P) ? reinterpret_cast<const void*>(attn_tile_kernel<true>)
                                                       : reinterpret_cast<const void*>(attn_tile_kernel<false>);
    CU(cudaLaunchCooperativeKernel(fn, dim3(pl->launch_ctas), dim3(ATTN_THREADS), args, ATTN_SMEM_BYTES, as_stream(stream)));
    return LLATTN_OK;
}

// Host-buffer path, pipelined over consecutive calls: inputs go up on the context's own copy stream into one of two
// staging slots, the kernels run on the caller's stream once their slot has landed, results go down on a second copy
// stream. Call k's upload therefore overlaps call k-1's kernels and call k-1's download overlaps call k's kernels.
int llattn_attention_host(llattn_ctx* c, const llattn_plan* pl, const llattn_io* h, void* stream) {
    using namespace llattn;
    if (!c || !pl || pl->ctx != c) return fail(LLATTN_EINVAL, "attention_host: plan does not belong to this context");
    if (int rc = check_io(h, "attention_host")) return rc;
    int dev = -1;
    CU(cudaGetDevice(&dev));
    if (dev != c->device) return fail(LLATTN_EINVAL, "attention_host: current device %d, context device %d", dev, c->device);
    const size_t nq = size_t(pl->stats.nq_total), rows = nq * BLK;
    const size_t bQ = rows * NQH * D * 2, bKV = rows * NKV * D * 2;
    const size_t bO16 = h->O16 ? bQ : 0, bO32 = h->O32 ? rows * NQH * D * 4 : 0, bLSE = h->LSE ? rows * NQH * 4 : 0;
    const size_t bq8 = h->q8 ? rows * 2048 : 0, bs8 = h->q8 ? rows * NQH * 4 : 0;
    auto up = [](size_t x) { return (x + 255) / 256 * 256; };
    const size_t need = up(bQ) + 2 * up(bKV) + up(bO16) + up(bO32) + up(bLSE) + up(bq8) + 2 * up(bs8);
    std::lock_guard<std::mutex> lk(c->mu);
    if (!c->host_ready) {
        CU(cudaStreamCreateWithFlags(&c->s_in, cudaStreamNonBlocking));
        CU(cudaStreamCreateWithFlags(&c->s_out, cudaStreamNonBlocking));
        for (int i = 0; i < 2; ++i) {
            CU(cudaEventCreateWithFlags(&c->ev_in[i], cudaEventDisableTiming));
            CU(cudaEventCreateWithFlags(&c->ev_comp[i], cudaEventDisableTiming));
            CU(cudaEventCreateWithFlags(&c->ev_out[i], cudaEventDisableTiming));
        }
        c->host_ready = true;
    }
    if (2 * need > c->stage_bytes) {          // growing frees the old staging area: nothing may still be using it
        CU(cudaDeviceSynchronize());
        if (int rc = grow(&c->stage, &c->stage_bytes, 2 * need)) return rc;
        c->stage_slot_bytes = c->stage_bytes / 2 / 256 * 256;
    }
    const int slot = c->host_slot;
    c->host_slot ^= 1;
    uint8_t* d = static_cast<uint8_t*>(c->stage) + size_t(slot) * c->stage_slot_bytes;
    cudaStream_t st = as_stream(stream);
    llattn_io dio{};
    uint8_t* dQ = d; d += up(bQ);
    uint8_t* dK = d; d += up(bKV);
    uint8_t* dV = d; d += up(bKV);
    dio.Q = dQ; dio.Kf = dK; dio.Vf = dV; dio.scale = h->scale; dio.flags = h->flags; dio.cache_offset = h->cache_offset;
    if (bO16) { dio.O16 = d; d += up(bO16); }
    if (bO32) { dio.O32 = reinterpret_cast<float*>(d); d += up(bO32); }
    if (bLSE) { dio.LSE = reinterpret_cast<float*>(d); d += up(bLSE); }
    if (bq8) {
        dio.q8 = reinterpret_cast<int8_t*>(d); d += up(bq8);
        dio.s8 = reinterpret_cast<float*>(d); d += up(bs8);
        dio.sum8 = reinterpret_cast<int32_t*>(d); d += up(bs8);
    }
    // upload: the slot's previous kernels (two calls ago) must have finished reading it, and its previous download must
    // have drained the output area (a plan with more query blocks lays the slot out differently)
    CU(cudaStreamWaitEvent(c->s_in, c->ev_comp[slot], 0));
    CU(cudaStreamWaitEvent(c->s_in, c->ev_out[slot], 0));
    CU(cudaMemcpyAsync(dQ, h->Q, bQ, cudaMemcpyHostToDevice, c->s_in));
    CU(cudaMemcpyAsync(dK, h->Kf, bKV, cudaMemcpyHostToDevice, c->s_in));
    CU(cudaMemcpyAsync(dV, h->Vf, bKV, cudaMemcpyHostToDevice, c->s_in));
    CU(cudaEventRecord(c->ev_in[slot], c->s_in));
    // kernels: after the upload, and after the slot's previous download has drained its output area
    CU(cudaStreamWaitEvent(st, c->ev_in[slot], 0));
    CU(cudaStreamWaitEvent(st, c->ev_out[slot], 0));
    if (int rc = llattn_attention(c, pl, &dio, stream)) return rc;
    CU(cudaEventRecord(c->ev_comp[slot], st));
    // download
    CU(cudaStreamWaitEvent(c->s_out, c->ev_comp[slot], 0));
    if (bO16) CU(cudaMemcpyAsync(h->O16, dio.O16, bO16, cudaMemcpyDeviceToHost, c->s_out));
    if (bO32) CU(cudaMemcpyAsync(h->O32, dio.O32, bO32, cudaMemcpyDeviceToHost, c->s_out));
    if (bLSE) CU(cudaMemcpyAsync(h->LSE, dio.LSE, bLSE, cudaMemcpyDeviceToHost, c->s_out));
    if (bq8) {
        CU(cudaMemcpyAsync(h->q8, dio.q8, bq8, cudaMemcpyDeviceToHost, c->s_out));
        CU(cudaMemcpyAsync(h->s8, dio.s8, bs8, cudaMemcpyDeviceToHost, c->s_out));
        CU(cudaMemcpyAsync(h->sum8, dio.sum8, bs8, cudaMemcpyDeviceToHost, c->s_out));
    }
    CU(cudaEventRecord(c->ev_out[slot], c->s_out));
    return LLATTN_OK;
}

int llattn_host_flush(llattn_ctx* c, void* stream) {
    if (!c) return fail(LLATTN_EINVAL, "host_flush: null context");
    std::lock_guard<std::mutex> lk(c->mu);
    if (!c->host_ready) return LLATTN_OK;
    for (int i = 0; i < 2; ++i) CU(cudaStreamWaitEvent(as_stream(stream), c->ev_out[i], 0));
    return LLATTN_OK;
}

int llattn_device_status(llattn_ctx* c, void* stream, int* code) {
    if (!c || !code) return fail(LLATTN_EINVAL, "device_status: null pointer");
    CU(cudaStreamSynchronize(as_stream(stream)));
    CU(cudaMemcpy(code, c->err_word, sizeof(int), cudaMemcpyDeviceToHost));
    if (*code) {
        CU(cudaMemset(c->err_word, 0, sizeof(int)));
        if (c->workspace) CU(cudaMemset(c->workspace, 0, COUNTER_BYTES));      // an aborted launch may have left tile counters behind
        return fail(LLATTN_EDEVICE, "a kernel wait ran out (error bits 0x%x)", *code);
    }
    return LLATTN_OK;
}

}  // extern "C"
