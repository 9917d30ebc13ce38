"""CPU-side checks: the C-ABI library loads and exports every symbol the header declares, argument errors come back
as status codes without touching a GPU, the host planner covers every KV unit exactly once within its CTA budget,
and the request sharding balances. No compute call is made here."""
import ctypes
import importlib
import os
import re

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def api(pkg):
    m = importlib.import_module(pkg.__name__ + ".api")
    if not os.path.exists(m.LIB_PATH):
        importlib.import_module(pkg.__name__ + ".build").build()
    m.lib()
    return m


def test_library_exports_every_declared_symbol(api):
    hdr = open(os.path.join(ROOT, "include", "llattn.h")).read()
    declared = set(re.findall(r"^(?:int|void|const char\*)\s+(llattn_[a-z0-9_]+)\s*\(", hdr, flags=re.M))
    assert declared, "no declarations parsed"
    L = api.lib()
    for name in sorted(declared):
        assert hasattr(L, name), f"{name} declared in include/llattn.h but not exported"
    assert declared == set(api.EXPORTS)
    assert b"sm_100a" in L.llattn_version()


def test_reference_split_policy_helpers(api):
    # attn::pick_bpc / chunks_for of the reference (engine/attn.cu:67,361-364), values from its launch-shape table
    assert [api.pick_bpc(n, 1) for n in (4, 32, 256, 512, 1024)] == [1, 8, 64, 128, 256]
    assert api.pick_bpc(1007, 16) == 1007 and api.pick_bpc(100, 2) == 50 and api.pick_bpc(0, 1) == 1
    assert api.chunks_for(0, 8) == 1 and api.chunks_for(1024, 256) == 4 and api.chunks_for(33, 8) == 5


def test_shim_default_split_fits_the_reference_engines_partial_buffers():
    """The source-level shim spreads a context over up to 37 chunks per kv head, while an unmodified engine allocates
    its partial buffers for 16 query blocks x 4 kv heads x 4 chunks = 256 slots (engine/engine.cu:301-304) and calls
    pick_bpc with two arguments. The slot index a launch writes stays below nb * 4 * nchunks; this restates the shim's
    policy (include/attn_shim.cuh) and checks the bound for every batch size and context length the engine can reach."""
    def shim_pick_bpc(nblocks, nbatch, max_chunks=37):
        want = max(1, min(max_chunks, (148 + 4 * nbatch - 1) // (4 * nbatch)))
        bpc = max(1, (nblocks + want - 1) // want)
        bpc = max(bpc, min(nblocks, 8))
        return (bpc + 3) // 4 * 4
    worst = 0
    for nb in range(1, 17):
        for nblocks in list(range(0, 300)) + [511, 512, 992, 1007, 1023, 1024, 4095]:
            vis = nblocks + nb - 1
            bpc = shim_pick_bpc(vis, nb)
            nch = 1 if vis <= 0 else (vis + bpc - 1) // bpc
            worst = max(worst, nb * 4 * nch)
            assert bpc % 4 == 0 and nb * 4 * nch <= 256, (nb, nblocks, bpc, nch)
    assert worst <= 192
    src = open(os.path.join(ROOT, "include", "attn_shim.cuh")).read()
    assert "static_assert(slots_fit_reference(1)" in src and "MAX_CHUNKS_HINT = 37" in src


def test_argument_errors_are_status_codes_without_a_gpu(api):
    L = api.lib()
    assert L.llattn_kv_commit(None, None, None, 4, 0, 1, None) == api.EINVAL
    assert b"null" in L.llattn_last_error()
    buf = ctypes.create_string_buffer(64)
    a = ctypes.addressof(buf) + (16 - ctypes.addressof(buf) % 16)
    assert L.llattn_kv_commit(a, a, a, 4, 3, 2, None) == api.EINVAL          # blocks 3..4 in a 4-block cache
    assert L.llattn_kv_commit(a + 2, a, a, 4, 0, 1, None) == api.EINVAL      # misaligned
    assert L.llattn_kv_commit(a, a, a, 4, 0, 0, None) == api.OK              # nothing to do
    assert L.llattn_attn_combine(None, None, None, 1, 0, 1, None, None, None, None, 1, None) == api.EINVAL
    assert L.llattn_attention_static(a, a, a, a, 8, 4, 17, 0.0, a, None, None, None, None, None, None, None) == api.EINVAL
    assert L.llattn_plan_get_stats(None, None) == api.EINVAL
    st = api.PlanStats()
    assert L.llattn_plan_preview(None, 1, 1, ctypes.byref(st), None, 0, None, 0) == api.EINVAL


@pytest.mark.parametrize("lengths,nq,nctas", [
    ([1024] * 64, None, 148), ([256], None, 148), ([0], None, 148), ([3, 0, 17, 250, 1, 64], None, 7),
    ([992], [16], 148), ([5, 40], [3, 2], 148), (list(range(0, 300, 7)), None, 148), ([1024] * 3, None, 1),
])
def test_planner_covers_every_unit_once(api, lengths, nq, nctas):
    st, items, cta_first = api.plan_preview(lengths, nctas, nq)
    nqs = [1] * len(lengths) if nq is None else nq
    assert 1 <= st.nctas <= nctas
    assert cta_first[0] == 0 and cta_first[-1] == st.nitems and np.all(np.diff(cta_first) >= 0)
    assert np.array_equal(items[:, 6], np.arange(st.nitems))                 # one partial slot per run, in order
    seen = {}
    for seq, qb, kvh, rec0, nrec, fresh, slot, _ in items:
        key = (seq, qb, kvh)
        cover = seen.setdefault(key, [0, 0])
        assert rec0 == cover[0], "runs of a tile must be consecutive"
        assert rec0 % api.tile_units() == 0, "cuts fall on MMA tile boundaries"
        assert nrec + fresh > 0
        cover[0] += nrec
        cover[1] += fresh
    total = 0
    for s, n in enumerate(lengths):
        for j in range(nqs[s]):
            for h in range(4):
                assert seen[(s, j, h)] == [n + j, 1], (s, j, h)
                total += n + j + 1
    assert total == st.total_units
    per_cta = [int(items[cta_first[c]:cta_first[c + 1], 4:6].sum()) for c in range(st.nctas)]
    assert max(per_cta) == st.max_cta_units
    if st.total_units >= 64 * nctas:                                         # enough work: shares are near equal
        assert max(per_cta) <= 1.02 * st.total_units / st.nctas + 12         # (a cut never leaves a piece under 12 units)


def test_planner_gives_every_run_its_own_cta_when_the_step_is_small(api):
    """Fewer output tiles than CTAs: a run per CTA, tiles cut into equal runs of about 0.75 sqrt(units) units; with more work
    than that the shares are contiguous again and a tile straddles at most two CTAs' lists per cut."""
    for nblocks, lo, hi in ((64, 7, 10), (256, 17, 24), (1024, 30, 37)):
        st, items, cta_first = api.plan_preview([nblocks], 148)
        assert st.nitems == st.nctas and np.all(np.diff(cta_first[:st.nctas + 1]) == 1)
        per_tile = np.bincount(items[:, 7])
        assert len(per_tile) == 4 and per_tile.min() == per_tile.max() and lo <= per_tile[0] <= hi, per_tile
        units = items[:, 4] + items[:, 5]
        assert units.max() - units[items[:, 5] == 0].min() <= 4 and np.all(items[:, 3] % api.tile_units() == 0)
    st, items, cta_first = api.plan_preview([1024] * 30, 148)                 # 120 tiles of 1025 units on 148 CTAs
    assert st.nctas == 148 and st.nitems > 148 and st.max_cta_units <= 1.02 * st.total_units / 148 + 12
    st, items, cta_first = api.plan_preview([0, 1, 2, 3], 148)                # 16 tiny tiles: one CTA each
    assert st.nctas == 16 and st.nitems == 16
    st, items, cta_first = api.plan_preview([64] * 36, 148)                   # tiles of 65 units, shares of 64: no 1-unit runs
    assert (items[:, 4] + items[:, 5]).min() >= 12


def test_planner_invariants_on_random_batches(api):
    """300 seeded random batches (1 .. 40 sequences, 0 .. 1100 blocks, 1 .. 3 query blocks, 1 .. 148 CTAs): every unit is
    covered exactly once and in order, cuts fall on tile boundaries, runs never outnumber tiles + CTAs (the capacity a
    plan reserves so that updates never allocate), a CTA holds at most one run of a tile (the folding relies on it)."""
    g = np.random.default_rng(2024)
    for _ in range(300):
        nseq = int(g.integers(1, 41))
        lengths = [int(x) for x in g.choice([0, 1, 3, 7, 31, 64, 255, 256, 1024, 1100], nseq)]
        nq = [int(x) for x in g.integers(1, 4, nseq)]
        nctas = int(g.choice([1, 2, 7, 37, 64, 148]))
        st, items, cta_first = api.plan_preview(lengths, nctas, nq)
        tiles = 4 * sum(nq)
        assert 1 <= st.nctas <= nctas and st.nitems <= tiles + nctas
        assert np.array_equal(items[:, 6], np.arange(st.nitems)) and np.all(items[:, 3] % api.tile_units() == 0)
        done = {}
        for seq, qb, kvh, rec0, nrec, fresh, slot, tile in items:
            c = done.setdefault((seq, qb, kvh), [0, 0, tile])
            assert rec0 == c[0] and c[1] == 0 and tile == c[2] and nrec + fresh > 0
            c[0] += nrec; c[1] += fresh
        assert len(done) == tiles
        for (seq, qb, kvh), (nrec, fresh, _) in done.items():
            assert nrec == lengths[seq] + qb and fresh == 1
        for c in range(st.nctas):
            mine = items[cta_first[c]:cta_first[c + 1], 7]
            assert len(set(mine.tolist())) == len(mine)


def test_sharding_balances_ragged_requests(pkg):
    sh, wl = pkg.sharding, pkg.workload
    lens = wl.ragged_lengths(256)
    assert lens.min() >= 4 and lens.max() <= 1024 and len(lens) == 256
    assert np.array_equal(lens, wl.ragged_lengths(256))                       # seeded
    for world in (1, 2, 4, 8):
        shards = sh.shard_lpt(lens, world)
        assert sorted(i for s in shards for i in s) == list(range(256))
        assert sh.imbalance(lens, shards) <= 1.01
    rr = sh.shard_round_robin(64, 8)
    assert all(len(s) == 8 for s in rr) and sorted(i for s in rr for i in s) == list(range(64))


def test_workload_is_reproducible_and_shaped(pkg):
    wl = pkg.workload
    K, V = wl.context_blocks(3, seq=5, layer=2)
    K2, V2 = wl.context_blocks(3, seq=5, layer=2)
    assert K.shape == (3, 32, 4, 128) and K.dtype == np.float16 and np.array_equal(K, K2) and np.array_equal(V, V2)
    out = list(wl.OUTLIER_CHANNELS)
    rest = [c for c in range(128) if c not in out]
    big = wl.context_blocks(64, seq=1)[0].astype(np.float32)
    assert 6.0 < big[..., out].std() < 10.0 and 0.9 < big[..., rest].std() < 1.1
    assert wl.algorithmic_bytes(1024) == 592 * 32768 + 327680
    assert wl.algorithmic_flops(1024) == 262144 * (32768 + 32)


def test_decoder_commit_policy(api):
    """engine/decode.cu:267-280: KV-only commit exactly when the last forward ran on the block's final ids."""
    blk = list(range(100, 132))
    assert api.commit_needs_forward(blk, None) and api.commit_needs_forward(blk, [])
    assert not api.commit_needs_forward(blk, list(blk)) and not api.commit_needs_forward(np.array(blk), tuple(blk))
    other = list(blk); other[17] = 156895
    assert api.commit_needs_forward(blk, other) and api.commit_needs_forward(blk, blk[:31])
    with pytest.raises(ValueError):
        api.commit_block(blk, other, None, None, None, 4, 0)        # a forward pass is needed and none was given
