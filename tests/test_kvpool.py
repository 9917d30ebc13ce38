"""Page manager with prefix reuse (llattn_kvpool_*): host logic, no GPU.

The rule it generalises is the reference's: leading full 32-token blocks of a new prompt that equal the committed ids are
kept and not prefilled again (engine/decode.cu:469-481)."""
import importlib
import os

import numpy as np
import pytest


@pytest.fixture(scope="module")
def api(pkg):
    m = importlib.import_module(pkg.__name__ + ".api")
    if not os.path.exists(m.LIB_PATH):
        importlib.import_module(pkg.__name__ + ".build").build()
    m.lib()
    return m


def _tokens(seed, n):
    return np.random.default_rng(seed).integers(0, 150000, n, dtype=np.int32)


def test_prefix_reuse_same_prompt(api):
    pool = api.KvPool(64)
    t = _tokens(1, 32 * 5 + 7)                      # 5 full blocks + a ragged tail that gets no page
    s1, r1, p1 = pool.open(t)
    assert r1 == 0 and len(p1) == 5 and len(set(p1.tolist())) == 5
    pool.mark_committed(s1)                         # the caller has run the commit kernel on p1
    s2, r2, p2 = pool.open(t)
    assert r2 == 5 and p2.tolist() == p1.tolist()
    st = pool.stats()
    assert st["hits"] == 5 and st["misses"] == 5 and st["free"] == 64 - 5 and st["cached"] == 0
    pool.close(s1)
    assert pool.stats()["cached"] == 0              # still held by s2
    pool.close(s2)
    assert pool.stats()["cached"] == 5
    s3, r3, p3 = pool.open(t[:32 * 3])
    assert r3 == 3 and p3.tolist() == p1[:3].tolist()


def test_divergence_and_reference_rule(api):
    """Same count as the reference's loop: blocks are reused up to the first block that differs."""
    pool = api.KvPool(64)
    a = _tokens(2, 32 * 6)
    b = a.copy()
    b[32 * 3 + 5] += 1                               # block 3 differs
    sa, _, pa = pool.open(a)
    pool.mark_committed(sa)
    sb, rb, pb = pool.open(b)
    keep = 0
    while keep < 6 and np.array_equal(a[keep * 32:(keep + 1) * 32], b[keep * 32:(keep + 1) * 32]):
        keep += 1
    assert rb == keep == 3
    assert pb[:3].tolist() == pa[:3].tolist()
    assert not set(pb[3:].tolist()) & set(pa.tolist())
    # blocks 4, 5 hold the same ids as a's but follow a different block 3: not shared
    assert pool.stats()["misses"] == 6 + 3


def test_append_and_shared_continuation(api):
    pool = api.KvPool(32)
    t = _tokens(3, 64)
    s1, _, _ = pool.open(t)
    pool.mark_committed(s1)
    s2, r2, _ = pool.open(t)
    assert r2 == 2
    blk = _tokens(4, 32)
    p1, hit1 = pool.append(s1, blk)
    pool.mark_committed(s1)
    p2, hit2 = pool.append(s2, blk)
    assert not hit1 and hit2 and p1 == p2
    p3, hit3 = pool.append(s2, _tokens(5, 32))
    assert not hit3 and p3 != p1
    assert pool.pages(s1).tolist()[-1] == p1 and len(pool.pages(s2)) == 4
    with pytest.raises(ValueError):
        pool.append(s1, blk[:31])


def test_lru_eviction_and_exhaustion(api):
    pool = api.KvPool(8)
    a, b, c = _tokens(6, 32 * 4), _tokens(7, 32 * 4), _tokens(8, 32 * 4)
    sa, _, pa = pool.open(a)
    sb, _, pb = pool.open(b)
    pool.mark_committed(sa); pool.mark_committed(sb)
    with pytest.raises(RuntimeError, match="exhausted"):
        pool.open(c)                                 # every page is held
    st = pool.stats()
    assert st["free"] == 0 and st["cached"] == 0     # the failed open gave its pages back ... there were none
    pool.close(sa)                                   # a's pages become reusable, deepest block first in the LRU order
    sc, rc, pc = pool.open(c[:64])                   # takes two of them: a's blocks 3 and 2
    assert rc == 0 and set(pc.tolist()) == set(pa[2:].tolist())
    assert pool.stats()["evictions"] == 2
    with pytest.raises(RuntimeError, match="exhausted"):
        pool.open(a)                                 # blocks 0, 1 are cached, but 2, 3 need pages and none is left
    assert pool.stats()["cached"] == 2               # the failed open let go of the two it had found
    pool.close(sc)                                   # never committed: its two pages are free again, not cached
    assert pool.stats()["free"] == 2 and pool.stats()["cached"] == 2
    s4, r4, p4 = pool.open(a)                        # blocks 0, 1 still cached; 2, 3 were evicted: c's pages recycled
    assert r4 == 2 and p4[:2].tolist() == pa[:2].tolist()
    assert pool.stats()["free"] == 0 and pool.stats()["cached"] == 0
    pool.mark_committed(s4)
    pool.close(sb); pool.close(s4)
    assert pool.stats()["cached"] == 8


def test_failed_open_rolls_back(api):
    pool = api.KvPool(4)
    s, _, _ = pool.open(_tokens(9, 64))
    with pytest.raises(RuntimeError, match="exhausted"):
        pool.open(_tokens(10, 32 * 3))
    st = pool.stats()
    assert st["free"] == 2 and st["cached"] == 0     # the two pages it had taken are free again and registered nowhere
    s2, r2, p2 = pool.open(_tokens(10, 64))          # the same leading blocks as the failed open: nothing to reuse
    assert r2 == 0 and len(p2) == 2
    assert pool.stats()["hits"] == 0


def test_only_committed_pages_are_reused(api):
    """A page is reported as reused only after the caller said its records exist; a sequence closed before its commit
    leaves nothing behind."""
    pool = api.KvPool(16)
    t = _tokens(20, 32 * 3)
    s1, r1, p1 = pool.open(t)
    s2, r2, p2 = pool.open(t)                        # s1 has not committed yet: same pages, but s2 must prefill too
    assert r1 == 0 and r2 == 0 and p2.tolist() == p1.tolist()
    pool.mark_committed(s1, 2)                       # two of the three blocks are written
    s3, r3, p3 = pool.open(t)
    assert r3 == 2 and p3.tolist() == p1.tolist()
    with pytest.raises(RuntimeError, match="blocks"):
        pool.mark_committed(s1, 4)
    pool.close(s1); pool.close(s2); pool.close(s3)
    st = pool.stats()
    assert st["cached"] == 2 and st["free"] == 14    # the uncommitted third page went back to the free list
    u = _tokens(21, 64)
    s4, _, _ = pool.open(u)
    pool.close(s4)                                   # closed before any commit
    s5, r5, _ = pool.open(u)
    assert r5 == 0 and pool.stats()["cached"] == 2


def test_errors(api):
    with pytest.raises(RuntimeError):
        api.KvPool(0)
    pool = api.KvPool(4)
    with pytest.raises(RuntimeError, match="not open"):
        pool.close(99)
    with pytest.raises(RuntimeError, match="not open"):
        pool.pages(5)
    s, r, p = pool.open(np.zeros(0, np.int32))       # empty prompt: a sequence with no pages yet
    assert r == 0 and len(p) == 0 and len(pool.pages(s)) == 0
    s2, r2, p2 = pool.open(_tokens(12, 31))          # shorter than a block
    assert len(p2) == 0


def test_page_table(api):
    t = api.KvPool.page_table([3, 0, 7], head_stride=5)
    assert t.shape == (4, 5) and t.dtype == np.int32
    assert t[:, :3].tolist() == [[12, 0, 28], [13, 1, 29], [14, 2, 30], [15, 3, 31]]
