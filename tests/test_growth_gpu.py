"""Tables that grow: reserve, the automatic doubling at the top of the
insert-like calls, and set_max_capacity, through the C ABI on the GPU.

The cases follow tests/merlin_hashtable_test.cc.cu:1080-1222 (test_rehash) and
:1223-1368 (test_rehash_on_big_batch) of the reference: everything inserted
before a doubling is still found afterwards with its row and score, in pure-HBM
tables and in tables whose rows spill into pinned host memory.
"""
import numpy as np
import pytest

from tests.hkv_testlib import (OracleTable, ProductTable, RefTable, ref_available, sorted_by_key,
                               unique_keys, values_for)

pytestmark = pytest.mark.gpu
CUSTOMIZED = 4


@pytest.mark.parametrize("max_hbm", [16 << 30, 0])
def test_rehash_keeps_every_entry(max_hbm):
    """One bucket of 128 slots grows to four while 256 keys arrive, as in the
    reference's test_rehash (reserved_key_start_bit 5, HBM and host rows)."""
    init, top, dim, n = 128, 512, 8, 256
    for round_ in range(5):
        t = ProductTable(init, dim, CUSTOMIZED, reserved_key_start_bit=5, max_capacity=top,
                         max_hbm_for_vectors=max_hbm)
        keys = unique_keys(n, seed=900 + round_, reserved_key_start_bit=5)
        vals = values_for(keys, dim)
        assert t.size() == 0 and t.capacity() == init
        t.insert_or_assign(keys, vals, keys.copy())
        assert t.capacity() == top          # 256 / 128 and 256 / 256 are above 0.5
        k, v, s = t.export_batch()
        # four buckets of 128 almost surely hold 256 random keys; whatever was
        # admitted must survive the reserve below untouched
        admitted = k.size
        assert admitted == t.size() and admitted > 200
        t.reserve(top)
        assert t.capacity() == top and t.size() == admitted
        fv, ff, fs = t.find(keys)
        assert ff.sum() == admitted
        np.testing.assert_array_equal(fs[ff], keys[ff])
        np.testing.assert_array_equal(fv[ff], vals[ff])
        np.testing.assert_array_equal(t.contains(keys), ff)
        t.clear()
        assert t.size() == 0
        t.close()


def test_reserve_steps_and_limits():
    dim = 4
    t = ProductTable(1024, dim, CUSTOMIZED, max_capacity=1 << 15, max_load_factor=0.9)
    o = OracleTable(1024, dim, CUSTOMIZED, max_capacity=1 << 15, max_load_factor=0.9)
    keys = unique_keys(600, seed=77)
    for x in (t, o):
        x.insert_or_assign(keys, values_for(keys, dim), np.arange(1, 601, dtype=np.uint64))
    for request, want in [(1024, 1024), (1025, 2048), (5000, 8192), (4096, 8192),
                          (1 << 16, 8192), (1 << 15, 1 << 15), (1 << 15, 1 << 15)]:
        t.reserve(request)
        o.reserve(request)
        assert t.capacity() == want == o.capacity(), (request, t.capacity(), o.capacity())
        assert t.size() == 600
    v, f, s = t.find(keys)
    assert f.all()
    np.testing.assert_array_equal(v, values_for(keys, dim))
    np.testing.assert_array_equal(s, np.arange(1, 601, dtype=np.uint64))
    with pytest.raises(ValueError):
        t.set_max_capacity(3 << 14)
    t.set_max_capacity(1 << 16)
    t.reserve(1 << 16)
    assert t.capacity() == 1 << 16 and t.size() == 600
    t.close()


def test_growth_moves_rows_between_hbm_and_host():
    """With a small max_hbm_for_vectors the first buckets keep their rows in
    HBM and the buckets added by a doubling keep theirs in pinned host memory."""
    dim = 16
    hbm = 2048 * dim * 4          # rows of 2048 slots
    t = ProductTable(1024, dim, CUSTOMIZED, max_capacity=8192, max_hbm_for_vectors=hbm,
                     max_load_factor=0.75)
    o = OracleTable(1024, dim, CUSTOMIZED, max_capacity=8192, max_load_factor=0.75)
    keys = unique_keys(5000, seed=31)
    at = 0
    for n in (700, 700, 1400, 2200):
        part = keys[at:at + n]
        sc = np.arange(at + 1, at + n + 1, dtype=np.uint64)
        for x in (t, o):
            x.insert_or_assign(part, values_for(part, dim, seed=at), sc)
        at += n
        assert t.capacity() == o.capacity()
        view = t.t.view()
        assert view.hbm_slots == min(2048, t.capacity())
        pv, pf, ps = t.find(keys[:at])
        ov, of, os_ = o.find(keys[:at])
        np.testing.assert_array_equal(pf, of)
        np.testing.assert_array_equal(pv[pf], ov[of])
        np.testing.assert_array_equal(ps[pf], os_[of])
    assert t.capacity() == 8192
    pk, pv, ps = sorted_by_key(*t.export_batch())
    ok, ov, os_ = sorted_by_key(*o.export_batch())
    np.testing.assert_array_equal(pk, ok)
    np.testing.assert_array_equal(pv, ov)
    np.testing.assert_array_equal(ps, os_)
    t.close()


def test_big_batches_grow_like_the_reference():
    """Batches larger than the table (the reference's test_rehash_on_big_batch):
    the table doubles until the batch fits under max_load_factor."""
    dim = 8
    kw = dict(max_capacity=1 << 18, max_load_factor=0.5)
    t = ProductTable(1 << 12, dim, CUSTOMIZED, **kw)
    o = OracleTable(1 << 12, dim, CUSTOMIZED, **kw)
    r = RefTable(1 << 12, dim, CUSTOMIZED, **kw) if ref_available(CUSTOMIZED) else None
    keys = unique_keys(90000, seed=5)
    tables = [x for x in (t, o, r) if x is not None]
    at = 0
    for n in (20000, 1000, 60000):
        part = keys[at:at + n]
        sc = np.arange(at + 1, at + n + 1, dtype=np.uint64)
        for x in tables:
            x.insert_or_assign(part, values_for(part, dim), sc)
        at += n
        caps = [x.capacity() for x in tables]
        sizes = [x.size() for x in tables]
        assert len(set(caps)) == 1 and len(set(sizes)) == 1, (caps, sizes)
    want = sorted_by_key(*o.export_batch())
    for x in tables:
        got = sorted_by_key(*x.export_batch())
        for a, b in zip(got, want):
            np.testing.assert_array_equal(a, b)
    t.close()
    if r is not None:
        r.close()


def test_large_rehash_keeps_rows_and_scores():
    """4 Mi slots -> 8 Mi slots with 3 M entries: every key, row and score
    survives; counts per bucket stay consistent (size == live keys)."""
    import torch

    dim = 32
    t = ProductTable(1 << 22, dim, CUSTOMIZED, max_capacity=1 << 23, max_load_factor=1.0)
    n = 3_000_000
    keys = unique_keys(n, seed=1234)
    vals = values_for(keys, dim)
    sc = np.arange(1, n + 1, dtype=np.uint64)
    t.insert_or_assign(keys, vals, sc)
    before = t.size()
    assert t.capacity() == 1 << 22
    t.reserve(1 << 23)
    torch.cuda.synchronize()
    assert t.capacity() == 1 << 23 and t.size() == before
    fv, ff, fs = t.find(keys)
    assert ff.sum() == before
    np.testing.assert_array_equal(fs[ff], sc[ff])
    np.testing.assert_array_equal(fv[ff], vals[ff])
    k, _, _ = t.export_batch()
    assert k.size == before and np.unique(k).size == before
    t.close()


def test_dynamic_max_capacity_like_the_reference():
    """tests/dynamic_max_capacity_test.cc.cu of the reference, scaled down:
    insert_and_evict (LRU) fills a growing table to load factor 0.98, then
    set_max_capacity + reserve double it, again and again; at the end every key
    ever inserted is either in the table or was handed back as evicted, with its
    own row."""
    LRU = 0
    dim, n = 4, 10000
    max_cap, uplimit = 1 << 14, 1 << 17
    t = ProductTable(1 << 12, dim, LRU, max_capacity=max_cap,
                     max_hbm_for_vectors=uplimit * dim * 4)
    seen = {}
    offset = 0
    while True:
        keys = np.arange(offset, offset + n, dtype=np.uint64)
        rows = np.repeat(keys.astype(np.float32)[:, None], dim, axis=1)
        ek, ev, _ = t.insert_and_evict(keys, rows, use_counter=False)
        offset += n
        for k, v in zip(ek.tolist(), ev):
            assert np.all(v == np.float32(k))
            seen[k] = True
        if t.size() / t.capacity() >= 0.98:
            assert t.size() >= int(max_cap * 0.98)
            max_cap *= 2
            if max_cap > uplimit:
                break
            t.set_max_capacity(max_cap)
            t.reserve(max_cap)
            assert t.capacity() == max_cap
            assert t.size() / t.capacity() <= 0.5
        assert offset <= 4 * uplimit, "walked too many keys without finishing"
    k, v, _ = t.export_batch()
    assert np.all(v == k.astype(np.float32)[:, None])
    for key in k.tolist():
        seen[key] = True
    assert t.capacity() * 2 == max_cap
    assert len(seen) >= int(t.capacity() * 0.98)
    assert len(seen) == offset           # nothing was lost: resident or returned as evicted
    t.close()
