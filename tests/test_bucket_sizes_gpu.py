"""Bucket sizes other than 128 (HashTableOptions::max_bucket_size).

The reference accepts any power of two whose key and score lines are
128-byte aligned (include/merlin_hashtable.cuh:107, 1032-1048) and serves the
sizes its pipeline kernels do not cover with its tile kernels
(include/merlin/core_kernels/lookup.cuh:873-925).  Its own test of that path,
tests/find_with_missed_keys_test.cc.cu:55-57, 158-212, runs bucket size 128 and
256 at load factors 0 / 0.2 / 0.5 / 0.75 / 1.0 with the value rows in HBM, half
in HBM and half in pinned host memory, and all in host memory; the same grid is
run here through the product, the CPU oracle and the reference's kernels live,
plus the smaller sizes.
"""
import numpy as np
import pytest

from tests.hkv_testlib import (OracleTable, ProductTable, RefTable, ref_available, sorted_by_key,
                               unique_keys, values_for)

pytestmark = pytest.mark.gpu
CUSTOMIZED = 4
CAP, DIM = 16 * 1024, 16          # 16 Ki slots x 64-byte rows = 1 MiB of rows
ROWS = CAP * DIM * 4
PLACEMENT = {"hbm": 1 << 30, "hybrid": ROWS // 2, "hmem": 0}


@pytest.mark.parametrize("placement", ["hbm", "hybrid", "hmem"])
@pytest.mark.parametrize("load_factor", [0.0, 0.2, 0.5, 0.75, 1.0])
@pytest.mark.parametrize("bucket", [128, 256])
def test_find_with_missed_keys_over_bucket_sizes(bucket, load_factor, placement):
    kw = dict(max_hbm_for_vectors=PLACEMENT[placement], max_bucket_size=bucket)
    p = ProductTable(CAP, DIM, CUSTOMIZED, **kw)
    o = OracleTable(CAP, DIM, CUSTOMIZED, max_bucket_size=bucket)
    r = RefTable(CAP, DIM, CUSTOMIZED, **kw) if ref_available(CUSTOMIZED) else None
    tables = [x for x in (p, o, r) if x is not None]
    keys = unique_keys(CAP, seed=1000 + bucket)
    n_in = int(CAP * load_factor)
    # distinct scores that grow with the position: what survives eviction does
    # not depend on the order in which a batch is applied
    scores = np.arange(1, CAP + 1, dtype=np.uint64)
    if n_in:
        for x in tables:
            x.insert_or_assign(keys[:n_in], values_for(keys[:n_in], DIM), scores[:n_in])
    assert [x.size() for x in tables] == [o.size()] * len(tables)
    want_v, want_f, want_s = o.find(keys)
    assert want_f[n_in:].sum() == 0 and (n_in == 0 or want_f[:n_in].mean() > 0.8)
    v, f, s = p.find(keys)
    np.testing.assert_array_equal(f, want_f)
    np.testing.assert_array_equal(v[f].view(np.uint32), want_v[f].view(np.uint32))
    np.testing.assert_array_equal(s[f], want_s[f])
    if r is not None:
        # Where a batch overflows buckets, the reference's concurrent evictions do not
        # always remove the smallest score (its scan ignores slots other threads hold,
        # include/merlin/core_kernels/upsert.cuh:179-183), so which keys survive is its
        # own; what it finds must be what was inserted, and about as much of it.
        v, f, s = r.find(keys)
        assert f[n_in:].sum() == 0
        if load_factor <= 0.5:
            np.testing.assert_array_equal(f, want_f)
        else:
            assert abs(int(f.sum()) - int(want_f.sum())) <= 0.02 * CAP
        np.testing.assert_array_equal(v[f].view(np.uint32), values_for(keys, DIM)[f].view(np.uint32))
        np.testing.assert_array_equal(s[f], scores[f])
    # the overload that returns the missed keys and their batch indices
    mv, mk, mi = p.find_missed(keys)
    miss = ~want_f
    assert mk.size == miss.sum()
    order = np.argsort(mi)
    np.testing.assert_array_equal(mi[order], np.nonzero(miss)[0])
    np.testing.assert_array_equal(mk[order], keys[miss])
    np.testing.assert_array_equal(mv[want_f].view(np.uint32), want_v[want_f].view(np.uint32))
    for x in tables:
        if hasattr(x, "close"):
            x.close()


@pytest.mark.parametrize("bucket,slot_layout", [(16, 0), (32, 1), (64, 0), (256, 1), (1024, 0),
                                                (128, 0), (128, 1)])
def test_every_operation_on_other_bucket_sizes(bucket, slot_layout):
    """insert_or_assign with eviction, find_or_insert, assign, accum_or_assign,
    erase, insert_and_evict, export and size on tables whose buckets are not 128
    slots, and on both slot layouts (keys and scores in separate arrays, or
    sharing 128-byte lines): product against the CPU oracle."""
    cap = bucket * 96
    p = ProductTable(cap, 8, CUSTOMIZED, max_bucket_size=bucket, slot_layout=slot_layout)
    o = OracleTable(cap, 8, CUSTOMIZED, max_bucket_size=bucket)
    assert p.t.max_bucket_size() == bucket and p.bucket_count() == o.bucket_count() == 96
    keys = unique_keys(3 * cap, seed=2000 + bucket)
    sc = np.arange(1, keys.size + 1, dtype=np.uint64)

    def same_tables():
        a, b = sorted_by_key(*p.export_batch()), sorted_by_key(*o.export_batch())
        for x, y in zip(a, b):
            np.testing.assert_array_equal(x, y)
        assert p.size() == o.size()

    half = cap // 2
    for t in (p, o):
        t.insert_or_assign(keys[:half], values_for(keys[:half], 8), sc[:half])
    same_tables()
    # overfill: every bucket evicts its smallest scores
    for t in (p, o):
        t.insert_or_assign(keys[half:2 * cap], values_for(keys[half:2 * cap], 8, seed=1), sc[half:2 * cap])
    same_tables()
    assert p.size() > 0.95 * cap
    q = keys[cap:2 * cap + 500]
    pv, pf, ps = p.find(q)
    ov, of, os_ = o.find(q)
    np.testing.assert_array_equal(pf, of)
    np.testing.assert_array_equal(pv[pf], ov[of])
    np.testing.assert_array_equal(ps[pf], os_[of])
    # find_or_insert: hits return the stored rows, misses insert
    k2 = keys[2 * cap - 300:2 * cap + 300]
    rows_p = values_for(k2, 8, seed=2)
    rows_o = rows_p.copy()
    rows_p = p.find_or_insert(k2, rows_p, sc[2 * cap - 300:2 * cap + 300])
    rows_o = o.find_or_insert(k2, rows_o, sc[2 * cap - 300:2 * cap + 300])
    np.testing.assert_array_equal(rows_p, rows_o)
    same_tables()
    # assign (hits only), accum_or_assign, erase
    k3 = keys[2 * cap - 100:2 * cap + 700]
    for t in (p, o):
        t.assign(k3, values_for(k3, 8, seed=3), sc[:k3.size] + np.uint64(10 ** 7))
    same_tables()
    flags = (np.arange(k3.size) % 2 == 0)
    for t in (p, o):
        t.accum_or_assign(k3, values_for(k3, 8, seed=4), flags, sc[:k3.size] + np.uint64(2 * 10 ** 7))
    same_tables()
    for t in (p, o):
        t.erase(np.ascontiguousarray(k3[::3]))
    same_tables()
    # insert_and_evict returns what it displaced
    k4 = keys[2 * cap + 700:3 * cap]
    s4 = sc[2 * cap + 700:3 * cap] + np.uint64(10 ** 8)
    ep = sorted_by_key(*p.insert_and_evict(k4, values_for(k4, 8, seed=5), s4))
    eo = sorted_by_key(*o.insert_and_evict(k4, values_for(k4, 8, seed=5), s4))
    for x, y in zip(ep, eo):
        np.testing.assert_array_equal(x, y)
    same_tables()
    p.close()


def test_growth_with_256_slot_buckets():
    """reserve() doubles a table of 256-slot buckets: every entry survives."""
    cap = 256 * 16
    p = ProductTable(cap, 4, CUSTOMIZED, max_capacity=4 * cap, max_bucket_size=256,
                     max_load_factor=0.99)
    keys = unique_keys(cap // 2, seed=31)
    sc = np.arange(1, keys.size + 1, dtype=np.uint64)
    p.insert_or_assign(keys, values_for(keys, 4), sc)
    before = sorted_by_key(*p.export_batch())
    p.reserve(4 * cap)
    assert p.capacity() == 4 * cap and p.bucket_count() == 64
    after = sorted_by_key(*p.export_batch())
    for x, y in zip(before, after):
        np.testing.assert_array_equal(x, y)
    v, f, s = p.find(keys)
    assert f.all()
    np.testing.assert_array_equal(s, sc)
    p.close()


def test_bucket_sizes_the_library_refuses():
    import hierarchicalkv_b200 as hkv

    for bad in (8, 2048, 100):
        t = hkv.HashTable(hkv.EvictStrategy.kCustomized)
        with pytest.raises(hkv.MerlinException):
            t.init(hkv.HashTableOptions(init_capacity=bad * 64, max_capacity=bad * 64,
                                        max_hbm_for_vectors=1 << 30, dim=4, max_bucket_size=bad))
