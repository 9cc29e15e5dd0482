"""Parity of the CUDA path (through the C ABI) with the CPU oracle and, when
it was built, with the reference's own kernels -- same seeded inputs.

Bit-exact for found flags, keys, scores (non-LRU strategies) and copied
value rows on unique-key batches.  Table contents are compared as key-sorted
exports: slot positions are race-dependent in the reference itself.
"""
import numpy as np
import pytest

from tests.hkv_testlib import (OracleTable, ProductTable, RefTable, bucket_of, ref_available,
                               sorted_by_key, unique_keys, values_for)

pytestmark = pytest.mark.gpu

LRU, LFU, EPOCH_LRU, EPOCH_LFU, CUSTOMIZED = range(5)


def make_impls(capacity, dim, strategy, **kw):
    impls = {"product": ProductTable(capacity, dim, strategy, **kw),
             "oracle": OracleTable(capacity, dim, strategy,
                                   reserved_key_start_bit=kw.get("reserved_key_start_bit", 0))}
    if ref_available(strategy):
        impls["reference"] = RefTable(capacity, dim, strategy, **kw)
    return impls


def close_all(impls):
    for t in impls.values():
        if hasattr(t, "close"):
            t.close()


def assert_same_table(impls, with_scores=True):
    exports = {name: sorted_by_key(*t.export_batch()) for name, t in impls.items()}
    base_name = "oracle"
    bk, bv, bs = exports[base_name]
    for name, (k, v, s) in exports.items():
        assert k.size == impls[name].size(), name
        np.testing.assert_array_equal(k, bk, err_msg=f"{name} keys")
        np.testing.assert_array_equal(v.view(np.uint32), bv.view(np.uint32), err_msg=f"{name} values")
        if with_scores:
            np.testing.assert_array_equal(s, bs, err_msg=f"{name} scores")


def test_config1_fill_and_find_customized():
    """Capacity 1,048,576 (8192 x 128), dim 8; fill to load factor 0.5 in
    65,536-key insert_or_assign batches, then find batches that are half
    present, half fresh.  Customized scores (distinct) make every output
    comparable bit for bit."""
    capacity, dim, batch = 1 << 20, 8, 65536
    impls = make_impls(capacity, dim, CUSTOMIZED)
    keys = unique_keys(capacity // 2 + 4 * batch, seed=11)
    present, fresh = keys[: capacity // 2], keys[capacity // 2:]
    for b in range(0, present.size, batch):
        k = present[b:b + batch]
        v = values_for(k, dim)
        s = (np.arange(k.size, dtype=np.uint64) + np.uint64(b + 1))
        for t in impls.values():
            t.insert_or_assign(k, v, s)
    sizes = {name: t.size() for name, t in impls.items()}
    assert len(set(sizes.values())) == 1, sizes
    assert_same_table(impls)
    rng = np.random.default_rng(5)
    for r in range(4):
        q = np.concatenate([rng.choice(present, batch // 2, replace=False),
                            fresh[r * (batch // 2):(r + 1) * (batch // 2)]])
        rng.shuffle(q)
        out = {name: t.find(q) for name, t in impls.items()}
        ov, of, osc = out["oracle"]
        assert of.sum() == batch // 2
        for name, (v, f, s) in out.items():
            np.testing.assert_array_equal(f, of, err_msg=name)
            np.testing.assert_array_equal(v.view(np.uint32), ov.view(np.uint32), err_msg=name)
            np.testing.assert_array_equal(s[f], osc[of], err_msg=name)
    close_all(impls)


def test_config1_lru_hit_miss_sets():
    """Same workload under LRU: scores come from the device timer, so found
    flags and values are compared, scores only for being non-decreasing
    across batches."""
    capacity, dim, batch = 1 << 20, 8, 65536
    impls = make_impls(capacity, dim, LRU)
    keys = unique_keys(capacity // 2 + batch, seed=12)
    present, fresh = keys[: capacity // 2], keys[capacity // 2:]
    for b in range(0, present.size, batch):
        k = present[b:b + batch]
        for t in impls.values():
            t.insert_or_assign(k, values_for(k, dim))
    assert_same_table(impls, with_scores=False)
    q = np.concatenate([present[:batch // 2], fresh[:batch // 2]])
    out = {name: t.find(q) for name, t in impls.items()}
    for name, (v, f, s) in out.items():
        np.testing.assert_array_equal(f, out["oracle"][1], err_msg=name)
        np.testing.assert_array_equal(v.view(np.uint32), out["oracle"][0].view(np.uint32))
    # product LRU scores: later batches carry later timestamps
    pk, _, ps = impls["product"].export_batch()
    order = {int(k): i for i, k in enumerate(present)}
    idx = np.array([order[int(k)] for k in pk])
    batch_id = idx // batch
    lo = np.array([ps[batch_id == b].min() for b in range(batch_id.max() + 1)])
    hi = np.array([ps[batch_id == b].max() for b in range(batch_id.max() + 1)])
    assert np.all(hi[:-1] <= lo[1:])
    close_all(impls)
