"""hkv_size_no_alloc against hkv_size, through the C ABI.

The no-allocation variant exists for callers whose set-up phase is over and
that may not allocate any more (a serving loop with a fixed memory budget, a
plug-in inside an application that owns all allocations).  Its partial sums
sit in a fixed array inside the library, shared by every call and never
cleared, so the check is made on two calls in a row with different table
contents: a stale value left by the first call would show in the second.

Collected last on purpose (file name), so a run that stops at the first
failure has already run every other test.
"""
import numpy as np
import pytest

from tests.hkv_testlib import ProductTable, unique_keys, values_for

pytestmark = pytest.mark.gpu


def test_size_no_alloc_matches_size_on_two_calls_in_a_row():
    cap, dim = 128 * 3000, 4          # 3000 buckets: three blocks of partial sums, the last ragged
    t = ProductTable(cap, dim, strategy=4)
    keys = unique_keys(150000, seed=77)
    first, second = keys[:100000], keys[100000:]
    t.insert_or_assign(first, values_for(first, dim), np.arange(1, first.size + 1, dtype=np.uint64))
    want = t.t.size()
    assert want == first.size
    assert t.t.size_no_alloc() == want          # integer result: exact
    t.insert_or_assign(second, values_for(second, dim),
                       np.arange(200001, 200001 + second.size, dtype=np.uint64))
    want2 = t.t.size()
    assert want2 == keys.size
    assert t.t.size_no_alloc() == want2
    # and once more after the table shrank, on a stream of its own
    import torch

    t.erase(first[:4321])
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        assert t.t.size_no_alloc(stream) == t.t.size(stream) == keys.size - 4321
    t.close()


def test_size_no_alloc_on_an_empty_and_a_tiny_table():
    t = ProductTable(128, 4, strategy=4)           # a single bucket
    assert t.t.size_no_alloc() == t.t.size() == 0
    k = unique_keys(50, seed=78)
    t.insert_or_assign(k, values_for(k, 4), np.arange(1, 51, dtype=np.uint64))
    assert t.t.size_no_alloc() == t.t.size() == 50
    t.close()
