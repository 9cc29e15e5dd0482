"""save / load across the two implementations.

The reference stores a table as three raw little-endian arrays without a
header -- keys (n x 8 bytes), values (n x dim x sizeof(V)), scores (n x 8) --
written by LocalKVFile (include/merlin_localfile.hpp:44-158 of the reference)
from HashTable::save / load (include/merlin_hashtable.cuh:3615-3758).  The
drop-in header claims the same format.  Both directions are checked here:

  * the reference's own save writes the files, the product's load (the C++
    client tests/cpp/ckpt_tool.cu, which uses the drop-in header) reads them;
  * the product's save writes the files, the reference's own load reads them;

and in both cases the loader's table must hold exactly what the files hold:
keys, rows and scores compared bit for bit after sorting by key.
"""
import os
import subprocess

import numpy as np
import pytest

from tests.hkv_testlib import (RefTable, ref_available, sorted_by_key, unique_keys, values_for)

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TOOL = os.path.join(ROOT, "tests", "cpp", "build", "ckpt_tool")
CUSTOMIZED = 4


def _tool(*args):
    if not os.path.exists(TOOL):
        subprocess.run(["make", "-C", os.path.join(ROOT, "tests", "cpp")], check=True)
    r = subprocess.run([TOOL, *[str(a) for a in args]], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    return r.stdout


def _read(prefix, dim, score_dtype=np.uint64):
    keys = np.fromfile(prefix + ".keys", dtype=np.uint64)
    values = np.fromfile(prefix + ".values", dtype=np.float32).reshape(-1, dim)
    scores = np.fromfile(prefix + ".scores", dtype=score_dtype)
    assert keys.size == values.shape[0] == scores.size
    return sorted_by_key(keys, values, scores.astype(np.uint64))


def _same(a, b):
    for x, y in zip(a, b):
        np.testing.assert_array_equal(x.view(np.uint8), y.view(np.uint8))


@pytest.mark.skipif(not ref_available(CUSTOMIZED), reason="the reference is not built")
def test_product_loads_what_the_reference_saved(tmp_path, product_lib):
    cap, dim, n = 128 * 64, 8, 6000
    ref = RefTable(cap, dim, CUSTOMIZED)
    keys = unique_keys(n, seed=501)
    scores = np.arange(1, n + 1, dtype=np.uint64) * np.uint64(3)
    ref.insert_or_assign(keys, values_for(keys, dim, seed=5), scores)
    prefix = str(tmp_path / "from_reference")
    assert ref.save(prefix, max_workspace_size=64 * 1024) == n
    written = _read(prefix, dim)
    _same(written, sorted_by_key(keys, values_for(keys, dim, seed=5), scores))
    out = str(tmp_path / "product_export")
    _tool("load", prefix, cap, dim, out, 8)
    _same(_read(out, dim), written)
    ref.close()


@pytest.mark.skipif(not ref_available(CUSTOMIZED), reason="the reference is not built")
def test_reference_loads_what_the_product_saved(tmp_path, product_lib):
    cap, dim, n = 128 * 64, 8, 6000
    prefix = str(tmp_path / "from_product")
    _tool("save", prefix, cap, dim, n, 77, 8)
    written = _read(prefix, dim)
    assert written[0].size == n and np.unique(written[0]).size == n
    ref = RefTable(cap, dim, CUSTOMIZED)
    assert ref.load(prefix, max_workspace_size=48 * 1024) == n
    assert ref.size() == n
    _same(sorted_by_key(*ref.export_batch()), written)
    ref.close()


def test_product_round_trip_with_32_bit_scores(tmp_path, product_lib):
    """sizeof(S) == 4 (Customized only): the score file holds n x 4 bytes."""
    cap, dim, n = 128 * 32, 4, 3000
    prefix = str(tmp_path / "u32")
    _tool("save", prefix, cap, dim, n, 78, 4)
    assert os.path.getsize(prefix + ".scores") == n * 4
    assert os.path.getsize(prefix + ".keys") == n * 8
    assert os.path.getsize(prefix + ".values") == n * dim * 4
    written = _read(prefix, dim, np.uint32)
    out = str(tmp_path / "u32_again")
    _tool("load", prefix, cap, dim, out, 4)
    _same(_read(out, dim, np.uint32), written)
