"""The C-ABI library without a GPU: it loads, exports every entry point that
include/hkv_b200.h declares, and its option checks (which run before any CUDA
call) raise the reference's exception types with the reference's messages."""
import ctypes
import os
import re

import pytest

import hierarchicalkv_b200 as hkv
from hierarchicalkv_b200 import table as tbl

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "hkv_b200.h")


def declared_entry_points():
    text = open(HEADER).read()
    return sorted(set(re.findall(r"HKV_API\s+[\w\s\*]+?\b(hkv_\w+)\s*\(", text)))


def test_header_declares_the_expected_surface():
    names = declared_entry_points()
    for must in ("hkv_table_create", "hkv_find", "hkv_find_ptr", "hkv_insert_or_assign",
                 "hkv_insert_and_evict", "hkv_find_or_insert", "hkv_find_or_insert_ptr",
                 "hkv_assign", "hkv_accum_or_assign", "hkv_export_batch", "hkv_export_batch_if",
                 "hkv_size", "hkv_load_factor", "hkv_clear", "hkv_last_error"):
        assert must in names


def test_library_exports_every_declared_symbol(product_lib):
    raw = ctypes.CDLL(hkv.library_path())
    for name in declared_entry_points():
        assert hasattr(raw, name), f"{name} is declared in hkv_b200.h but not exported"


def test_python_binding_covers_every_declared_symbol():
    assert sorted(tbl._SIGNATURES) == declared_entry_points()


def test_each_declaration_cites_the_reference():
    text = open(HEADER).read()
    blocks = re.split(r"\n\n", text)
    for b in blocks:
        if "HKV_API int hkv_" in b and "hkv_last_error" not in b:
            # these have no counterpart in the reference; all others cite a file:line
            if re.search(r"hkv_(get_view|device_status|external_begin|size_no_alloc|shard_|sharded_|"
                         r"promote_hot_buckets)\w*\b", b):
                continue
            assert re.search(r"include/merlin[\w/_.]*:\d+", b), b[:120]


@pytest.mark.parametrize("kwargs,exc,fragment", [
    (dict(reserved_key_start_bit=63), hkv.MerlinException, "reserved_key_start_bit"),
    (dict(reserved_key_start_bit=-1), hkv.MerlinException, "reserved_key_start_bit"),
    (dict(max_bucket_size=100), hkv.MerlinException, "pow of 2"),
    (dict(max_bucket_size=8), hkv.MerlinException, "between 16 and 1024"),
    (dict(max_bucket_size=2048, init_capacity=4096, max_capacity=4096), hkv.MerlinException,
     "between 16 and 1024"),
    (dict(table_mode=1, max_bucket_size=256), hkv.MerlinException, "max_bucket_size == 128"),
    (dict(num_of_buckets_per_alloc=3), hkv.MerlinException, "num_of_buckets_per_alloc"),
    (dict(init_capacity=128, max_capacity=128, num_of_buckets_per_alloc=2), hkv.MerlinException,
     "num_of_buckets_per_alloc"),
    (dict(io_by_cpu=True, max_hbm_for_vectors=1 << 20), hkv.MerlinException, "io_by_cpu"),
    # dual-bucket tables: include/merlin_hashtable.cuh:991-1015 of the reference
    (dict(table_mode=1, max_capacity=2048), hkv.MerlinException, "init_capacity must equal"),
    (dict(table_mode=1, max_hbm_for_vectors=1 << 20), hkv.MerlinException, "max_hbm_for_vectors = 0"),
    (dict(table_mode=1, init_capacity=128, max_capacity=128), hkv.MerlinException, "at least 2 buckets"),
    (dict(table_mode=1, dim=225), hkv.MerlinException, "896 bytes"),
    (dict(table_mode=2), hkv.MerlinException, "table_mode"),
])
def test_option_checks_raise_like_the_reference(product_lib, kwargs, exc, fragment):
    opts = dict(init_capacity=1024, max_capacity=1024, dim=4)
    opts.update(kwargs)
    t = hkv.HashTable(hkv.EvictStrategy.kLru)
    with pytest.raises(exc) as e:
        t.init(hkv.HashTableOptions(**opts))
    assert fragment in str(e.value)


def test_missing_library_fails_loudly(tmp_path):
    with pytest.raises(RuntimeError) as e:
        tbl.load_library(str(tmp_path / "libhkv_b200.so"))
    assert "no CPU or PyTorch fallback" in str(e.value)


def test_product_package_never_touches_the_oracle():
    """The oracle is test infrastructure: nothing under the package may import,
    link or open it."""
    pkg = os.path.join(ROOT, "hierarchicalkv_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h", ".cpp")):
                text = open(os.path.join(dirpath, f), errors="ignore").read()
                assert "hkv_oracle" not in text and "oracle/" not in text, f
    for f in ("merlin_hashtable.cuh", "hkv_b200.h"):
        p = os.path.join(ROOT, "include", f)
        if os.path.exists(p):
            assert "oracle" not in open(p).read()
