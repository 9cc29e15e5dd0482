"""Shared test helpers: seeded inputs, the CPU oracle and the compiled
reference behind ctypes.  Only tests, the smoke check and the CPU-baseline leg
of the benchmark import this module."""
from __future__ import annotations

import ctypes
import os
import subprocess
from typing import Optional

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ORACLE_DIR = os.path.join(ROOT, "oracle")
ORACLE_SO = os.path.join(ORACLE_DIR, "libhkv_oracle.so")
REF_DIR = os.path.join(ORACLE_DIR, "_ref")

_P = ctypes.c_void_p
_U64 = ctypes.c_uint64
_INT = ctypes.c_int


# ---------------------------------------------------------------------------
# seeded inputs
# ---------------------------------------------------------------------------
def unique_keys(n: int, seed: int, reserved_key_start_bit: int = 0, lo_bits: int = 64) -> np.ndarray:
    """n distinct uint64 keys drawn uniformly from a seed, none of them reserved."""
    rng = np.random.default_rng(seed)
    out = np.empty(0, dtype=np.uint64)
    while out.size < n:
        k = rng.integers(0, 2**63, size=int(n * 1.1) + 16, dtype=np.uint64)
        k = (k << np.uint64(1)) | rng.integers(0, 2, size=k.size, dtype=np.uint64)
        if lo_bits < 64:
            k &= np.uint64((1 << lo_bits) - 1)
        k = k[~is_reserved(k, reserved_key_start_bit)]
        out = np.unique(np.concatenate([out, k]))
    rng.shuffle(out)
    return np.ascontiguousarray(out[:n])


def is_reserved(keys: np.ndarray, bit: int = 0) -> np.ndarray:
    if bit == 0:
        mask = np.uint64(0xFFFFFFFFFFFFFFFC)
        return (keys & mask) == mask
    m1 = np.uint64(~(3 << bit) & 0xFFFFFFFFFFFFFFFF)
    m2 = m1 & np.uint64(0xFFFFFFFFFFFFFFFE)
    return (keys & m1) == m2


def values_for(keys: np.ndarray, dim: int, seed: int = 0) -> np.ndarray:
    """float32 rows in U(-1, 1), a function of (key, column, seed) only."""
    k = keys.astype(np.uint64)[:, None] * np.uint64(0x9E3779B97F4A7C15)
    c = (np.arange(dim, dtype=np.uint64)[None, :] + np.uint64(seed * 1000003 + 1)) * np.uint64(
        0xBF58476D1CE4E5B9)
    x = k ^ c
    x ^= x >> np.uint64(31)
    x *= np.uint64(0x94D049BB133111EB)
    x ^= x >> np.uint64(29)
    u = (x >> np.uint64(40)).astype(np.float64) / float(1 << 24)
    return np.ascontiguousarray((u * 2.0 - 1.0).astype(np.float32))


def fmix64(keys: np.ndarray) -> np.ndarray:
    k = keys.astype(np.uint64).copy()
    k ^= k >> np.uint64(33)
    k *= np.uint64(0xFF51AFD7ED558CCD)
    k ^= k >> np.uint64(33)
    k *= np.uint64(0xC4CEB9FE1A85EC53)
    k ^= k >> np.uint64(33)
    return k


def bucket_of(keys: np.ndarray, capacity: int) -> np.ndarray:
    return (fmix64(keys) % np.uint64(capacity)) // np.uint64(128)


# ---------------------------------------------------------------------------
# CPU oracle
# ---------------------------------------------------------------------------
_ORACLE_SIGS = {
    "orc_create": ([_U64, _U64, _U64, ctypes.c_uint32, _INT, _INT], _P),
    "orc_create_sized": ([_U64, _U64, _U64, ctypes.c_uint32, _INT, _INT, _INT], _P),
    "orc_destroy": ([_P], None),
    "orc_reserve": ([_P, _U64], None),
    "orc_set_max_capacity": ([_P, _U64], _INT),
    "orc_set_max_load_factor": ([_P, ctypes.c_float], None),
    "orc_set_value_kind": ([_P, _INT], None),
    "orc_set_dual_bucket": ([_P], None),
    "orc_capacity": ([_P], _U64),
    "orc_bucket_count": ([_P], _U64),
    "orc_set_global_epoch": ([_P, _U64], None),
    "orc_set_clock": ([_P, _U64], None),
    "orc_size": ([_P], _U64),
    "orc_clear": ([_P], None),
    "orc_hash": ([_U64], _U64),
    "orc_locate": ([_P, _U64, ctypes.POINTER(_U64), ctypes.POINTER(ctypes.c_uint32),
                    ctypes.POINTER(ctypes.c_uint32)], None),
    "orc_reserved_keys": ([_INT, ctypes.POINTER(_U64)], None),
    "orc_is_reserved": ([_INT, _U64], _INT),
    "orc_find": ([_P, _U64, _P, _P, _P, _P, _INT], None),
    "orc_contains": ([_P, _U64, _P, _P], None),
    "orc_insert_or_assign": ([_P, _U64, _P, _P, _P, _INT, _INT], None),
    "orc_find_or_insert": ([_P, _U64, _P, _P, _P, _INT], None),
    "orc_find_or_insert_ptr": ([_P, _U64, _P, _P, _P], None),
    "orc_insert_and_evict": ([_P, _U64, _P, _P, _P, _P, _P, _P, ctypes.POINTER(_U64), _INT], None),
    "orc_accum_or_assign": ([_P, _U64, _P, _P, _P, _P, _INT], None),
    "orc_assign": ([_P, _INT, _U64, _P, _P, _P], None),
    "orc_erase": ([_P, _U64, _P], None),
    "orc_export_batch_if": ([_P, _INT, _U64, _U64, _U64, _U64, _P, _P, _P], _U64),
    "orc_erase_if": ([_P, _INT, _U64, _U64], _U64),
    "orc_bucket_min_score": ([_P, _U64], _U64),
    "orc_hardware_threads": ([], _INT),
}
_oracle = None


def load_oracle() -> ctypes.CDLL:
    global _oracle
    if _oracle is not None:
        return _oracle
    src = os.path.join(ORACLE_DIR, "hkv_oracle.cpp")
    if not os.path.exists(ORACLE_SO) or os.path.getmtime(ORACLE_SO) < os.path.getmtime(src):
        subprocess.run(["make", "-C", ORACLE_DIR, "libhkv_oracle.so"], check=True,
                       capture_output=True)
    lib = ctypes.CDLL(ORACLE_SO)
    for name, (args, res) in _ORACLE_SIGS.items():
        fn = getattr(lib, name)
        fn.argtypes = args
        fn.restype = res
    _oracle = lib
    return lib


def _np(a: Optional[np.ndarray]):
    if a is None:
        return None
    assert a.flags["C_CONTIGUOUS"]
    return a.ctypes.data


class OracleTable:
    """Sequential CPU model with the reference's method names (numpy in/out)."""

    def __init__(self, capacity: int, dim: int, strategy: int = 0, reserved_key_start_bit: int = 0,
                 max_capacity: Optional[int] = None, value_size: int = 4,
                 max_load_factor: Optional[float] = None, memory_mode: bool = False,
                 max_bucket_size: int = 128):
        self.lib = load_oracle()
        self.dim = dim
        self.strategy = strategy
        self.h = self.lib.orc_create_sized(capacity, max_capacity or capacity, dim, value_size,
                                           strategy, reserved_key_start_bit, max_bucket_size)
        if max_load_factor is not None:
            self.lib.orc_set_max_load_factor(self.h, max_load_factor)
        if memory_mode:
            self.lib.orc_set_dual_bucket(self.h)

    def reserve(self, new_capacity):
        self.lib.orc_reserve(self.h, new_capacity)

    def set_max_capacity(self, new_max_capacity):
        if not self.lib.orc_set_max_capacity(self.h, new_max_capacity):
            raise ValueError("None power-of-2 new_max_capacity is not supported.")

    def __del__(self):
        if getattr(self, "h", None):
            self.lib.orc_destroy(self.h)
            self.h = None

    def capacity(self):
        return self.lib.orc_capacity(self.h)

    def bucket_count(self):
        return self.lib.orc_bucket_count(self.h)

    def size(self):
        return self.lib.orc_size(self.h)

    def clear(self):
        self.lib.orc_clear(self.h)

    def set_global_epoch(self, e):
        self.lib.orc_set_global_epoch(self.h, e)

    def set_clock(self, now):
        self.lib.orc_set_clock(self.h, now)

    def insert_or_assign(self, keys, values, scores=None, ignore_evict_strategy=False, threads=1):
        self.lib.orc_insert_or_assign(self.h, keys.size, _np(keys), _np(values), _np(scores),
                                      int(ignore_evict_strategy), threads)

    def find(self, keys, with_scores=True, threads=1):
        n = keys.size
        values = np.zeros((n, self.dim), dtype=np.float32)
        founds = np.zeros(n, dtype=np.bool_)
        scores = np.zeros(n, dtype=np.uint64) if with_scores else None
        self.lib.orc_find(self.h, n, _np(keys), _np(values), _np(founds), _np(scores), threads)
        return values, founds, scores

    def contains(self, keys):
        founds = np.zeros(keys.size, dtype=np.bool_)
        self.lib.orc_contains(self.h, keys.size, _np(keys), _np(founds))
        return founds

    def find_or_insert(self, keys, values, scores=None, threads=1):
        values = np.ascontiguousarray(values).copy()
        self.lib.orc_find_or_insert(self.h, keys.size, _np(keys), _np(values), _np(scores), threads)
        return values

    def find_or_insert_ptr(self, keys, scores=None):
        founds = np.zeros(keys.size, dtype=np.bool_)
        self.lib.orc_find_or_insert_ptr(self.h, keys.size, _np(keys), _np(founds), _np(scores))
        return founds

    def insert_and_evict(self, keys, values, scores=None, threads=1):
        n = keys.size
        ek = np.zeros(n, dtype=np.uint64)
        ev = np.zeros((n, self.dim), dtype=np.float32)
        es = np.zeros(n, dtype=np.uint64)
        cnt = _U64(0)
        self.lib.orc_insert_and_evict(self.h, n, _np(keys), _np(values), _np(scores), _np(ek),
                                      _np(ev), _np(es), ctypes.byref(cnt), threads)
        c = cnt.value
        return ek[:c], ev[:c], es[:c]

    def accum_or_assign(self, keys, values, flags, scores=None, threads=1):
        self.lib.orc_accum_or_assign(self.h, keys.size, _np(keys), _np(values), _np(flags),
                                     _np(scores), threads)

    def assign(self, keys, values, scores=None):
        self.lib.orc_assign(self.h, 0, keys.size, _np(keys), _np(values), _np(scores))

    def assign_scores(self, keys, scores=None):
        self.lib.orc_assign(self.h, 1, keys.size, _np(keys), None, _np(scores))

    def assign_values(self, keys, values):
        self.lib.orc_assign(self.h, 2, keys.size, _np(keys), _np(values), None)

    def erase(self, keys):
        self.lib.orc_erase(self.h, keys.size, _np(keys))

    def erase_if(self, pred, pattern, threshold):
        return self.lib.orc_erase_if(self.h, pred, pattern, threshold)

    def export_batch_if(self, pred=0, pattern=0, threshold=0, n=None, offset=0):
        cap = self.capacity()
        n = cap if n is None else n
        m = min(n, max(cap - offset, 0))
        keys = np.zeros(m, dtype=np.uint64)
        values = np.zeros((m, self.dim), dtype=np.float32)
        scores = np.zeros(m, dtype=np.uint64)
        c = self.lib.orc_export_batch_if(self.h, pred, pattern, threshold, n, offset, _np(keys),
                                         _np(values), _np(scores))
        return keys[:c], values[:c], scores[:c]

    def export_batch(self, n=None, offset=0):
        return self.export_batch_if(0, 0, 0, n, offset)

    def bucket_min_score(self, key: int) -> int:
        return self.lib.orc_bucket_min_score(self.h, key)


def sorted_by_key(keys, values, scores):
    order = np.argsort(keys, kind="stable")
    return keys[order], values[order], scores[order]


# ---------------------------------------------------------------------------
# GPU wrappers (import torch lazily so the CPU tests stay light)
# ---------------------------------------------------------------------------
def to_dev(a: np.ndarray):
    import torch

    if a.dtype == np.uint64:
        a = a.view(np.int64)
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def to_np_u64(t) -> np.ndarray:
    return t.cpu().numpy().view(np.uint64)


class ProductTable:
    """numpy-in / numpy-out convenience over hierarchicalkv_b200.HashTable for
    the parity tests (every call goes through the C ABI)."""

    def __init__(self, capacity, dim, strategy=0, reserved_key_start_bit=0, max_capacity=None,
                 max_hbm_for_vectors=None, api_lock=True, max_load_factor=None,
                 memory_mode=False, max_bucket_size=128, slot_layout=None):
        import torch
        import hierarchicalkv_b200 as hkv

        if slot_layout is None:     # HKV_TEST_SLOT_LAYOUT=1 runs the whole suite on shared lines
            slot_layout = int(os.environ.get("HKV_TEST_SLOT_LAYOUT", "0"))

        self.torch = torch
        self.dim = dim
        self.t = hkv.HashTable(hkv.EvictStrategy(strategy))
        hbm = (16 << 30) if max_hbm_for_vectors is None else max_hbm_for_vectors
        extra = {} if max_load_factor is None else {"max_load_factor": max_load_factor}
        if memory_mode:          # the reference's dual-bucket tables want max_hbm_for_vectors == 0
            extra["table_mode"] = 1
            hbm = 0
        self.t.init(hkv.HashTableOptions(
            init_capacity=capacity, max_capacity=max_capacity or capacity,
            max_hbm_for_vectors=hbm, dim=dim, reserved_key_start_bit=reserved_key_start_bit,
            api_lock=api_lock, max_bucket_size=max_bucket_size, slot_layout=slot_layout, **extra))

    def reserve(self, new_capacity):
        self.t.reserve(new_capacity, self.torch.cuda.current_stream().cuda_stream)

    def set_max_capacity(self, new_max_capacity):
        self.t.set_max_capacity(new_max_capacity)

    def close(self):
        self.t.close()

    def capacity(self):
        return self.t.capacity()

    def bucket_count(self):
        return self.t.bucket_count()

    def size(self):
        return self.t.size()

    def clear(self):
        self.t.clear()

    def set_global_epoch(self, e):
        self.t.set_global_epoch(e)

    def insert_or_assign(self, keys, values, scores=None, unique_key=True,
                         ignore_evict_strategy=False):
        k, v = to_dev(keys), to_dev(values)
        s = to_dev(scores) if scores is not None else None
        self.t.insert_or_assign(keys.size, k, v, s, unique_key=unique_key,
                                ignore_evict_strategy=ignore_evict_strategy)
        self.torch.cuda.synchronize()

    def find(self, keys, with_scores=True):
        torch = self.torch
        n = keys.size
        k = to_dev(keys)
        v = torch.zeros((n, self.dim), dtype=torch.float32, device="cuda")
        f = torch.zeros(n, dtype=torch.bool, device="cuda")
        s = torch.zeros(n, dtype=torch.int64, device="cuda") if with_scores else None
        self.t.find(n, k, v, f, s)
        torch.cuda.synchronize()
        return v.cpu().numpy(), f.cpu().numpy(), (to_np_u64(s) if with_scores else None)

    def find_missed(self, keys):
        torch = self.torch
        n = keys.size
        k = to_dev(keys)
        v = torch.zeros((n, self.dim), dtype=torch.float32, device="cuda")
        mk = torch.zeros(n, dtype=torch.int64, device="cuda")
        mi = torch.zeros(n, dtype=torch.int32, device="cuda")
        ms = torch.zeros(1, dtype=torch.int32, device="cuda")
        self.t.find_missed(n, k, v, mk, mi, ms)
        torch.cuda.synchronize()
        c = int(ms.item())
        return v.cpu().numpy(), to_np_u64(mk)[:c], mi.cpu().numpy()[:c]

    def find_ptr(self, keys):
        torch = self.torch
        n = keys.size
        k = to_dev(keys)
        p = torch.zeros(n, dtype=torch.int64, device="cuda")
        f = torch.zeros(n, dtype=torch.bool, device="cuda")
        s = torch.zeros(n, dtype=torch.int64, device="cuda")
        self.t.find_ptr(n, k, p, f, s)
        torch.cuda.synchronize()
        return p.cpu().numpy(), f.cpu().numpy(), to_np_u64(s)

    def contains(self, keys):
        torch = self.torch
        k = to_dev(keys)
        f = torch.zeros(keys.size, dtype=torch.bool, device="cuda")
        self.t.contains(keys.size, k, f)
        torch.cuda.synchronize()
        return f.cpu().numpy()

    def find_or_insert(self, keys, values, scores=None, unique_key=True):
        k, v = to_dev(keys), to_dev(values)
        s = to_dev(scores) if scores is not None else None
        self.t.find_or_insert(keys.size, k, v, s, unique_key=unique_key)
        self.torch.cuda.synchronize()
        return v.cpu().numpy()

    def find_or_insert_ptr(self, keys, scores=None):
        torch = self.torch
        n = keys.size
        k = to_dev(keys)
        p = torch.zeros(n, dtype=torch.int64, device="cuda")
        f = torch.zeros(n, dtype=torch.bool, device="cuda")
        s = to_dev(scores) if scores is not None else None
        self.t.find_or_insert_ptr(n, k, p, f, s)
        torch.cuda.synchronize()
        return p.cpu().numpy(), f.cpu().numpy()

    def insert_and_evict(self, keys, values, scores=None, unique_key=True, use_counter=True):
        torch = self.torch
        n = keys.size
        k, v = to_dev(keys), to_dev(values)
        s = to_dev(scores) if scores is not None else None
        ek = torch.zeros(n, dtype=torch.int64, device="cuda")
        ev = torch.zeros((n, self.dim), dtype=torch.float32, device="cuda")
        es = torch.zeros(n, dtype=torch.int64, device="cuda")
        if use_counter:
            c = torch.zeros(1, dtype=torch.int64, device="cuda")
            self.t.insert_and_evict(n, k, v, s, ek, ev, es, c, unique_key=unique_key)
            torch.cuda.synchronize()
            cnt = int(c.item())
        else:
            cnt = self.t.insert_and_evict(n, k, v, s, ek, ev, es, None, unique_key=unique_key)
        return to_np_u64(ek)[:cnt], ev.cpu().numpy()[:cnt], to_np_u64(es)[:cnt]

    def accum_or_assign(self, keys, values, flags, scores=None):
        k, v, f = to_dev(keys), to_dev(values), to_dev(flags)
        s = to_dev(scores) if scores is not None else None
        self.t.accum_or_assign(keys.size, k, v, f, s)
        self.torch.cuda.synchronize()

    def assign(self, keys, values, scores=None):
        k, v = to_dev(keys), to_dev(values)
        s = to_dev(scores) if scores is not None else None
        self.t.assign(keys.size, k, v, s)
        self.torch.cuda.synchronize()

    def assign_scores(self, keys, scores=None):
        s = to_dev(scores) if scores is not None else None
        self.t.assign_scores(keys.size, to_dev(keys), s)
        self.torch.cuda.synchronize()

    def assign_values(self, keys, values):
        self.t.assign_values(keys.size, to_dev(keys), to_dev(values))
        self.torch.cuda.synchronize()

    def erase(self, keys):
        self.t.erase(keys.size, to_dev(keys))
        self.torch.cuda.synchronize()

    def erase_if(self, pred, pattern, threshold):
        return self.t.erase_if(pred, pattern, threshold)

    def export_batch_if(self, pred=0, pattern=0, threshold=0, n=None, offset=0):
        torch = self.torch
        cap = self.capacity()
        n = cap if n is None else n
        m = max(min(n, cap - offset), 0)
        k = torch.zeros(max(m, 1), dtype=torch.int64, device="cuda")
        v = torch.zeros((max(m, 1), self.dim), dtype=torch.float32, device="cuda")
        s = torch.zeros(max(m, 1), dtype=torch.int64, device="cuda")
        c = torch.zeros(1, dtype=torch.int64, device="cuda")
        self.t.export_batch_if(pred, pattern, threshold, n, offset, c, k, v, s)
        torch.cuda.synchronize()
        cnt = int(c.item())
        return to_np_u64(k)[:cnt], v.cpu().numpy()[:cnt], to_np_u64(s)[:cnt]

    def export_batch(self, n=None, offset=0):
        return self.export_batch_if(0, 0, 0, n, offset)


# ---------------------------------------------------------------------------
# the reference itself, compiled behind oracle/ref_shim.cu
# ---------------------------------------------------------------------------
def ref_available(strategy: int = 0) -> bool:
    return os.path.exists(os.path.join(REF_DIR, f"libhkv_ref_s{strategy}.so"))


_ref_libs = {}


def load_ref(strategy: int, private: bool = False) -> ctypes.CDLL:
    """private=True loads a fresh copy of the library: the reference keeps its
    reserved keys in __constant__ memory of the loaded module, so a table with
    a non-default reserved_key_start_bit changes them for every later table of
    that module (include/merlin/types.cuh:80-109)."""
    if strategy in _ref_libs and not private:
        return _ref_libs[strategy]
    path = os.path.join(REF_DIR, f"libhkv_ref_s{strategy}.so")
    if private:
        import shutil
        import tempfile

        tmp = tempfile.NamedTemporaryFile(prefix=f"hkv_ref_s{strategy}_", suffix=".so", delete=False)
        tmp.close()
        shutil.copyfile(path, tmp.name)
        path = tmp.name
    lib = ctypes.CDLL(path, mode=ctypes.RTLD_LOCAL)
    lib.ref_last_error.restype = ctypes.c_char_p
    sig = {
        "ref_create": [_U64, _U64, _U64, _U64, _U64, _INT, _INT, ctypes.POINTER(_P)],
        "ref_destroy": [_P],
        "ref_create_growable": [_U64, _U64, _U64, _U64, ctypes.c_float, ctypes.POINTER(_P)],
        "ref_reserve": [_P, _U64, _P],
        "ref_save": [_P, ctypes.c_char_p, _U64, _P, ctypes.POINTER(_U64)],
        "ref_load": [_P, ctypes.c_char_p, _U64, _P, ctypes.POINTER(_U64)],
        "ref_set_max_capacity": [_P, _U64],
        "ref_create_memory_mode": [_U64, _U64, ctypes.POINTER(_P)],
        "ref_set_global_epoch": [_P, _U64],
        "ref_insert_or_assign": [_P, _U64, _P, _P, _P, _P, _INT],
        "ref_insert_and_evict": [_P, _U64, _P, _P, _P, _P, _P, _P, _P, _P, _INT],
        "ref_accum_or_assign": [_P, _U64, _P, _P, _P, _P, _P],
        "ref_find_or_insert": [_P, _U64, _P, _P, _P, _P, _INT],
        "ref_find_or_insert_ptr": [_P, _U64, _P, _P, _P, _P, _P, _INT],
        "ref_assign": [_P, _U64, _P, _P, _P, _P, _INT],
        "ref_assign_scores": [_P, _U64, _P, _P, _P, _INT],
        "ref_find": [_P, _U64, _P, _P, _P, _P, _P],
        "ref_find_missed": [_P, _U64, _P, _P, _P, _P, _P, _P, _P],
        "ref_find_ptr": [_P, _U64, _P, _P, _P, _P, _P, _INT],
        "ref_contains": [_P, _U64, _P, _P, _P],
        "ref_erase": [_P, _U64, _P, _P],
        "ref_export_batch": [_P, _U64, _U64, _P, _P, _P, _P, _P],
        "ref_export_batch_if": [_P, _INT, _U64, _U64, _U64, _U64, _P, _P, _P, _P, _P],
        "ref_size": [_P, _P, ctypes.POINTER(_U64)],
        "ref_capacity": [_P, ctypes.POINTER(_U64)],
        "ref_bucket_count": [_P, ctypes.POINTER(_U64)],
        "ref_load_factor": [_P, _P, ctypes.POINTER(ctypes.c_float)],
        "ref_clear": [_P, _P],
    }
    sig["ref_probe_reserved"] = [_INT, _P]
    sig["ref_probe_keys"] = [_U64, _P, _P, _P, _P]
    for name, args in sig.items():
        fn = getattr(lib, name)
        fn.argtypes = args
        fn.restype = _INT
    if not private:
        _ref_libs[strategy] = lib
    return lib


class RefTable:
    """The unmodified reference (its own CUDA kernels) with numpy in/out."""

    # ref_shim predicate numbers for the product's Predicate values
    _PRED = {1: 0, 2: 1, 3: 2}

    def __init__(self, capacity, dim, strategy=0, reserved_key_start_bit=0, max_capacity=None,
                 max_hbm_for_vectors=None, api_lock=True, max_load_factor=None,
                 memory_mode=False, max_bucket_size=128):
        import torch

        self.torch = torch
        self.dim = dim
        self.lib = load_ref(strategy, private=reserved_key_start_bit != 0)
        self.h = _P()
        hbm = (16 << 30) if max_hbm_for_vectors is None else max_hbm_for_vectors
        if memory_mode:
            assert reserved_key_start_bit == 0 and api_lock and max_capacity in (None, capacity)
            self._chk(self.lib.ref_create_memory_mode(capacity, dim, ctypes.byref(self.h)))
        elif max_load_factor is not None:
            assert reserved_key_start_bit == 0 and api_lock
            self._chk(self.lib.ref_create_growable(capacity, max_capacity or capacity, hbm, dim,
                                                   max_load_factor, ctypes.byref(self.h)))
        else:
            self._chk(self.lib.ref_create(capacity, max_capacity or capacity, hbm, dim,
                                          max_bucket_size, reserved_key_start_bit, int(api_lock),
                                          ctypes.byref(self.h)))

    def reserve(self, new_capacity):
        self._chk(self.lib.ref_reserve(self.h, new_capacity, self._s()))

    def save(self, prefix: str, max_workspace_size: int = 1 << 20) -> int:
        """HashTable::save into <prefix>.keys / .values / .scores with the reference's LocalKVFile"""
        out = _U64(0)
        self._chk(self.lib.ref_save(self.h, prefix.encode(), max_workspace_size, self._s(),
                                    ctypes.byref(out)))
        return out.value

    def load(self, prefix: str, max_workspace_size: int = 1 << 20) -> int:
        out = _U64(0)
        self._chk(self.lib.ref_load(self.h, prefix.encode(), max_workspace_size, self._s(),
                                    ctypes.byref(out)))
        return out.value

    def set_max_capacity(self, new_max_capacity):
        rc = self.lib.ref_set_max_capacity(self.h, new_max_capacity)
        if rc == 1:
            raise ValueError((self.lib.ref_last_error() or b"").decode())
        self._chk(rc)

    def _chk(self, rc):
        if rc:
            raise RuntimeError("reference: " + (self.lib.ref_last_error() or b"").decode())

    def _s(self):
        return self.torch.cuda.current_stream().cuda_stream or None

    def close(self):
        if self.h:
            self.lib.ref_destroy(self.h)
            self.h = _P()

    def capacity(self):
        o = _U64(0)
        self._chk(self.lib.ref_capacity(self.h, ctypes.byref(o)))
        return o.value

    def bucket_count(self):
        o = _U64(0)
        self._chk(self.lib.ref_bucket_count(self.h, ctypes.byref(o)))
        return o.value

    def size(self):
        o = _U64(0)
        self._chk(self.lib.ref_size(self.h, self._s(), ctypes.byref(o)))
        return o.value

    def clear(self):
        self._chk(self.lib.ref_clear(self.h, self._s()))
        self.torch.cuda.synchronize()

    def set_global_epoch(self, e):
        self._chk(self.lib.ref_set_global_epoch(self.h, e))

    @staticmethod
    def _p(t):
        return None if t is None else t.data_ptr()

    def insert_or_assign(self, keys, values, scores=None, unique_key=True):
        k, v = to_dev(keys), to_dev(values)
        s = to_dev(scores) if scores is not None else None
        self._chk(self.lib.ref_insert_or_assign(self.h, keys.size, self._p(k), self._p(v),
                                                self._p(s), self._s(), int(unique_key)))
        self.torch.cuda.synchronize()

    def find(self, keys, with_scores=True):
        torch = self.torch
        n = keys.size
        k = to_dev(keys)
        v = torch.zeros((n, self.dim), dtype=torch.float32, device="cuda")
        f = torch.zeros(n, dtype=torch.bool, device="cuda")
        s = torch.zeros(n, dtype=torch.int64, device="cuda") if with_scores else None
        self._chk(self.lib.ref_find(self.h, n, self._p(k), self._p(v), self._p(f), self._p(s),
                                    self._s()))
        torch.cuda.synchronize()
        return v.cpu().numpy(), f.cpu().numpy(), (to_np_u64(s) if with_scores else None)

    def find_or_insert(self, keys, values, scores=None, unique_key=True):
        k, v = to_dev(keys), to_dev(values)
        s = to_dev(scores) if scores is not None else None
        self._chk(self.lib.ref_find_or_insert(self.h, keys.size, self._p(k), self._p(v),
                                              self._p(s), self._s(), int(unique_key)))
        self.torch.cuda.synchronize()
        return v.cpu().numpy()

    def insert_and_evict(self, keys, values, scores=None, unique_key=True):
        torch = self.torch
        n = keys.size
        k, v = to_dev(keys), to_dev(values)
        s = to_dev(scores) if scores is not None else None
        ek = torch.zeros(n, dtype=torch.int64, device="cuda")
        ev = torch.zeros((n, self.dim), dtype=torch.float32, device="cuda")
        es = torch.zeros(n, dtype=torch.int64, device="cuda")
        c = torch.zeros(1, dtype=torch.int64, device="cuda")
        self._chk(self.lib.ref_insert_and_evict(self.h, n, self._p(k), self._p(v), self._p(s),
                                                self._p(ek), self._p(ev), self._p(es), self._p(c),
                                                self._s(), int(unique_key)))
        torch.cuda.synchronize()
        cnt = int(c.item())
        return to_np_u64(ek)[:cnt], ev.cpu().numpy()[:cnt], to_np_u64(es)[:cnt]

    def accum_or_assign(self, keys, values, flags, scores=None):
        k, v, f = to_dev(keys), to_dev(values), to_dev(flags)
        s = to_dev(scores) if scores is not None else None
        self._chk(self.lib.ref_accum_or_assign(self.h, keys.size, self._p(k), self._p(v),
                                               self._p(f), self._p(s), self._s()))
        self.torch.cuda.synchronize()

    def assign(self, keys, values, scores=None):
        k, v = to_dev(keys), to_dev(values)
        s = to_dev(scores) if scores is not None else None
        self._chk(self.lib.ref_assign(self.h, keys.size, self._p(k), self._p(v), self._p(s),
                                      self._s(), 1))
        self.torch.cuda.synchronize()

    def assign_scores(self, keys, scores=None):
        k = to_dev(keys)
        s = to_dev(scores) if scores is not None else None
        self._chk(self.lib.ref_assign_scores(self.h, keys.size, self._p(k), self._p(s), self._s(),
                                             1))
        self.torch.cuda.synchronize()

    def contains(self, keys):
        torch = self.torch
        k = to_dev(keys)
        f = torch.zeros(keys.size, dtype=torch.bool, device="cuda")
        self._chk(self.lib.ref_contains(self.h, keys.size, self._p(k), self._p(f), self._s()))
        torch.cuda.synchronize()
        return f.cpu().numpy()

    def erase(self, keys):
        k = to_dev(keys)
        self._chk(self.lib.ref_erase(self.h, keys.size, self._p(k), self._s()))
        self.torch.cuda.synchronize()

    def export_batch_if(self, pred=0, pattern=0, threshold=0, n=None, offset=0):
        torch = self.torch
        cap = self.capacity()
        n = cap if n is None else n
        m = max(min(n, cap - offset), 0)
        k = torch.zeros(max(m, 1), dtype=torch.int64, device="cuda")
        v = torch.zeros((max(m, 1), self.dim), dtype=torch.float32, device="cuda")
        s = torch.zeros(max(m, 1), dtype=torch.int64, device="cuda")
        c = torch.zeros(1, dtype=torch.int64, device="cuda")
        if pred == 0:
            self._chk(self.lib.ref_export_batch(self.h, n, offset, self._p(c), self._p(k),
                                                self._p(v), self._p(s), self._s()))
        else:
            self._chk(self.lib.ref_export_batch_if(self.h, self._PRED[pred], pattern, threshold, n,
                                                   offset, self._p(c), self._p(k), self._p(v),
                                                   self._p(s), self._s()))
        torch.cuda.synchronize()
        cnt = int(c.item())
        return to_np_u64(k)[:cnt], v.cpu().numpy()[:cnt], to_np_u64(s)[:cnt]

    def export_batch(self, n=None, offset=0):
        return self.export_batch_if(0, 0, 0, n, offset)
