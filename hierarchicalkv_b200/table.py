"""ctypes binding of include/hkv_b200.h and the HashTable mirror class.

Mirrors ``nv::merlin::HashTable<K, V, S, Strategy>`` of the reference
(include/merlin_hashtable.cuh:910-3892): method names, argument order,
defaults and the exceptions raised are the reference's; tensors replace raw
pointers.  Batch tensors must live on the table's device (or be mapped pinned
host memory), as the reference requires of its callers.
"""
from __future__ import annotations

import ctypes
import dataclasses
import enum
import os
from typing import Optional

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB: Optional[ctypes.CDLL] = None

GB = 1 << 30


class MerlinException(RuntimeError):
    """nv::merlin::MerlinException (include/merlin/debug.hpp:40-55)."""


class CudaException(RuntimeError):
    """nv::merlin::CudaException (include/merlin/debug.hpp:27-38)."""


class EvictStrategy(enum.IntEnum):
    """include/merlin_hashtable.cuh:79-87"""

    kLru = 0
    kLfu = 1
    kEpochLru = 2
    kEpochLfu = 3
    kCustomized = 4


class Predicate(enum.IntEnum):
    """Built-in predicates of export_batch_if / size_if (hkv_predicate)."""

    ALL = 0
    SCORE_LESS = 1
    SCORE_GREATER_EQ = 2
    KEY_MASK_EQ = 3
    SCORE_GREATER = 4
    SCORE_LESS_EQ = 5


class _Options(ctypes.Structure):
    _fields_ = [
        ("init_capacity", ctypes.c_uint64),
        ("max_capacity", ctypes.c_uint64),
        ("max_hbm_for_vectors", ctypes.c_uint64),
        ("max_bucket_size", ctypes.c_uint64),
        ("dim", ctypes.c_uint64),
        ("max_load_factor", ctypes.c_float),
        ("block_size", ctypes.c_int32),
        ("io_block_size", ctypes.c_int32),
        ("device_id", ctypes.c_int32),
        ("io_by_cpu", ctypes.c_int32),
        ("use_constant_memory", ctypes.c_int32),
        ("reserved_key_start_bit", ctypes.c_int32),
        ("num_of_buckets_per_alloc", ctypes.c_uint64),
        ("api_lock", ctypes.c_int32),
        ("table_mode", ctypes.c_int32),
        ("evict_strategy", ctypes.c_int32),
        ("value_size", ctypes.c_uint32),
        ("score_size", ctypes.c_uint32),
        ("value_kind", ctypes.c_uint32),
        ("slot_layout", ctypes.c_uint32),
    ]


class TableView(ctypes.Structure):
    """hkv_table_view"""

    _fields_ = [
        ("digests", ctypes.c_void_p),
        ("keys", ctypes.c_void_p),
        ("scores", ctypes.c_void_p),
        ("values_hbm", ctypes.c_void_p),
        ("values_host", ctypes.c_void_p),
        ("bucket_sizes", ctypes.c_void_p),
        ("bucket_map", ctypes.c_void_p),
        ("buckets", ctypes.c_uint64),
        ("capacity", ctypes.c_uint64),
        ("hbm_slots", ctypes.c_uint64),
        ("row_bytes", ctypes.c_uint64),
        ("empty_key", ctypes.c_uint64),
        ("reclaim_key", ctypes.c_uint64),
        ("locked_key", ctypes.c_uint64),
        ("reserved_mask", ctypes.c_uint64),
        ("reserved_value", ctypes.c_uint64),
        ("max_bucket_size", ctypes.c_uint64),
        ("slot_word_mask", ctypes.c_uint64),
    ]

    def slot_word(self, slot: int) -> int:
        """HKV_SLOT_WORD: index of slot's key in `keys` and of its score in `scores`"""
        return slot + ((slot & ~7) & self.slot_word_mask)


@dataclasses.dataclass
class HashTableOptions:
    """include/merlin_hashtable.cuh:103-136, same fields and defaults."""

    init_capacity: int = 0
    max_capacity: int = 0
    max_hbm_for_vectors: int = 0
    max_bucket_size: int = 128
    dim: int = 64
    max_load_factor: float = 0.5
    block_size: int = 128
    io_block_size: int = 1024
    device_id: int = -1
    io_by_cpu: bool = False
    use_constant_memory: bool = False
    reserved_key_start_bit: int = 0
    num_of_buckets_per_alloc: int = 1
    api_lock: bool = True
    table_mode: int = 0
    # not in the reference: 0 separate key and score arrays, 1 keys and scores of 8
    # slots share a 128-byte line (hkv_slot_layout)
    slot_layout: int = 0


def library_path() -> str:
    return os.path.join(_HERE, "libhkv_b200.so")


_P = ctypes.c_void_p
_U64 = ctypes.c_uint64
_INT = ctypes.c_int

# name -> argtypes (restype is int unless listed in _RESTYPES)
_SIGNATURES = {
    "hkv_table_create": [ctypes.POINTER(_Options), _P, ctypes.POINTER(_P)],
    "hkv_table_destroy": [_P],
    "hkv_insert_or_assign": [_P, _U64, _P, _P, _P, _P, _INT, _INT],
    "hkv_insert_and_evict": [_P, _U64, _P, _P, _P, _P, _P, _P, _P, _P, _INT, _INT],
    "hkv_insert_and_evict_count": [_P, _U64, _P, _P, _P, _P, _P, _P, _P, _INT, _INT,
                                   ctypes.POINTER(_U64)],
    "hkv_accum_or_assign": [_P, _U64, _P, _P, _P, _P, _P, _INT],
    "hkv_find_or_insert": [_P, _U64, _P, _P, _P, _P, _INT, _INT],
    "hkv_find_or_insert_ptr": [_P, _U64, _P, _P, _P, _P, _P, _INT, _INT, _P],
    "hkv_lock_keys": [_P, _U64, _P, _P, _P, _P, _P],
    "hkv_unlock_keys": [_P, _U64, _P, _P, _P, _P],
    "hkv_assign": [_P, _U64, _P, _P, _P, _P, _INT],
    "hkv_assign_scores": [_P, _U64, _P, _P, _P, _INT],
    "hkv_assign_values": [_P, _U64, _P, _P, _P, _INT],
    "hkv_find": [_P, _U64, _P, _P, _P, _P, _P],
    "hkv_find_host": [_P, _U64, _P, _P, _P, _P, _P],
    "hkv_find_missed": [_P, _U64, _P, _P, _P, _P, _P, _P, _P],
    "hkv_find_ptr": [_P, _U64, _P, _P, _P, _P, _P, _INT],
    "hkv_find_and_update": [_P, _U64, _P, _P, _P, _P, _P, _INT],
    "hkv_contains": [_P, _U64, _P, _P, _P],
    "hkv_erase": [_P, _U64, _P, _P],
    "hkv_erase_if": [_P, _INT, _U64, _U64, _P, ctypes.POINTER(_U64)],
    "hkv_clear": [_P, _P],
    "hkv_export_batch": [_P, _U64, _U64, _P, _P, _P, _P, _P],
    "hkv_export_batch_count": [_P, _U64, _U64, _P, _P, _P, _P, ctypes.POINTER(_U64)],
    "hkv_export_batch_if": [_P, _INT, _U64, _U64, _U64, _U64, _P, _P, _P, _P, _P],
    "hkv_size_if": [_P, _INT, _U64, _U64, _P, _P],
    "hkv_size": [_P, _P, ctypes.POINTER(_U64)],
    "hkv_load_factor": [_P, _P, ctypes.POINTER(ctypes.c_float)],
    "hkv_shard_partition": [_U64, _P, ctypes.c_uint32, _P, _P, _P, _P, _P, _P],
    "hkv_shard_gather_rows": [_U64, _U64, _P, _P, _P, _P],
    "hkv_shard_scatter_rows": [_U64, _U64, _P, _P, _P, _P],
    "hkv_shard_last_error": [],
    "hkv_shard_route_keys_p2p": [_U64, _P, ctypes.c_uint32, ctypes.c_uint32, _U64, _P, _P, _P, _P, _P],
    "hkv_shard_barrier": [ctypes.c_uint32, ctypes.c_uint32, _P, ctypes.c_uint32, _P,
                          ctypes.c_uint32, _P],
    "hkv_find_routed": [_P, ctypes.c_uint32, ctypes.c_uint32, _U64, _P, _P, _P, _P, _P, _P],
    "hkv_upsert_routed": [_P, ctypes.c_int, ctypes.c_uint32, ctypes.c_uint32, _U64, _P, _P, _P, _P,
                          _P, _P],
    "hkv_sharded_create": [_P, ctypes.c_uint32, ctypes.c_uint32, _U64, ctypes.c_uint32,
                           ctypes.POINTER(_P)],
    "hkv_sharded_destroy": [_P],
    "hkv_sharded_lanes": [_P],
    "hkv_sharded_max_batch": [_P],
    "hkv_sharded_ipc_handle": [_P, ctypes.c_uint32, _P],
    "hkv_sharded_connect_ipc": [_P, ctypes.c_uint32, _P],
    "hkv_sharded_workspace": [_P, ctypes.c_uint32],
    "hkv_sharded_workspace_bytes": [_P, ctypes.c_uint32, _U64, _P],
    "hkv_sharded_create_external": [_P, ctypes.c_uint32, ctypes.c_uint32, _U64, ctypes.c_uint32, _P, _P],
    "hkv_sharded_connect_pointers": [_P, ctypes.c_uint32, _P],
    "hkv_sharded_buffers": [_P, ctypes.c_uint32, ctypes.POINTER(_P), ctypes.POINTER(_P)],
    "hkv_sharded_find": [_P, ctypes.c_uint32, _U64, _P, ctypes.c_uint32, _P],
    "hkv_sharded_find_async": [_P, _U64, _P, ctypes.c_uint32, _P, ctypes.POINTER(ctypes.c_uint32)],
    "hkv_sharded_wait": [_P, ctypes.c_uint32, _P],
    "hkv_sharded_upsert": [_P, _INT, _U64, _P, _INT, ctypes.c_uint32, _P],
    "hkv_sharded_status": [_P, ctypes.c_uint32, _P, ctypes.POINTER(ctypes.c_uint32)],
    "hkv_sharded_last_error": [],
    "hkv_accum_or_assign_unique": [_P, _U64, _P, _P, _P, _P, _P, _INT],
    "hkv_size_no_alloc": [_P, _P, ctypes.POINTER(_U64)],
    "hkv_size_no_alloc_last_error": [],
    "hkv_capacity": [_P],
    "hkv_bucket_count": [_P],
    "hkv_dim": [_P],
    "hkv_max_bucket_size": [_P],
    "hkv_set_global_epoch": [_P, _U64],
    "hkv_reserve": [_P, _U64, _P],
    "hkv_set_max_capacity": [_P, _U64],
    "hkv_promote_hot_buckets": [_P, _P, ctypes.POINTER(ctypes.c_uint64)],
    "hkv_get_view": [_P, ctypes.POINTER(TableView)],
    "hkv_external_begin": [_P, _INT, _P],
    "hkv_external_end": [_P, _INT, _P],
    "hkv_device_status": [_P, _P, ctypes.POINTER(ctypes.c_uint32)],
    "hkv_last_error": [],
}
_RESTYPES = {
    "hkv_sharded_lanes": ctypes.c_uint32,
    "hkv_sharded_max_batch": _U64,
    "hkv_sharded_workspace": _P,
    "hkv_sharded_last_error": ctypes.c_char_p,
    "hkv_capacity": _U64,
    "hkv_bucket_count": _U64,
    "hkv_dim": _U64,
    "hkv_max_bucket_size": _U64,
    "hkv_last_error": ctypes.c_char_p,
    "hkv_size_no_alloc_last_error": ctypes.c_char_p,
    "hkv_shard_last_error": ctypes.c_char_p,
}


def load_library(path: Optional[str] = None) -> ctypes.CDLL:
    """Loads libhkv_b200.so; raises if it was not built (no fallback exists)."""
    global _LIB
    if _LIB is not None and path is None:
        return _LIB
    p = path or library_path()
    if not os.path.exists(p):
        raise RuntimeError(
            f"{p} is missing: build it with `python -m hierarchicalkv_b200.build` "
            "(there is no CPU or PyTorch fallback for the table operations)")
    lib = ctypes.CDLL(p)
    for name, argtypes in _SIGNATURES.items():
        fn = getattr(lib, name)
        fn.argtypes = argtypes
        fn.restype = _RESTYPES.get(name, ctypes.c_int)
    if path is None:
        _LIB = lib
    return lib


def _raise(lib: ctypes.CDLL, rc: int) -> None:
    msg = (lib.hkv_last_error() or b"").decode()
    if rc == 1:
        raise MerlinException(msg)
    if rc == 2:
        raise CudaException(msg)
    if rc == 4:
        raise ValueError(msg)  # std::invalid_argument
    if rc == 5:
        raise NotImplementedError(msg)
    raise RuntimeError(msg)  # std::runtime_error


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    if t is None:
        return None
    if not t.is_contiguous():
        raise ValueError("batch tensors must be contiguous")
    return t.data_ptr()


def _stream(stream) -> Optional[int]:
    if stream is None:
        return torch.cuda.current_stream().cuda_stream or None
    if isinstance(stream, int):
        return stream or None
    return stream.cuda_stream or None


_VALUE_SIZES = {
    torch.float32: 4, torch.float64: 8, torch.float16: 2, torch.bfloat16: 2,
    torch.int32: 4, torch.int64: 8, torch.int16: 2, torch.int8: 1, torch.uint8: 1,
}


# hkv_value_kind: the element types accum_or_assign can add
_VALUE_KINDS = {
    torch.float32: 1, torch.float64: 2, torch.int32: 3, torch.int64: 4, torch.float16: 5,
    torch.bfloat16: 6,
}


class HashTable:
    """Mirror of nv::merlin::HashTable<K, V, S, Strategy>.

    K is a 64-bit integer (torch.int64 tensors carry uint64 bit patterns),
    S is uint64 (carried as torch.int64) or, with kCustomized only, uint32
    (``score_dtype=torch.int32``: every score tensor is then int32), V is
    ``value_dtype``.
    """

    def __init__(self, evict_strategy: EvictStrategy = EvictStrategy.kLru,
                 value_dtype: torch.dtype = torch.float32,
                 score_dtype: torch.dtype = torch.int64):
        self.evict_strategy = EvictStrategy(evict_strategy)
        self.value_dtype = value_dtype
        if score_dtype not in (torch.int64, torch.int32):
            raise ValueError("The score_type must be uint64_t or uint32_t.")
        self.score_dtype = score_dtype
        self._lib = load_library()
        self._h = ctypes.c_void_p()
        self._opts: Optional[HashTableOptions] = None

    # -- life cycle -------------------------------------------------------
    def init(self, options: HashTableOptions) -> None:
        """HashTable::init, include/merlin_hashtable.cuh:984-1089 (idempotent)."""
        if self._h:
            return
        o = _Options(
            init_capacity=options.init_capacity, max_capacity=options.max_capacity,
            max_hbm_for_vectors=options.max_hbm_for_vectors,
            max_bucket_size=options.max_bucket_size, dim=options.dim,
            max_load_factor=options.max_load_factor, block_size=options.block_size,
            io_block_size=options.io_block_size, device_id=options.device_id,
            io_by_cpu=int(options.io_by_cpu),
            use_constant_memory=int(options.use_constant_memory),
            reserved_key_start_bit=options.reserved_key_start_bit,
            num_of_buckets_per_alloc=options.num_of_buckets_per_alloc,
            api_lock=int(options.api_lock), table_mode=int(options.table_mode),
            evict_strategy=int(self.evict_strategy),
            value_size=_VALUE_SIZES[self.value_dtype],
            score_size=8 if self.score_dtype == torch.int64 else 4,
            value_kind=_VALUE_KINDS.get(self.value_dtype, 0),
            slot_layout=int(getattr(options, "slot_layout", 0)))
        h = ctypes.c_void_p()
        rc = self._lib.hkv_table_create(ctypes.byref(o), None, ctypes.byref(h))
        if rc:
            _raise(self._lib, rc)
        self._h = h
        self._opts = options

    def close(self) -> None:
        if self._h:
            self._lib.hkv_table_destroy(self._h)
            self._h = ctypes.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _call(self, name: str, *args):
        rc = getattr(self._lib, name)(self._h, *args)
        if rc:
            _raise(self._lib, rc)

    # -- insert-like --------------------------------------------------------
    def insert_or_assign(self, n, keys, values, scores=None, stream=None, unique_key=True,
                         ignore_evict_strategy=False) -> None:
        self._call("hkv_insert_or_assign", n, _ptr(keys), _ptr(values), _ptr(scores),
                   _stream(stream), int(unique_key), int(ignore_evict_strategy))

    def insert_and_evict(self, n, keys, values, scores, evicted_keys, evicted_values,
                         evicted_scores, d_evicted_counter=None, stream=None, unique_key=True,
                         ignore_evict_strategy=False):
        """With ``d_evicted_counter`` (caller-zeroed) returns None; without it
        returns the evicted count and synchronises, as the two reference
        overloads do (include/merlin_hashtable.cuh:1351, 1518)."""
        if d_evicted_counter is not None:
            self._call("hkv_insert_and_evict", n, _ptr(keys), _ptr(values), _ptr(scores),
                       _ptr(evicted_keys), _ptr(evicted_values), _ptr(evicted_scores),
                       _ptr(d_evicted_counter), _stream(stream), int(unique_key),
                       int(ignore_evict_strategy))
            return None
        cnt = ctypes.c_uint64(0)
        self._call("hkv_insert_and_evict_count", n, _ptr(keys), _ptr(values), _ptr(scores),
                   _ptr(evicted_keys), _ptr(evicted_values), _ptr(evicted_scores),
                   _stream(stream), int(unique_key), int(ignore_evict_strategy),
                   ctypes.byref(cnt))
        return cnt.value

    def accum_or_assign(self, n, keys, value_or_deltas, accum_or_assigns, scores=None,
                        stream=None, ignore_evict_strategy=False) -> None:
        self._call("hkv_accum_or_assign", n, _ptr(keys), _ptr(value_or_deltas),
                   _ptr(accum_or_assigns), _ptr(scores), _stream(stream),
                   int(ignore_evict_strategy))

    def accum_or_assign_unique(self, n, keys, value_or_deltas, accum_or_assigns, scores=None,
                               stream=None, ignore_evict_strategy=False) -> None:
        """accum_or_assign for batches that hold each key once (hkv_accum_or_assign_unique)."""
        self._call("hkv_accum_or_assign_unique", n, _ptr(keys), _ptr(value_or_deltas),
                   _ptr(accum_or_assigns), _ptr(scores), _stream(stream),
                   int(ignore_evict_strategy))

    def find_or_insert(self, n, keys, values, scores=None, stream=None, unique_key=True,
                       ignore_evict_strategy=False) -> None:
        self._call("hkv_find_or_insert", n, _ptr(keys), _ptr(values), _ptr(scores),
                   _stream(stream), int(unique_key), int(ignore_evict_strategy))

    def find_or_insert_ptr(self, n, keys, value_ptrs, founds, scores=None, stream=None,
                           unique_key=True, ignore_evict_strategy=False,
                           locked_key_ptrs=None) -> None:
        """Pointer form of find_or_insert; ``value_ptrs`` is an int64 tensor of
        device addresses."""
        self._call("hkv_find_or_insert_ptr", n, _ptr(keys), _ptr(value_ptrs), _ptr(founds),
                   _ptr(scores), _stream(stream), int(unique_key), int(ignore_evict_strategy),
                   _ptr(locked_key_ptrs))

    def lock_keys(self, n, keys, locked_key_ptrs, success=None, stream=None, scores=None):
        self._call("hkv_lock_keys", n, _ptr(keys), _ptr(locked_key_ptrs), _ptr(success),
                   _stream(stream), _ptr(scores))

    def unlock_keys(self, n, locked_key_ptrs, keys, success=None, stream=None):
        self._call("hkv_unlock_keys", n, _ptr(locked_key_ptrs), _ptr(keys), _ptr(success),
                   _stream(stream))

    # -- update-like --------------------------------------------------------
    def assign(self, n, keys, values, scores=None, stream=None, unique_key=True) -> None:
        self._call("hkv_assign", n, _ptr(keys), _ptr(values), _ptr(scores), _stream(stream),
                   int(unique_key))

    def assign_scores(self, n, keys, scores=None, stream=None, unique_key=True) -> None:
        self._call("hkv_assign_scores", n, _ptr(keys), _ptr(scores), _stream(stream),
                   int(unique_key))

    def assign_values(self, n, keys, values, stream=None, unique_key=True) -> None:
        self._call("hkv_assign_values", n, _ptr(keys), _ptr(values), _stream(stream),
                   int(unique_key))

    # -- read-like ----------------------------------------------------------
    def find(self, n, keys, values, founds, scores=None, stream=None) -> None:
        self._call("hkv_find", n, _ptr(keys), _ptr(values), _ptr(founds), _ptr(scores),
                   _stream(stream))

    def find_host(self, n, keys, values, founds, scores=None, stream=None) -> None:
        """find for a batch in host memory (CPU tensors, pinned for asynchronous
        copies): chunks of the batch alternate over two internal streams, so the
        key copies and lookups run under the row copies.  The host buffers are
        complete once `stream` has passed the call; rows of misses are zero."""
        self._call("hkv_find_host", n, _ptr(keys), _ptr(values), _ptr(founds), _ptr(scores),
                   _stream(stream))

    def find_missed(self, n, keys, values, missed_keys, missed_indices, missed_size,
                    scores=None, stream=None) -> None:
        """find overload returning the compacted misses
        (include/merlin_hashtable.cuh:2600)."""
        self._call("hkv_find_missed", n, _ptr(keys), _ptr(values), _ptr(missed_keys),
                   _ptr(missed_indices), _ptr(missed_size), _ptr(scores), _stream(stream))

    def find_ptr(self, n, keys, value_ptrs, founds, scores=None, stream=None,
                 unique_key=True) -> None:
        self._call("hkv_find_ptr", n, _ptr(keys), _ptr(value_ptrs), _ptr(founds), _ptr(scores),
                   _stream(stream), int(unique_key))

    def find_and_update(self, n, keys, value_ptrs, founds, scores=None, stream=None,
                        unique_key=True) -> None:
        self._call("hkv_find_and_update", n, _ptr(keys), _ptr(value_ptrs), _ptr(founds),
                   _ptr(scores), _stream(stream), int(unique_key))

    def contains(self, n, keys, founds, stream=None) -> None:
        self._call("hkv_contains", n, _ptr(keys), _ptr(founds), _stream(stream))

    # -- erase / clear ------------------------------------------------------
    def erase(self, n, keys, stream=None) -> None:
        self._call("hkv_erase", n, _ptr(keys), _stream(stream))

    def erase_if(self, pred, pattern, threshold, stream=None) -> int:
        """erase_if with a built-in predicate; returns the number of erased keys."""
        out = ctypes.c_uint64(0)
        self._call("hkv_erase_if", int(pred), pattern, threshold, _stream(stream),
                   ctypes.byref(out))
        return out.value

    def clear(self, stream=None) -> None:
        self._call("hkv_clear", _stream(stream))

    # -- export -------------------------------------------------------------
    def export_batch(self, n, offset, d_counter, keys, values, scores=None, stream=None):
        """With ``d_counter`` enqueues and returns None; with ``d_counter=None``
        returns the count and synchronises (include/merlin_hashtable.cuh:3099, 3131)."""
        if d_counter is not None:
            self._call("hkv_export_batch", n, offset, _ptr(d_counter), _ptr(keys), _ptr(values),
                       _ptr(scores), _stream(stream))
            return None
        cnt = ctypes.c_uint64(0)
        self._call("hkv_export_batch_count", n, offset, _ptr(keys), _ptr(values), _ptr(scores),
                   _stream(stream), ctypes.byref(cnt))
        return cnt.value

    def export_batch_if(self, pred, pattern, threshold, n, offset, d_counter, keys, values,
                        scores=None, stream=None) -> None:
        self._call("hkv_export_batch_if", int(pred), pattern, threshold, n, offset,
                   _ptr(d_counter), _ptr(keys), _ptr(values), _ptr(scores), _stream(stream))

    def size_if(self, pred, pattern, threshold, d_counter, stream=None) -> None:
        self._call("hkv_size_if", int(pred), pattern, threshold, _ptr(d_counter), _stream(stream))

    # -- observers ----------------------------------------------------------
    def size(self, stream=None) -> int:
        out = ctypes.c_uint64(0)
        self._call("hkv_size", _stream(stream), ctypes.byref(out))
        return out.value

    def size_no_alloc(self, stream=None) -> int:
        """size() for callers that must not allocate (see hkv_size_no_alloc in
        include/hkv_b200.h for who they are and for the limits)."""
        out = ctypes.c_uint64(0)
        rc = self._lib.hkv_size_no_alloc(self._h, _stream(stream), ctypes.byref(out))
        if rc:
            msg = (self._lib.hkv_size_no_alloc_last_error() or b"").decode()
            if rc == 2:
                raise CudaException(msg)
            if rc == 4:
                raise ValueError(msg)
            raise RuntimeError(msg)
        return out.value

    def empty(self, stream=None) -> bool:
        return self.size(stream) == 0

    def load_factor(self, stream=None) -> float:
        out = ctypes.c_float(0)
        self._call("hkv_load_factor", _stream(stream), ctypes.byref(out))
        return out.value

    def capacity(self) -> int:
        return self._lib.hkv_capacity(self._h)

    def bucket_count(self) -> int:
        return self._lib.hkv_bucket_count(self._h)

    def dim(self) -> int:
        return self._lib.hkv_dim(self._h)

    def max_bucket_size(self) -> int:
        return self._lib.hkv_max_bucket_size(self._h)

    def set_global_epoch(self, epoch: int) -> None:
        self._call("hkv_set_global_epoch", epoch)

    def reserve(self, new_capacity: int, stream=None) -> None:
        self._call("hkv_reserve", new_capacity, _stream(stream))

    def promote_hot_buckets(self, stream=None) -> int:
        """Hybrid tables: moves the rows of the most looked-up host-resident
        buckets into HBM (no counterpart in the reference).  Returns how many."""
        out = ctypes.c_uint64(0)
        self._call("hkv_promote_hot_buckets", _stream(stream), ctypes.byref(out))
        return out.value

    def set_max_capacity(self, new_max_capacity: int) -> None:
        """Raises ValueError (std::invalid_argument in the reference) unless a power of two."""
        self._call("hkv_set_max_capacity", new_max_capacity)

    def view(self) -> TableView:
        v = TableView()
        self._call("hkv_get_view", ctypes.byref(v))
        return v

    def device_status(self, stream=None) -> int:
        out = ctypes.c_uint32(0)
        self._call("hkv_device_status", _stream(stream), ctypes.byref(out))
        return out.value

    @property
    def handle(self) -> ctypes.c_void_p:
        return self._h
