"""hierarchicalkv_b200 -- B200-native hash-table hot path of HierarchicalKV.

The product is ``libhkv_b200.so`` (hand-written sm_100a CUDA kernels behind
the C ABI declared in ``include/hkv_b200.h``) and the drop-in C++ header
``include/merlin_hashtable.cuh``.  This package is the Python mirror of the
reference's ``nv::merlin::HashTable`` interface over that C ABI: same method
names, argument order and error behaviour, with torch tensors standing in
for device pointers.  There is no CPU fallback: importing works without a
GPU, every table operation needs the CUDA library and a device.
"""
from .table import (  # noqa: F401
    CudaException,
    EvictStrategy,
    HashTable,
    HashTableOptions,
    MerlinException,
    Predicate,
    library_path,
    load_library,
)

__all__ = [
    "CudaException",
    "EvictStrategy",
    "HashTable",
    "HashTableOptions",
    "MerlinException",
    "Predicate",
    "library_path",
    "load_library",
]
