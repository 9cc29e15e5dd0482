"""The CPU oracle against what the reference itself computed.

* tests/golden/host_pins.json   -- printed by the reference's HOST functions
  (oracle/ref_host_pins.cu, built and run without a GPU);
* tests/golden/ref_device_pins.npz, ref_<scenario>.npz -- recorded from the
  reference's CUDA kernels on a B200 by tests/golden/make_ref_golden.py;
* known answers stated in the reference's own tests.
"""
import json
import os

import numpy as np
import pytest

from tests.hkv_testlib import OracleTable, fmix64, is_reserved, load_oracle, unique_keys, values_for
from tests.scenarios import build_scenarios, compare, run_scenario, table_kwargs

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
SCENARIOS = build_scenarios()


def test_hash_matches_reference_host_function():
    pins = json.load(open(os.path.join(GOLDEN, "host_pins.json")))
    lib = load_oracle()
    for key, want in pins["murmur3_host"].items():
        assert lib.orc_hash(int(key)) == int(want), key
    keys = np.array([int(k) for k in pins["murmur3_host"]], dtype=np.uint64)
    want = np.array([int(v) for v in pins["murmur3_host"].values()], dtype=np.uint64)
    np.testing.assert_array_equal(fmix64(keys), want)


def test_empty_key_per_start_bit_matches_reference_host_function():
    pins = json.load(open(os.path.join(GOLDEN, "host_pins.json")))
    lib = load_oracle()
    out = (np.zeros(7, dtype=np.uint64))
    for bit, want in enumerate(pins["empty_key_by_start_bit"]):
        lib.orc_reserved_keys(bit, out.ctypes.data_as(__import__("ctypes").POINTER(__import__("ctypes").c_uint64)))
        assert int(out[0]) == int(want), bit


def test_reserved_keys_and_digests_match_reference_device_code():
    """EMPTY / RECLAIM / LOCKED, their digests, per-key hash, digest and the
    IS_RESERVED_KEY truth value for reserved_key_start_bit 0..62, as the
    reference's device code computes them."""
    import ctypes

    pins = np.load(os.path.join(GOLDEN, "ref_device_pins.npz"))
    lib = load_oracle()
    out = np.zeros(7, dtype=np.uint64)
    for bit in range(63):
        lib.orc_reserved_keys(bit, out.ctypes.data_as(ctypes.POINTER(ctypes.c_uint64)))
        empty, reclaim, locked, edig, rdig = (int(x) for x in pins["constants"][bit])
        assert (int(out[0]), int(out[1]), int(out[2])) == (empty, reclaim, locked), bit
        assert (int(out[5]), int(out[6])) == (edig & 0xFF, rdig & 0xFF), bit
        keys = pins["keys"][bit]
        for k, h, d, r in zip(keys, pins["hashes"][bit], pins["digests"][bit], pins["reserved"][bit]):
            assert lib.orc_hash(int(k)) == int(h)
            assert (int(h) >> 32) & 0xFF == int(d)
            assert bool(lib.orc_is_reserved(bit, int(k))) == bool(r), (bit, hex(int(k)))
        np.testing.assert_array_equal(is_reserved(keys, bit), pins["reserved"][bit])


def test_reserved_key_truth_table_of_the_reference_test():
    """tests/reserved_keys_test.cc.cu:84-97: for every start bit EMPTY, RECLAIM
    and LOCKED are reserved, 0x0 and 0x10 are not, and the default EMPTY key is
    reserved only for bit 0."""
    import ctypes

    lib = load_oracle()
    out = np.zeros(7, dtype=np.uint64)
    for bit in range(63):
        lib.orc_reserved_keys(bit, out.ctypes.data_as(ctypes.POINTER(ctypes.c_uint64)))
        for k in out[:3]:
            assert lib.orc_is_reserved(bit, int(k)) == 1
        assert lib.orc_is_reserved(bit, 0x0) == 0
        assert lib.orc_is_reserved(bit, 0x10) == 0
        assert lib.orc_is_reserved(bit, 0xFFFFFFFFFFFFFFFF) == (1 if bit == 0 else 0)


def test_bucket_count_known_answer():
    """tests/merlin_hashtable_test.cc.cu:242-243: capacity 64Mi - 129 gives
    524287 buckets."""
    lib = load_oracle()
    cap = 64 * 1024 * 1024 - 129
    # only the arithmetic of create_table matters; a one-byte row keeps it light
    t = lib.orc_create(cap, cap, 1, 1, 0, 0)
    assert lib.orc_bucket_count(t) == 524287
    lib.orc_destroy(t)


@pytest.mark.parametrize("name", sorted(SCENARIOS))
def test_oracle_matches_recordings_of_the_reference_kernels(name):
    sc = SCENARIOS[name]
    path = os.path.join(GOLDEN, f"ref_{name}.npz")
    npz = np.load(path)
    want = [dict() for _ in sc["steps"]]
    for field in npz.files:
        step, what = field.split(".")
        want[int(step[4:])][what] = npz[field]
    got = run_scenario(OracleTable(sc["capacity"], sc["dim"], sc["strategy"], **table_kwargs(sc)),
                       sc)
    compare(got, want, f"{name}: oracle vs recording of the reference")
