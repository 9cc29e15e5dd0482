"""Every scenario of tests/scenarios.py on the CUDA product (through the C
ABI), compared bit for bit with the CPU oracle, with the reference's own
kernels when they were built, and with the committed recordings of the
reference."""
import os

import numpy as np
import pytest

from tests.hkv_testlib import OracleTable, ProductTable, RefTable, ref_available
from tests.scenarios import build_scenarios, compare, flatten, run_scenario, table_kwargs

pytestmark = pytest.mark.gpu

SCENARIOS = build_scenarios()
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def unflatten(npz, n_steps):
    out = [dict() for _ in range(n_steps)]
    for name in npz.files:
        step, field = name.split(".")
        out[int(step[4:])][field] = npz[name]
    return out


@pytest.mark.parametrize("name", sorted(SCENARIOS))
def test_product_matches_oracle_and_reference(name):
    sc = SCENARIOS[name]
    kw = table_kwargs(sc)
    prod = ProductTable(sc["capacity"], sc["dim"], sc["strategy"], **kw)
    got = run_scenario(prod, sc)
    prod.close()
    want = run_scenario(OracleTable(sc["capacity"], sc["dim"], sc["strategy"], **kw), sc)
    compare(got, want, f"{name}: product vs oracle")
    if ref_available(sc["strategy"]):
        ref = RefTable(sc["capacity"], sc["dim"], sc["strategy"], **kw)
        live = run_scenario(ref, sc)
        ref.close()
        compare(got, live, f"{name}: product vs reference kernels")
    path = os.path.join(GOLDEN, f"ref_{name}.npz")
    if os.path.exists(path):
        compare(got, unflatten(np.load(path), len(sc["steps"])), f"{name}: product vs recording")


@pytest.mark.parametrize("name", sorted(SCENARIOS))
def test_product_serialising_kernel_matches_oracle(name):
    """unique_key=false routes through the kernel that tolerates repeated keys;
    on unique batches it must give the same results."""
    sc = SCENARIOS[name]
    kw = table_kwargs(sc)

    class NonUnique(ProductTable):
        def insert_or_assign(self, keys, values, scores=None, **kw):
            return super().insert_or_assign(keys, values, scores, unique_key=False)

        def find_or_insert(self, keys, values, scores=None, **kw):
            return super().find_or_insert(keys, values, scores, unique_key=False)

        def insert_and_evict(self, keys, values, scores=None, **kw):
            return super().insert_and_evict(keys, values, scores, unique_key=False)

    prod = NonUnique(sc["capacity"], sc["dim"], sc["strategy"], **kw)
    got = run_scenario(prod, sc)
    prod.close()
    want = run_scenario(OracleTable(sc["capacity"], sc["dim"], sc["strategy"], **kw), sc)
    compare(got, want, f"{name}: serialising kernel vs oracle")
