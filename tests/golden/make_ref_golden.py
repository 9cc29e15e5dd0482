"""Regenerates the golden vectors under tests/golden/ from the REFERENCE.

Run on a machine with a GPU and the compiled reference (oracle/_ref, built by
`make -C oracle ref` where the reference checkout is present):

    python tests/golden/make_ref_golden.py [output_dir]

It plays every scenario of tests/scenarios.py on the reference's own CUDA
kernels (through oracle/ref_shim.cu) and stores the normalised outputs as
ref_<scenario>.npz; it also asks the reference's device code for its reserved
keys, digests and hashes (ref_device_pins.npz).  The CPU tests then hold the
oracle to these recordings without needing a GPU or the reference.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from tests.hkv_testlib import RefTable, load_ref, to_dev  # noqa: E402
from tests.scenarios import build_scenarios, flatten, run_scenario, table_kwargs  # noqa: E402


def device_pins(out_dir: str) -> None:
    import torch

    lib = load_ref(4, private=True)
    consts = np.zeros((63, 5), dtype=np.uint64)
    probe_keys = [0, 1, 42, 0x10, 0xFFFFFFFFFFFFFFFF, 0xFFFFFFFFFFFFFFFE, 0xFFFFFFFFFFFFFFFD,
                  0xFFFFFFFFFFFFFFFC, 0xFFFFFFFFFFFFFFFB, 0x0123456789ABCDEF]
    rows = []
    for bit in range(63):  # bit 0 first: the reference cannot go back to the defaults
        d = torch.zeros(5, dtype=torch.int64, device="cuda")
        assert lib.ref_probe_reserved(bit, d.data_ptr()) == 0
        consts[bit] = d.cpu().numpy().view(np.uint64)
        keys = np.array(probe_keys + [int(x) for x in consts[bit][:3]], dtype=np.uint64)
        k = to_dev(keys)
        h = torch.zeros(keys.size, dtype=torch.int64, device="cuda")
        dg = torch.zeros(keys.size, dtype=torch.uint8, device="cuda")
        rs = torch.zeros(keys.size, dtype=torch.bool, device="cuda")
        assert lib.ref_probe_keys(keys.size, k.data_ptr(), h.data_ptr(), dg.data_ptr(),
                                  rs.data_ptr()) == 0
        rows.append((keys, h.cpu().numpy().view(np.uint64), dg.cpu().numpy(), rs.cpu().numpy()))
    np.savez_compressed(
        os.path.join(out_dir, "ref_device_pins.npz"), constants=consts,
        keys=np.stack([r[0] for r in rows]), hashes=np.stack([r[1] for r in rows]),
        digests=np.stack([r[2] for r in rows]), reserved=np.stack([r[3] for r in rows]))


def main() -> None:
    out_dir = sys.argv[1] if len(sys.argv) > 1 else os.path.join(ROOT, "tests", "golden")
    os.makedirs(out_dir, exist_ok=True)
    device_pins(out_dir)
    for name, sc in build_scenarios().items():
        t = RefTable(sc["capacity"], sc["dim"], sc["strategy"], **table_kwargs(sc))
        res = run_scenario(t, sc)
        t.close()
        np.savez_compressed(os.path.join(out_dir, f"ref_{name}.npz"), **flatten(res))
        print("wrote", name, len(res), "steps")


if __name__ == "__main__":
    main()
