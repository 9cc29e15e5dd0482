"""The C++ host of the sharded table (include/hkv_sharded.hpp over the
hkv_sharded_* entry points): tests/cpp/sharded_test.cu run as one process per
GPU.  The processes exchange the CUDA IPC handles of their peer workspaces
through files and check insert_or_assign, find (plain and pipelined over two
lanes), find_or_insert and accum_or_assign against what one global table would
hold, bit for bit."""
import os
import subprocess

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BINARY = os.path.join(ROOT, "tests", "cpp", "build", "sharded_test")

pytestmark = pytest.mark.gpu


def _run(world, tmp_path, *extra):
    if not os.path.exists(BINARY):
        subprocess.run(["make", "-C", os.path.join(ROOT, "tests", "cpp")], check=True)
    procs = [subprocess.Popen([BINARY, str(r), str(world), str(tmp_path), *extra],
                              stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
             for r in range(world)]
    outs = []
    for p in procs:
        try:
            out, _ = p.communicate(timeout=240)
        except subprocess.TimeoutExpired:
            for q in procs:
                q.kill()
            raise
        outs.append(out)
    for r, (p, out) in enumerate(zip(procs, outs)):
        assert p.returncode == 0, f"rank {r}:\n{out}"
        assert f"rank {r} PASS" in out


def test_one_rank_is_the_local_table(tmp_path, product_lib):
    _run(1, tmp_path)


def test_workspaces_supplied_by_the_caller(tmp_path, product_lib):
    """hkv_sharded_create_external: the library adopts memory it did not
    allocate, cannot export it and does not free it."""
    _run(1, tmp_path, "external")


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_processes_match_one_global_table(tmp_path, product_lib):
    _run(2, tmp_path)
