"""Host logic of the key-hash sharded table on CPU: two `gloo` ranks, the
routing (group by owner, all-to-all out and back, merge of duplicates that
meet at the owner, un-permutation) exercised with test doubles for the device
helpers and with the CPU oracle as each rank's sub-table.  The merged result
must equal one global oracle table fed the same batches in rank order."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from tests.hkv_testlib import OracleTable, fmix64, unique_keys, values_for  # noqa: E402

WORLD = 2
DIM = 4
CAP = 128 * 64


class CpuOps:
    """Stand-in for hierarchicalkv_b200.sharded.CudaOps on CPU tensors."""

    def partition(self, keys, world):
        k = keys.numpy().view(np.uint64)
        owner = (fmix64(k) % np.uint64(world)).astype(np.int64)
        order = np.argsort(owner, kind="stable")
        counts = np.bincount(owner, minlength=world).tolist()
        return counts, torch.from_numpy(k[order].view(np.int64).copy()), torch.from_numpy(order.astype(np.int32))

    def gather_rows(self, src, index):
        return src.index_select(0, index.long()).contiguous()

    def scatter_rows(self, src, index, dst):
        idx = index.long()
        keep = idx >= 0
        dst[idx[keep]] = src[keep]


class OracleLocal:
    """The CPU oracle behind the HashTable method names, on CPU tensors."""

    def __init__(self, capacity, dim, strategy):
        self.t = OracleTable(capacity, dim, strategy)

    @staticmethod
    def _k(t):
        return np.ascontiguousarray(t.numpy().view(np.uint64))

    def insert_or_assign(self, n, keys, values, scores=None, stream=None):
        self.t.insert_or_assign(self._k(keys[:n]), np.ascontiguousarray(values[:n].numpy()),
                                None if scores is None else self._k(scores[:n]))

    def find(self, n, keys, values, founds, scores=None, stream=None):
        v, f, s = self.t.find(self._k(keys[:n]))
        fi = torch.from_numpy(f)
        values[:n][fi] = torch.from_numpy(v)[fi]
        founds[:n] = fi
        if scores is not None:
            scores[:n][fi] = torch.from_numpy(s.view(np.int64))[fi]

    def find_or_insert(self, n, keys, values, scores=None, stream=None):
        out = self.t.find_or_insert(self._k(keys[:n]), np.ascontiguousarray(values[:n].numpy()),
                                    None if scores is None else self._k(scores[:n]))
        values[:n] = torch.from_numpy(out)

    def accum_or_assign(self, n, keys, values, flags, scores=None, stream=None):
        self.t.accum_or_assign(self._k(keys[:n]), np.ascontiguousarray(values[:n].numpy()),
                               np.ascontiguousarray(flags[:n].numpy()),
                               None if scores is None else self._k(scores[:n]))

    def size(self, stream=None):
        return self.t.size()


def batches():
    """Per-rank batches; ranks share some keys on purpose."""
    keys = unique_keys(6000, seed=321)
    shared = keys[:500]
    per_rank = []
    for r in range(WORLD):
        own = keys[1000 + r * 1500: 1000 + (r + 1) * 1500]
        ins = np.concatenate([own[:1000], shared[:300]])
        foi = np.concatenate([own[800:1400], shared[200:500]])     # hits, new keys, keys shared by both ranks
        acc = np.concatenate([own[:400], shared[:500], keys[5000 + r * 100: 5100 + r * 100]])
        flags = np.ones(acc.size, dtype=np.bool_)
        flags[::5] = False
        per_rank.append(dict(ins=ins, foi=foi, acc=acc, flags=flags, query=keys[: 5500]))
    return per_rank


def tv(a):
    return torch.from_numpy(a.view(np.int64) if a.dtype == np.uint64 else a)


def worker(rank, port):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=WORLD)
    from hierarchicalkv_b200.sharded import ShardedHashTable

    CUSTOMIZED = 4
    local = OracleLocal(CAP, DIM, CUSTOMIZED)
    st = ShardedHashTable(local, ops=CpuOps())
    assert st.world == WORLD and st.rank == rank
    b = batches()
    mine = b[rank]

    # the same sequence on one global table, batches merged in rank order,
    # a key that comes from both ranks taken once from the lower rank
    glob = OracleTable(CAP * WORLD, DIM, CUSTOMIZED)

    def merged(field, seed, with_flags=False):
        ks, vs, ss, fs = [], [], [], []
        seen = set()
        for r in range(WORLD):
            k = b[r][field]
            v = values_for(k, DIM, seed=seed + r)
            s = np.arange(1, k.size + 1, dtype=np.uint64) + np.uint64(100000 * (seed + 1))
            for i, kk in enumerate(k.tolist()):
                ks.append(kk)
                vs.append(v[i])
                ss.append(s[i])
                if with_flags:
                    fs.append(b[r]["flags"][i])
        return (np.array(ks, dtype=np.uint64), np.stack(vs), np.array(ss, dtype=np.uint64),
                np.array(fs, dtype=np.bool_))

    def first_occurrence(k):
        _, idx = np.unique(k, return_index=True)
        return np.sort(idx)

    # 1. insert_or_assign
    k = mine["ins"]
    s = np.arange(1, k.size + 1, dtype=np.uint64) + np.uint64(100000)
    st.insert_or_assign(k.size, tv(k), tv(values_for(k, DIM, seed=rank)), tv(s))
    gk, gv, gs, _ = merged("ins", 0)
    keep = first_occurrence(gk)
    glob.insert_or_assign(gk[keep], gv[keep], gs[keep])
    assert st.size() == glob.size()
    # every key lives on the rank that owns it
    lk, _, _ = local.t.export_batch()
    assert np.all((fmix64(lk) % np.uint64(WORLD)) == rank)

    # 2. find over everything
    q = mine["query"]
    vals = torch.full((q.size, DIM), -7.0)
    founds = torch.zeros(q.size, dtype=torch.bool)
    scores = torch.full((q.size,), -1, dtype=torch.int64)
    st.find(q.size, tv(q), vals, founds, scores)
    ev, ef, es = glob.find(q)
    np.testing.assert_array_equal(founds.numpy(), ef)
    np.testing.assert_array_equal(vals.numpy()[ef], ev[ef])
    assert np.all(vals.numpy()[~ef] == -7.0)            # misses untouched
    np.testing.assert_array_equal(scores.numpy().view(np.uint64)[ef], es[ef])

    # 3. find_or_insert: rows of hits come back, new keys take the lowest rank's row
    k = mine["foi"]
    v = tv(values_for(k, DIM, seed=10 + rank).copy())
    s = np.arange(1, k.size + 1, dtype=np.uint64) + np.uint64(100000 * 11)
    st.find_or_insert(k.size, tv(k), v, tv(s))
    gk, gv, gs, _ = merged("foi", 10)
    keep = first_occurrence(gk)
    gout = glob.find_or_insert(gk[keep], gv[keep], gs[keep])
    lookup = {int(kk): gout[i] for i, kk in enumerate(gk[keep].tolist())}
    want = np.stack([lookup[int(kk)] for kk in k.tolist()])
    np.testing.assert_array_equal(v.numpy(), want)
    assert st.size() == glob.size()

    # 4. accum_or_assign: deltas for a shared key add up in rank order
    k = mine["acc"]
    d = values_for(k, DIM, seed=20 + rank)
    s = np.arange(1, k.size + 1, dtype=np.uint64) + np.uint64(100000 * 21)
    st.accum_or_assign(k.size, tv(k), tv(d), tv(mine["flags"]), tv(s))
    gk, gv, gs, gf = merged("acc", 20, with_flags=True)
    keep = first_occurrence(gk)
    acc = {}
    for i, kk in enumerate(gk.tolist()):
        if gf[i]:
            acc[kk] = acc.get(kk, np.zeros(DIM, dtype=np.float32)) + gv[i]
    rows = np.stack([acc[kk] if gf[i] else gv[i] for i, kk in zip(keep, gk[keep].tolist())])
    glob.accum_or_assign(gk[keep], rows.astype(np.float32), gf[keep], gs[keep])
    assert st.size() == glob.size()
    vals = torch.zeros((q.size, DIM))
    st.find(q.size, tv(q), vals, founds, None)
    ev, ef, _ = glob.find(q)
    np.testing.assert_array_equal(founds.numpy(), ef)
    np.testing.assert_array_equal(vals.numpy()[ef].view(np.uint32), ev[ef].view(np.uint32))
    dist.barrier()
    dist.destroy_process_group()


def free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def test_sharded_table_two_gloo_ranks():
    mp.spawn(worker, args=(free_port(),), nprocs=WORLD, join=True)


def test_single_rank_is_the_local_table():
    from hierarchicalkv_b200.sharded import ShardedHashTable

    local = OracleLocal(CAP, DIM, 4)
    st = ShardedHashTable(local, ops=CpuOps())
    assert st.world == 1
    k = unique_keys(300, seed=5)
    s = np.arange(1, 301, dtype=np.uint64)
    st.insert_or_assign(300, tv(k), tv(values_for(k, DIM)), tv(s))
    vals = torch.zeros((300, DIM))
    founds = torch.zeros(300, dtype=torch.bool)
    st.find(300, tv(k), vals, founds)
    assert founds.all() and st.size() == 300
    np.testing.assert_array_equal(vals.numpy(), values_for(k, DIM))
