"""The sharding helpers and the sharded table on GPUs: router kernels against
numpy on one GPU, a world of one rank against the plain table, and (when the
box has two or more GPUs) two NCCL ranks against one global CPU oracle."""
import os
import socket
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from tests.hkv_testlib import OracleTable, fmix64, to_dev, to_np_u64, unique_keys, values_for  # noqa: E402

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("world", [1, 2, 3, 8, 64])
@pytest.mark.parametrize("n", [1, 255, 256, 100003])
def test_partition_groups_keys_by_owner(world, n):
    from hierarchicalkv_b200.sharded import CudaOps

    ops = CudaOps()
    keys = unique_keys(n, seed=n + world)
    counts, grouped, origin = ops.partition(to_dev(keys), world)
    owner = (fmix64(keys) % np.uint64(world)).astype(np.int64)
    assert counts == np.bincount(owner, minlength=world).tolist()
    g = to_np_u64(grouped)
    o = origin.cpu().numpy().astype(np.int64)
    np.testing.assert_array_equal(keys[o], g)                 # origin points at the key's place
    assert np.unique(o).size == n                              # a permutation
    bounds = np.concatenate([[0], np.cumsum(counts)])
    for r in range(world):
        seg = g[bounds[r]:bounds[r + 1]]
        assert np.all((fmix64(seg) % np.uint64(world)) == r)


@pytest.mark.parametrize("shape,dtype", [((1000, 64), torch.float32), ((1000, 3), torch.float32),
                                         ((777,), torch.uint8), ((513,), torch.int64)])
def test_gather_and_scatter_rows(shape, dtype):
    from hierarchicalkv_b200.sharded import CudaOps

    ops = CudaOps()
    n = shape[0]
    rng = np.random.default_rng(1)
    src = torch.from_numpy(rng.integers(0, 100, size=shape)).to(dtype).cuda()
    perm = torch.from_numpy(rng.permutation(n).astype(np.int32)).cuda()
    got = ops.gather_rows(src, perm)
    torch.cuda.synchronize()
    assert torch.equal(got, src[perm.long()])
    dst = torch.zeros_like(src)
    ops.scatter_rows(src, perm, dst)
    torch.cuda.synchronize()
    want = torch.zeros_like(src)
    want[perm.long()] = src
    assert torch.equal(dst, want)
    # rows with index -1 are skipped
    masked = perm.clone()
    masked[::3] = -1
    dst.fill_(7)
    ops.scatter_rows(src, masked, dst)
    torch.cuda.synchronize()
    want = torch.full_like(src, 7)
    keep = masked >= 0
    want[masked[keep].long()] = src[keep]
    assert torch.equal(dst, want)


def test_world_of_one_is_the_local_table():
    import hierarchicalkv_b200 as hkv
    from hierarchicalkv_b200.sharded import ShardedHashTable

    t = hkv.HashTable(hkv.EvictStrategy.kCustomized)
    t.init(hkv.HashTableOptions(init_capacity=128 * 64, max_capacity=128 * 64,
                                max_hbm_for_vectors=1 << 30, dim=8))
    st = ShardedHashTable(t)
    assert st.world == 1
    keys = unique_keys(3000, seed=2)
    k, v = to_dev(keys[:2000]), to_dev(values_for(keys[:2000], 8))
    s = to_dev(np.arange(1, 2001, dtype=np.uint64))
    st.insert_or_assign(2000, k, v, s)
    q = to_dev(keys)
    out = torch.zeros((3000, 8), device="cuda")
    f = torch.zeros(3000, dtype=torch.bool, device="cuda")
    st.find(3000, q, out, f)
    torch.cuda.synchronize()
    assert f[:2000].all() and not f[2000:].any() and st.size() == 2000
    assert torch.equal(out[:2000], v)
    t.close()


def _nccl_worker(rank, world, port, dim, cap):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    import torch.distributed as dist

    import hierarchicalkv_b200 as hkv
    from hierarchicalkv_b200.sharded import ShardedHashTable

    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world,
                            device_id=torch.device("cuda", rank))
    t = hkv.HashTable(hkv.EvictStrategy.kCustomized)
    t.init(hkv.HashTableOptions(init_capacity=cap, max_capacity=cap, max_hbm_for_vectors=1 << 30,
                                dim=dim))
    st = ShardedHashTable(t)
    keys = unique_keys(40000, seed=55)
    glob = OracleTable(cap * world, dim, 4)
    # every rank inserts its own slice; the global oracle sees them in rank order
    per = 8000
    for r in range(world):
        kk = keys[r * per:(r + 1) * per]
        glob.insert_or_assign(kk, values_for(kk, dim, seed=r),
                              np.arange(1, per + 1, dtype=np.uint64) + np.uint64(r * 100000))
    mine = keys[rank * per:(rank + 1) * per]
    st.insert_or_assign(per, to_dev(mine), to_dev(values_for(mine, dim, seed=rank)),
                        to_dev(np.arange(1, per + 1, dtype=np.uint64) + np.uint64(rank * 100000)))
    torch.cuda.synchronize()
    assert st.size() == glob.size()
    q = keys[: world * per + 3000]
    out = torch.full((q.size, dim), -3.0, device="cuda")
    f = torch.zeros(q.size, dtype=torch.bool, device="cuda")
    sc = torch.zeros(q.size, dtype=torch.int64, device="cuda")
    st.find(q.size, to_dev(q), out, f, sc)
    torch.cuda.synchronize()
    ev, ef, es = glob.find(q)
    assert np.array_equal(f.cpu().numpy(), ef)
    assert np.array_equal(out.cpu().numpy()[ef], ev[ef])
    assert np.all(out.cpu().numpy()[~ef] == -3.0)
    assert np.array_equal(to_np_u64(sc)[ef], es[ef])
    # find_or_insert with keys both ranks ask for, then accum_or_assign of deltas
    shared = keys[world * per: world * per + 2000]
    rows = to_dev(values_for(shared, dim, seed=70 + rank))
    st.find_or_insert(shared.size, to_dev(shared), rows,
                      to_dev(np.arange(1, shared.size + 1, dtype=np.uint64) + np.uint64(900000)))
    torch.cuda.synchronize()
    # the lowest rank's row is stored and returned to everybody
    assert np.array_equal(rows.cpu().numpy(), values_for(shared, dim, seed=70))
    deltas = values_for(shared, dim, seed=80 + rank)
    st.accum_or_assign(shared.size, to_dev(shared), to_dev(deltas),
                       to_dev(np.ones(shared.size, dtype=np.bool_)),
                       to_dev(np.arange(1, shared.size + 1, dtype=np.uint64) + np.uint64(950000)))
    torch.cuda.synchronize()
    want = values_for(shared, dim, seed=70).copy()
    acc = np.zeros_like(want)
    for r in range(world):
        acc = acc + values_for(shared, dim, seed=80 + r)      # rank order
    want = want + acc
    out = torch.zeros((shared.size, dim), device="cuda")
    f = torch.zeros(shared.size, dtype=torch.bool, device="cuda")
    st.find(shared.size, to_dev(shared), out, f)
    torch.cuda.synchronize()
    assert bool(f.all())
    assert np.array_equal(out.cpu().numpy().view(np.uint32), want.astype(np.float32).view(np.uint32))
    # fused find: peer stores instead of NCCL, same answers
    glob.insert_or_assign(shared, want.astype(np.float32),
                          np.arange(1, shared.size + 1, dtype=np.uint64) + np.uint64(900000))
    st.enable_fused_find(max_batch=q.size, dim=dim)
    for rep in range(3):                      # repeated use of the same inboxes and result buffers
        qq = np.roll(q, rep * 977)
        st.peer.out_values.fill_(-3.0)
        rows, flags = st.find_fused(qq.size, to_dev(qq))
        torch.cuda.synchronize()
        ev, ef, _ = glob.find(qq)
        assert np.array_equal(flags.cpu().numpy(), ef)
        got = rows.cpu().numpy()
        assert np.array_equal(got[ef].view(np.uint32), ev[ef].view(np.uint32))
        assert np.all(got[~ef] == -3.0)
        assert st.peer.status() == 0
    # the same lookups through two workspaces in rotation: batch k + 1 is issued
    # before batch k is waited for, and every batch still gets its own answers
    stp = ShardedHashTable(st.local)
    stp.enable_fused_find(max_batch=q.size, dim=dim, lanes=2)
    batches = [np.roll(q, 131 * i)[: q.size - 64 * i] for i in range(5)]
    dev_batches = [to_dev(b) for b in batches]
    for w_ in stp.lanes:
        w_.out_values.fill_(-3.0)
    torch.cuda.synchronize()

    def check(i, res):
        rows, flags, done = res
        done.wait()
        got, gf = rows.cpu().numpy(), flags.cpu().numpy()
        ev, ef, _ = glob.find(batches[i])
        assert np.array_equal(gf, ef)
        assert np.array_equal(got[ef].view(np.uint32), ev[ef].view(np.uint32))

    prev = None
    for i, b in enumerate(dev_batches):
        res = stp.find_fused_async(batches[i].size, b)
        if prev is not None:
            check(i - 1, prev)
        prev = res
    check(len(batches) - 1, prev)
    stp.join_lanes()
    torch.cuda.synchronize()
    assert all(w_.status() == 0 for w_ in stp.lanes)
    # fused update path on an LRU table: rows travel straight between the ranks' buffers
    t2 = hkv.HashTable(hkv.EvictStrategy.kLru)
    t2.init(hkv.HashTableOptions(init_capacity=cap, max_capacity=cap, max_hbm_for_vectors=1 << 30,
                                 dim=dim))
    st2 = ShardedHashTable(t2)
    st2.share_workspace(st)                  # fused paths of the same shape
    w = st2.peer
    both = keys[30000:33000]                 # every rank sends the same keys: all of them collide
    own = keys[33000 + rank * 1500: 33000 + (rank + 1) * 1500]
    mine2 = np.concatenate([both, own])
    w.out_values[:mine2.size].copy_(to_dev(values_for(mine2, dim, seed=200 + rank)))
    got = st2.upsert_fused("find_or_insert", mine2.size, to_dev(mine2))
    torch.cuda.synchronize()
    owner = (fmix64(both) % np.uint64(world)).astype(np.int64)
    first = (owner + 1) % world              # the rank whose batch an owner applies first
    def rows_of(seed_base, src):
        """row i as rank src[i] sent it"""
        out = np.zeros((both.size, dim), dtype=np.float32)
        for r in range(world):
            out[src == r] = values_for(both, dim, seed=seed_base + r)[src == r]
        return out

    want_both = rows_of(200, first)
    g = got.cpu().numpy()
    assert np.array_equal(g[:both.size].view(np.uint32), want_both.view(np.uint32))
    assert np.array_equal(g[both.size:].view(np.uint32),
                          values_for(own, dim, seed=200 + rank).view(np.uint32))
    # deltas from both ranks: (row + delta_first) + delta_second in the owner's order
    w.out_values[:mine2.size].copy_(to_dev(values_for(mine2, dim, seed=300 + rank)))
    w.out_founds[:mine2.size].fill_(True)
    st2.upsert_fused("accum_or_assign", mine2.size, to_dev(mine2))
    torch.cuda.synchronize()
    rows, flags = st2.find_fused(mine2.size, to_dev(mine2))
    torch.cuda.synchronize()
    assert bool(flags.all())
    want = want_both.copy()
    for turn in range(world):
        src = (first + turn) % world
        want = (want + rows_of(300, src)).astype(np.float32)
    g = rows.cpu().numpy()
    assert np.array_equal(g[:both.size].view(np.uint32), want.view(np.uint32))
    want_own = (values_for(own, dim, seed=200 + rank) + values_for(own, dim, seed=300 + rank))
    assert np.array_equal(g[both.size:].view(np.uint32), want_own.astype(np.float32).view(np.uint32))
    assert st2.size() == both.size + world * 1500
    assert w.status() == 0
    dist.barrier()
    t2.close()
    t.close()
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_nccl_ranks_match_one_global_oracle():
    import torch.multiprocessing as mp

    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    mp.spawn(_nccl_worker, args=(2, port, 8, 128 * 256), nprocs=2, join=True)


@pytest.mark.parametrize("world,n", [(2, 100000), (8, 4097), (16, 33), (3, 1), (5, 0)])
def test_route_keys_into_the_owners_inboxes(world, n):
    """The sending side of the fused routing on one GPU: `world` inboxes in
    this GPU's memory stand in for the peers'.  Segment `me` of owner r's inbox
    must hold exactly the keys r owns, each with its batch index, and r's count
    for `me` must say how many."""
    import ctypes

    from hierarchicalkv_b200.sharded import CudaOps, _PeerPtrs

    lib = CudaOps().lib
    me = world - 1
    cap_seg = max(32, (n + 31) // 32 * 32)
    keys = unique_keys(max(n, 1), seed=world * 1000 + n)[:n]
    d_keys = to_dev(keys) if n else torch.zeros(1, dtype=torch.int64, device="cuda")
    inbox_k = [torch.full((world * cap_seg,), -1, dtype=torch.int64, device="cuda") for _ in range(world)]
    inbox_o = [torch.full((world * cap_seg,), -1, dtype=torch.int32, device="cuda") for _ in range(world)]
    inbox_c = [torch.full((16,), -1, dtype=torch.int64, device="cuda") for _ in range(world)]
    pk, po, pc = _PeerPtrs(), _PeerPtrs(), _PeerPtrs()
    for r in range(world):
        pk.p[r], po.p[r], pc.p[r] = inbox_k[r].data_ptr(), inbox_o[r].data_ptr(), inbox_c[r].data_ptr()
    cursors = torch.zeros(32, dtype=torch.int64, device="cuda")
    for rep in range(2):                      # the cursors are reset by the call itself
        rc = lib.hkv_shard_route_keys_p2p(n, d_keys.data_ptr(), world, me, cap_seg, ctypes.byref(pk),
                                          ctypes.byref(po), ctypes.byref(pc), cursors.data_ptr(), None)
        assert rc == 0, (lib.hkv_shard_last_error() or b"").decode()
        torch.cuda.synchronize()
        owner = (fmix64(keys) % np.uint64(world)).astype(np.int64) if n else np.zeros(0, dtype=np.int64)
        for r in range(world):
            want_idx = np.nonzero(owner == r)[0]
            cnt = int(inbox_c[r][me].item())
            assert cnt == want_idx.size
            seg_k = to_np_u64(inbox_k[r][me * cap_seg: me * cap_seg + cnt])
            seg_o = inbox_o[r][me * cap_seg: me * cap_seg + cnt].cpu().numpy().astype(np.int64)
            assert np.array_equal(np.sort(seg_o), want_idx)          # every index once
            assert np.array_equal(seg_k, keys[seg_o])                # next to its own key
            # nothing outside this rank's segment was touched
            rest = torch.cat([inbox_o[r][: me * cap_seg], inbox_o[r][me * cap_seg + cnt:]])
            assert bool((rest == -1).all())


def _routed_call(lib, table, op, world, my_rank, cap_seg, inbox_keys, inbox_origin, counts, bufs,
                 flags=None):
    import ctypes

    from hierarchicalkv_b200.sharded import _PeerPtrs

    pv, pf = _PeerPtrs(), _PeerPtrs()
    for r in range(world):
        pv.p[r] = bufs[r].data_ptr()
        if flags is not None:
            pf.p[r] = flags[r].data_ptr()
    rc = lib.hkv_upsert_routed(table.handle, op, world, my_rank, cap_seg, inbox_keys.data_ptr(),
                               inbox_origin.data_ptr(), counts.data_ptr(), ctypes.byref(pv),
                               ctypes.byref(pf) if flags is not None else None, None)
    assert rc == 0, (lib.hkv_last_error() or b"").decode()
    torch.cuda.synchronize()


@pytest.mark.parametrize("world,me", [(3, 1), (8, 5), (16, 0)])
@pytest.mark.parametrize("dim", [8, 5])
def test_upsert_routed_applies_the_ranks_one_after_the_other(dim, world, me):
    """The owner side of the fused sharded update on one GPU: several source
    ranks' inbox segments, their batch buffers standing in for peer memory.
    Keys that several ranks send (with eight and sixteen ranks most keys come
    from most ranks) are applied in the order rank owner + 1, owner + 2, ...
    -- checked against the CPU oracle fed in that order."""
    import hierarchicalkv_b200 as hkv
    from hierarchicalkv_b200.sharded import CudaOps

    lib = CudaOps().lib
    cap_seg, nbuf = 2048, 3000
    cap = 128 * 64
    t = hkv.HashTable(hkv.EvictStrategy.kLru)
    t.init(hkv.HashTableOptions(init_capacity=cap, max_capacity=cap, max_hbm_for_vectors=1 << 30,
                                dim=dim))
    o = OracleTable(cap, dim, 0)
    keys = unique_keys(5200, seed=91)
    old = keys[:1500]
    t.insert_or_assign(old.size, to_dev(old), to_dev(values_for(old, dim, seed=1)))
    o.insert_or_assign(old, values_for(old, dim, seed=1))
    rng = np.random.default_rng(5)
    order = [(me + 1 + k) % world for k in range(world)]

    def make_step(pool, seed):
        """per source rank: keys (a random subset of the pool, so ranks overlap),
        their rows in that rank's buffer, and where the rows sit in the buffer"""
        per = {}
        for r in range(world):
            n = int(rng.integers(1200, 2000))
            kk = rng.choice(pool, size=n, replace=False)
            at = rng.permutation(nbuf)[:n].astype(np.uint32)      # origin: any row of the buffer
            buf = np.full((nbuf, dim), -7.0, dtype=np.float32)
            buf[at] = values_for(kk, dim, seed=seed + r)
            per[r] = (kk, at, buf)
        inbox_keys = np.zeros(world * cap_seg, dtype=np.uint64)
        inbox_origin = np.zeros(world * cap_seg, dtype=np.uint32)
        counts = np.zeros(16, dtype=np.uint64)
        for r in range(world):
            kk, at, _ = per[r]
            inbox_keys[r * cap_seg: r * cap_seg + kk.size] = kk
            inbox_keys[r * cap_seg + kk.size: (r + 1) * cap_seg] = 12345    # stale entries beyond the count
            inbox_origin[r * cap_seg: r * cap_seg + kk.size] = at
            counts[r] = kk.size
        return per, to_dev(inbox_keys), torch.from_numpy(inbox_origin.view(np.int32)).cuda(), to_dev(counts)

    def table_rows(which):
        out = torch.zeros((which.size, dim), device="cuda")
        f = torch.zeros(which.size, dtype=torch.bool, device="cuda")
        t.find(which.size, to_dev(which), out, f)
        torch.cuda.synchronize()
        return out.cpu().numpy(), f.cpu().numpy()

    def check_table(which):
        got, gf = table_rows(which)
        want, wf, _ = o.find(which)
        np.testing.assert_array_equal(gf, wf)
        np.testing.assert_array_equal(got[gf].view(np.uint32), want[wf].view(np.uint32))

    # find_or_insert: hits return the stored row into the rank's buffer, misses store the rank's row
    pool = keys[1000:3000]                      # 500 old keys, 1500 new ones
    per, ik, io, cnt = make_step(pool, seed=20)
    bufs = [torch.from_numpy(per[r][2].copy()).cuda() for r in range(world)]
    _routed_call(lib, t, 1, world, me, cap_seg, ik, io, cnt, bufs)
    for r in order:
        kk, at, buf = per[r]
        rows = np.ascontiguousarray(buf[at])
        got_rows = o.find_or_insert(kk, rows)
        back = bufs[r].cpu().numpy()
        np.testing.assert_array_equal(back[at].view(np.uint32), got_rows.view(np.uint32))
        untouched = np.ones(nbuf, dtype=bool)
        untouched[at] = False
        assert np.all(back[untouched] == -7.0)
    check_table(keys[:3500])
    assert t.size() == o.size()

    # accum_or_assign: deltas add up rank after rank; assignments only insert missing keys
    pool = keys[2000:4200]
    per, ik, io, cnt = make_step(pool, seed=40)
    bufs = [torch.from_numpy(per[r][2].copy()).cuda() for r in range(world)]
    flag_np = [rng.integers(0, 4, size=nbuf) != 0 for _ in range(world)]     # 75 % accumulate
    flags = [torch.from_numpy(f).cuda() for f in flag_np]
    _routed_call(lib, t, 2, world, me, cap_seg, ik, io, cnt, bufs, flags)
    for r in order:
        kk, at, buf = per[r]
        o.accum_or_assign(kk, np.ascontiguousarray(buf[at]), np.ascontiguousarray(flag_np[r][at]))
    check_table(keys[:4500])
    assert t.size() == o.size()

    # insert_or_assign: the last rank in the order wins
    pool = keys[3200:5200]
    per, ik, io, cnt = make_step(pool, seed=60)
    bufs = [torch.from_numpy(per[r][2].copy()).cuda() for r in range(world)]
    _routed_call(lib, t, 0, world, me, cap_seg, ik, io, cnt, bufs)
    for r in order:
        kk, at, buf = per[r]
        o.insert_or_assign(kk, np.ascontiguousarray(buf[at]))
    check_table(keys)
    assert t.size() == o.size()
    assert t.device_status() == 0
    # strategies that need scores cannot be routed
    lfu = hkv.HashTable(hkv.EvictStrategy.kLfu)
    lfu.init(hkv.HashTableOptions(init_capacity=cap, max_capacity=cap, max_hbm_for_vectors=1 << 30,
                                  dim=dim))
    from hierarchicalkv_b200.sharded import _PeerPtrs
    import ctypes
    pv = _PeerPtrs()
    assert lib.hkv_upsert_routed(lfu.handle, 0, world, me, cap_seg, ik.data_ptr(), io.data_ptr(),
                                 cnt.data_ptr(), ctypes.byref(pv), None, None) != 0
    lfu.close()
    t.close()


@pytest.mark.parametrize("world,me", [(2, 0), (8, 3)])
def test_upsert_routed_steps_back_to_back(world, me):
    """The sharded embedding step as the owner sees it, several steps without a
    host synchronisation in between: find_or_insert of every rank's keys, then
    accum_or_assign of deltas for the same inbox (the route is reused), with
    keys most ranks share and buffers that are rewritten between the calls.
    The table must hold what the CPU oracle holds when the ranks' batches are
    applied in the order owner + 1, owner + 2, ..."""
    import ctypes

    import hierarchicalkv_b200 as hkv
    from hierarchicalkv_b200.sharded import CudaOps, _PeerPtrs

    lib = CudaOps().lib
    dim, cap_seg, nbuf, cap = 8, 1024, 1024, 128 * 64
    t = hkv.HashTable(hkv.EvictStrategy.kLru)
    t.init(hkv.HashTableOptions(init_capacity=cap, max_capacity=cap, max_hbm_for_vectors=1 << 30,
                                dim=dim))
    o = OracleTable(cap, dim, 0)
    keys = unique_keys(3000, seed=17)
    rng = np.random.default_rng(23)
    order = [(me + 1 + k) % world for k in range(world)]
    bufs = [torch.zeros((nbuf, dim), device="cuda") for _ in range(world)]
    flags = [torch.ones(nbuf, dtype=torch.bool, device="cuda") for _ in range(world)]
    pv, pf = _PeerPtrs(), _PeerPtrs()
    for r in range(world):
        pv.p[r], pf.p[r] = bufs[r].data_ptr(), flags[r].data_ptr()
    inbox_k = torch.zeros(world * cap_seg, dtype=torch.int64, device="cuda")
    inbox_o = torch.zeros(world * cap_seg, dtype=torch.int32, device="cuda")
    counts = torch.zeros(16, dtype=torch.int64, device="cuda")

    def call(op):
        rc = lib.hkv_upsert_routed(t.handle, op, world, me, cap_seg, inbox_k.data_ptr(),
                                   inbox_o.data_ptr(), counts.data_ptr(), ctypes.byref(pv),
                                   ctypes.byref(pf), None)
        assert rc == 0, (lib.hkv_last_error() or b"").decode()

    steps = []
    for step in range(6):
        hot = keys[:300]                                   # every rank sends these in every step
        per = {}
        for r in range(world):
            own = rng.choice(keys[300:], size=int(rng.integers(200, 600)), replace=False)
            kk = np.concatenate([hot, own])
            at = rng.permutation(nbuf)[:kk.size].astype(np.int32)
            init = values_for(kk, dim, seed=100 * step + r)
            delta = values_for(kk, dim, seed=5000 + 100 * step + r) * np.float32(1e-3)
            per[r] = (kk, at, init, delta)
            inbox_k[r * cap_seg: r * cap_seg + kk.size] = to_dev(kk)
            inbox_o[r * cap_seg: r * cap_seg + kk.size] = torch.from_numpy(at).cuda()
            counts[r] = kk.size
            bufs[r][torch.from_numpy(at.astype(np.int64)).cuda()] = torch.from_numpy(init).cuda()
        call(1)                                            # find_or_insert: rows come back
        for r in range(world):                             # the "gradients" take their place
            kk, at, init, delta = per[r]
            bufs[r][torch.from_numpy(at.astype(np.int64)).cuda()] = torch.from_numpy(delta).cuda()
        call(2)                                            # accum_or_assign on the same inbox
        steps.append(per)
    torch.cuda.synchronize()
    for per in steps:
        for r in order:
            kk, at, init, delta = per[r]
            o.find_or_insert(kk, init)
        for r in order:
            kk, at, init, delta = per[r]
            o.accum_or_assign(kk, delta, np.ones(kk.size, dtype=bool))
    out = torch.zeros((keys.size, dim), device="cuda")
    f = torch.zeros(keys.size, dtype=torch.bool, device="cuda")
    t.find(keys.size, to_dev(keys), out, f)
    torch.cuda.synchronize()
    want, wf, _ = o.find(keys)
    np.testing.assert_array_equal(f.cpu().numpy(), wf)
    np.testing.assert_array_equal(out.cpu().numpy()[wf].view(np.uint32), want[wf].view(np.uint32))
    assert t.device_status() == 0
    t.close()


def test_peer_barrier_times_out_instead_of_hanging():
    """The barrier of the fused routing waits for flags the peers raise.  With a
    peer that never arrives the wait runs out after its poll limit, the kernel
    returns, and the status word says so; the context stays usable."""
    import ctypes

    from hierarchicalkv_b200.sharded import CudaOps, _PeerPtrs

    lib = CudaOps().lib
    flags = torch.zeros((2, 16), dtype=torch.int32, device="cuda")   # "rank 0" and "rank 1" flags
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    peers = _PeerPtrs()
    peers.p[0] = flags[0].data_ptr()
    peers.p[1] = flags[1].data_ptr()
    sp = torch.cuda.current_stream().cuda_stream or None
    # rank 0 arrives at epoch 1; nobody plays rank 1
    rc = lib.hkv_shard_barrier(2, 0, ctypes.byref(peers), 1, status.data_ptr(), 2000, sp)
    assert rc == 0
    torch.cuda.synchronize()
    assert int(status.item()) == 1
    assert int(flags[1, 0].item()) == 1            # the arrival was announced to the peer
    # once the peer's flag is there the same barrier passes
    status.zero_()
    flags[0, 1] = 1
    rc = lib.hkv_shard_barrier(2, 0, ctypes.byref(peers), 1, status.data_ptr(), 2000, sp)
    torch.cuda.synchronize()
    assert rc == 0 and int(status.item()) == 0
