"""Key-hash sharded table across the GPUs of one node.

The reference is a single-GPU library; its users shard by hand with one table
per GPU.  This module is that pattern made explicit: every rank owns one
independent sub-table, ``owner(key) = Murmur3(key) % world_size`` (the
table's own hash, include/merlin/utils.cuh:137-145 of the reference), and a
batch is routed with an all-to-all over NVLink -- keys out, rows and found
flags back -- around the local operation.

One process per GPU.  Two routings: the fused one (find_fused, upsert_fused:
keys, rows and flags travel over peer memory inside the library's own kernels;
the host side is the library's C++ sharded table, csrc/hkv_sharded.cu, which
this module only binds) and the plain one, where ``torch.distributed`` (NCCL)
carries the exchange and the grouping by owner and the row permutations are
CUDA kernels of libhkv_b200.so (csrc/hkv_shard.cu).  With a world of one rank
the exchange is skipped and every call is exactly the local table's.
"""
from __future__ import annotations

import ctypes
from typing import List, Optional

import torch

from .table import HashTable, load_library


def _stream_ptr() -> Optional[int]:
    return torch.cuda.current_stream().cuda_stream or None


class CudaOps:
    """Device-side helpers of the router (hkv_shard_* of the C ABI)."""

    def __init__(self):
        self.lib = load_library()

    def _chk(self, rc: int) -> None:
        if rc:
            raise RuntimeError((self.lib.hkv_shard_last_error() or b"").decode())

    def partition(self, keys: torch.Tensor, world: int):
        """-> (counts on the host, keys grouped by owner, batch index of each grouped key)"""
        n = keys.numel()
        dev = keys.device
        meta = torch.empty(3 * world, dtype=torch.int64, device=dev)
        grouped = torch.empty(n, dtype=torch.int64, device=dev)
        origin = torch.empty(n, dtype=torch.int32, device=dev)
        self._chk(self.lib.hkv_shard_partition(
            n, keys.data_ptr(), world, meta.data_ptr(), meta[world:].data_ptr(),
            meta[2 * world:].data_ptr(), grouped.data_ptr(), origin.data_ptr(), _stream_ptr()))
        counts = meta[:world].cpu().tolist()  # the split sizes are needed on the host
        return counts, grouped, origin

    def gather_rows(self, src: torch.Tensor, index: torch.Tensor) -> torch.Tensor:
        """dst[i] = src[index[i]]"""
        n = index.numel()
        dst = torch.empty((n,) + tuple(src.shape[1:]), dtype=src.dtype, device=src.device)
        row_bytes = src.element_size() * (src[0].numel() if src.dim() > 1 else 1)
        self._chk(self.lib.hkv_shard_gather_rows(n, row_bytes, src.data_ptr(), index.data_ptr(),
                                                 dst.data_ptr(), _stream_ptr()))
        return dst

    def scatter_rows(self, src: torch.Tensor, index: torch.Tensor, dst: torch.Tensor) -> None:
        """dst[index[i]] = src[i]; rows whose index is -1 are skipped"""
        n = index.numel()
        row_bytes = src.element_size() * (src[0].numel() if src.dim() > 1 else 1)
        self._chk(self.lib.hkv_shard_scatter_rows(n, row_bytes, src.data_ptr(), index.data_ptr(),
                                                  dst.data_ptr(), _stream_ptr()))


class _PeerPtrs(ctypes.Structure):
    """hkv_peer_ptrs"""

    _fields_ = [("p", ctypes.c_void_p * 16)]


class _IpcHandle(ctypes.Structure):
    """hkv_ipc_handle"""

    _fields_ = [("bytes", ctypes.c_ubyte * 64)]


class _DeviceBytes:
    """A range of device memory torch can wrap without copying."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1",
                                         "data": (ptr, False), "version": 2}


class PeerWorkspace:
    """One lane of the sharded table's C++ host (hkv_sharded, csrc/hkv_sharded.cu):
    this rank's inbox of routed keys and its batch / result buffers, which the
    other ranks of the node store into over NVLink.  The object only holds
    torch views of this rank's buffers; allocation, the mapping of the peers'
    workspaces and the barrier epochs live in the library."""

    def __init__(self, lib, host, lane: int, max_batch: int, dim: int, dtype: torch.dtype):
        self.lib, self.host, self.lane = lib, host, lane
        self.max_batch = max_batch
        self.dim = dim
        self.dtype = dtype
        rows, flags = ctypes.c_void_p(), ctypes.c_void_p()
        if lib.hkv_sharded_buffers(host, lane, ctypes.byref(rows), ctypes.byref(flags)):
            raise RuntimeError((lib.hkv_sharded_last_error() or b"").decode())
        row_bytes = dim * torch.empty((), dtype=dtype).element_size()
        ov = torch.as_tensor(_DeviceBytes(rows.value, max_batch * row_bytes), device="cuda")
        self.out_values = ov.view(dtype).view(max_batch, dim)
        self.out_founds = torch.as_tensor(_DeviceBytes(flags.value, max_batch),
                                          device="cuda").view(torch.bool)

    def status(self) -> int:
        """Non-zero after a barrier timed out (a peer never arrived)."""
        out = ctypes.c_uint32(0)
        if self.lib.hkv_sharded_status(self.host, self.lane, _stream_ptr(), ctypes.byref(out)):
            raise RuntimeError((self.lib.hkv_sharded_last_error() or b"").decode())
        return out.value


class LaneResult:
    """Completion of one find_fused_async call."""

    def __init__(self, table, lane: int, keys):
        self._table, self.lane, self._keys = table, lane, keys   # the keys stay alive until waited for

    def wait(self) -> None:
        """Makes the current stream wait for the lane's results."""
        self._table._chk_host(self._table.ops.lib.hkv_sharded_wait(self._table._host, self.lane,
                                                                   _stream_ptr()))
        self._keys = None


class _Route:
    """How one batch travels: who gets how many keys, and the way back."""

    __slots__ = ("send_counts", "recv_counts", "origin", "recv_keys", "n")

    def __init__(self, send_counts, recv_counts, origin, recv_keys, n):
        self.send_counts: List[int] = send_counts
        self.recv_counts: List[int] = recv_counts
        self.origin = origin          # batch index of every grouped key (None: identity)
        self.recv_keys = recv_keys    # keys this rank has to serve, grouped by source rank
        self.n = n


class ShardedHashTable:
    """The reference's method names over a table sharded by key hash.

    ``local`` is this rank's sub-table (anything with the HashTable methods);
    ``group`` a torch.distributed process group (None: the default group, or a
    single rank when torch.distributed is not initialised).
    """

    def __init__(self, local: HashTable, group=None, ops=None):
        self.local = local
        self.group = group
        self.dist = None
        self.world = 1
        self.rank = 0
        if torch.distributed.is_available() and torch.distributed.is_initialized():
            self.dist = torch.distributed
            self.world = self.dist.get_world_size(group)
            self.rank = self.dist.get_rank(group)
        self.ops = ops if ops is not None else CudaOps()

    # -- routing ------------------------------------------------------------
    def _all_to_all(self, send: torch.Tensor, send_counts, recv_counts) -> torch.Tensor:
        out = torch.empty((sum(recv_counts),) + tuple(send.shape[1:]), dtype=send.dtype,
                          device=send.device)
        self.dist.all_to_all_single(out, send, output_split_sizes=list(recv_counts),
                                    input_split_sizes=list(send_counts), group=self.group)
        return out

    def _route(self, n: int, keys: torch.Tensor) -> _Route:
        if self.world == 1:
            return _Route([n], [n], None, keys, n)
        send_counts, grouped, origin = self.ops.partition(keys[:n], self.world)
        sc = torch.tensor(send_counts, dtype=torch.int64, device=keys.device)
        rc = torch.empty_like(sc)
        self.dist.all_to_all_single(rc, sc, group=self.group)
        recv_counts = rc.cpu().tolist()
        recv_keys = self._all_to_all(grouped, send_counts, recv_counts)
        return _Route(send_counts, recv_counts, origin, recv_keys, n)

    def _rows_out(self, route: _Route, rows: torch.Tensor) -> torch.Tensor:
        """Caller's rows -> the rows this rank has to apply, in recv_keys order."""
        if self.world == 1:
            return rows
        grouped = self.ops.gather_rows(rows, route.origin)
        return self._all_to_all(grouped, route.send_counts, route.recv_counts)

    def _rows_back(self, route: _Route, served: torch.Tensor, out: torch.Tensor) -> None:
        """Rows produced for recv_keys -> the caller's buffer, in the caller's order."""
        if self.world == 1:
            if served.data_ptr() != out.data_ptr():
                out[: route.n].copy_(served)
            return
        back = self._all_to_all(served, route.recv_counts, route.send_counts)
        self.ops.scatter_rows(back, route.origin, out)

    # -- duplicates that meet at the owner ---------------------------------------
    @staticmethod
    def _dedup(recv_keys: torch.Tensor):
        """Keys arriving from different ranks may coincide.  -> (unique keys,
        index of each received key in them, position of the first occurrence)."""
        uniq, inverse = torch.unique(recv_keys, return_inverse=True)
        first = torch.full((uniq.numel(),), recv_keys.numel(), dtype=torch.int64,
                           device=recv_keys.device)
        first.scatter_reduce_(0, inverse, torch.arange(recv_keys.numel(), device=recv_keys.device),
                              reduce="amin")
        return uniq, inverse, first

    # -- operations -----------------------------------------------------------
    def find(self, n, keys, values, founds, scores=None, stream=None) -> None:
        """HashTable::find over all shards; misses leave `values` untouched."""
        if n == 0:
            return
        route = self._route(n, keys)
        m = route.recv_keys.numel()
        if self.world == 1:
            self.local.find(n, keys, values, founds, scores, stream)
            return
        served = torch.empty((m,) + tuple(values.shape[1:]), dtype=values.dtype,
                             device=values.device)
        hit = torch.zeros(m, dtype=torch.bool, device=values.device)
        sc = torch.zeros(m, dtype=torch.int64, device=values.device) if scores is not None else None
        if m:
            self.local.find(m, route.recv_keys, served, hit, sc, stream)
        back = self._all_to_all(served, route.recv_counts, route.send_counts)
        hit_back = self._all_to_all(hit.view(torch.uint8), route.recv_counts, route.send_counts)
        self.ops.scatter_rows(hit_back, route.origin, founds[:n].view(torch.uint8))
        # only the rows of the hits may be written into the caller's buffer:
        # a miss gets the "skip" index
        where = torch.where(hit_back.view(torch.bool), route.origin,
                            torch.full_like(route.origin, -1))
        self.ops.scatter_rows(back, where, values)
        if scores is not None:
            sc_back = self._all_to_all(sc, route.recv_counts, route.send_counts)
            self.ops.scatter_rows(sc_back, where, scores)

    def enable_fused_find(self, max_batch: int, dim: int, dtype: torch.dtype = torch.float32,
                          lanes: int = 1, memory: str = "auto"):
        """Creates the C++ host of the fused paths for this rank's sub-table and
        connects the ranks' workspaces.  ``memory``: "symmetric" takes the
        workspaces from torch symmetric memory (CUDA virtual-memory allocations
        that every rank maps) and hands them to hkv_sharded_create_external;
        "ipc" lets the library allocate them and exchanges their CUDA IPC
        handles; "auto" tries the former and falls back to the latter.  Peer
        stores into IPC-mapped cudaMalloc memory measured much slower at eight
        GPUs (find 13.5 against 20.1 B-KV/s), level at two and four; the
        updates (upsert_fused), on the other hand, have passed their
        bit-for-bit replay check at eight ranks only on "ipc" workspaces (on
        symmetric memory at two and four), so a table that is updated across
        more than four ranks should keep a host with memory="ipc" for that.  With
        ``lanes`` > 1 there are that many independent workspaces (own inbox,
        flags, epochs and streams) for find_fused_async, which rotates through
        them so the routing of one batch overlaps the lookup of the previous
        one.  A collective call: every rank passes the same arguments."""
        lib = self.ops.lib
        lanes = max(1, lanes)
        host = ctypes.c_void_p()
        self._symmetric = None
        if self.world > 1 and memory in ("auto", "symmetric"):
            try:
                self._symmetric = self._symmetric_workspaces(max_batch, lanes)
            except Exception:
                if memory == "symmetric":
                    raise
                self._symmetric = None
            if memory == "auto":
                # all ranks take the same path
                ok = torch.tensor([1 if self._symmetric is not None else 0], device="cuda")
                self.dist.all_reduce(ok, op=self.dist.ReduceOp.MIN, group=self.group)
                if int(ok.item()) == 0:
                    self._symmetric = None
        if self._symmetric is not None:
            bufs, peer_ptrs = self._symmetric
            mine = (ctypes.c_void_p * lanes)(*[peer_ptrs[lane][self.rank] for lane in range(lanes)])
            self._chk_host(lib.hkv_sharded_create_external(self.local.handle, self.world, self.rank,
                                                           max_batch, lanes, mine, ctypes.byref(host)))
            self._host = host
            for lane in range(lanes):
                bases = (ctypes.c_void_p * self.world)(*peer_ptrs[lane])
                self._chk_host(lib.hkv_sharded_connect_pointers(host, lane, bases))
            torch.cuda.synchronize()
            self.dist.barrier(self.group)     # every rank's workspace is cleared and connected
        else:
            self._chk_host(lib.hkv_sharded_create(self.local.handle, self.world, self.rank, max_batch,
                                                  lanes, ctypes.byref(host)))
            self._host = host
            if self.world > 1:
                mine = []
                for lane in range(lanes):
                    h = _IpcHandle()
                    self._chk_host(lib.hkv_sharded_ipc_handle(host, lane, ctypes.byref(h)))
                    mine.append(bytes(h.bytes))
                everyone = [None] * self.world
                self.dist.all_gather_object(everyone, mine, group=self.group)
                for lane in range(lanes):
                    handles = (_IpcHandle * self.world)()
                    for r in range(self.world):
                        ctypes.memmove(handles[r].bytes, everyone[r][lane], 64)
                    self._chk_host(lib.hkv_sharded_connect_ipc(host, lane, handles))
                torch.cuda.synchronize()
                self.dist.barrier(self.group)     # every rank's workspace is mapped, its flags still zero
        n_lanes = lib.hkv_sharded_lanes(host)
        cap = lib.hkv_sharded_max_batch(host)
        self.lanes = [PeerWorkspace(lib, host, lane, cap, dim, dtype) for lane in range(n_lanes)]
        self._pending = [None for _ in self.lanes]
        self.peer = self.lanes[0]
        return self.peer

    def _symmetric_workspaces(self, max_batch: int, lanes: int):
        """One symmetric-memory buffer per lane, sized by the library, and every
        rank's address of it: ([buffers], [[address per rank] per lane])."""
        import torch.distributed._symmetric_memory as symm

        size = ctypes.c_uint64(0)
        self._chk_host(self.ops.lib.hkv_sharded_workspace_bytes(self.local.handle, self.world,
                                                                max_batch, ctypes.byref(size)))
        group = self.group if self.group is not None else self.dist.group.WORLD
        bufs, ptrs = [], []
        for _ in range(lanes):
            buf = symm.empty(size.value, dtype=torch.uint8,
                             device=torch.device("cuda", torch.cuda.current_device()))
            handle = symm.rendezvous(buf, group)
            bufs.append((buf, handle))
            ptrs.append([int(p) for p in handle.buffer_ptrs])
        return bufs, ptrs

    def share_workspace(self, other: "ShardedHashTable") -> None:
        """Gives this table fused paths shaped like `other`'s (a collective call:
        every host belongs to one sub-table and has workspaces of its own)."""
        self.enable_fused_find(other.peer.max_batch, other.peer.dim, other.peer.dtype,
                               lanes=len(other.lanes))

    def close_fused(self) -> None:
        """Destroys the C++ host (call it on every rank, after a barrier of their own)."""
        host = getattr(self, "_host", None)
        if host:
            self.ops.lib.hkv_sharded_destroy(host)
            self._host = None
        self._symmetric = None

    # -- fused paths: routing, lookup / update and transfer without NCCL ----------
    def _chk_host(self, rc: int) -> None:
        if rc:
            raise RuntimeError((self.ops.lib.hkv_sharded_last_error() or b"").decode())

    def find_fused(self, n, keys, max_polls: int = 50_000_000, lane: int = 0):
        """HashTable::find over all shards with lookup and transfer fused
        (hkv_sharded_find): keys are grouped by owner and stored straight into
        the owners' inboxes, every owner runs ONE lookup kernel over what
        arrived and stores hit rows and found flags straight into the
        requesters' result buffers over NVLink.  No NCCL call and no host
        synchronisation; two bounded peer barriers.  Returns views (rows, found
        flags) of this rank's result buffers, valid until the next call on the
        same lane; rows of misses keep their previous content."""
        w = self.lanes[lane]
        self._chk_host(self.ops.lib.hkv_sharded_find(self._host, lane, n, keys.data_ptr(), max_polls,
                                                     _stream_ptr()))
        return w.out_values[:n], w.out_founds[:n]

    def find_fused_async(self, n, keys, max_polls: int = 50_000_000):
        """find_fused on the next lane's own streams (hkv_sharded_find_async):
        returns (rows, found flags, result) at once; ``result.wait()`` makes the
        current stream wait for them.  Every rank must make the same sequence
        of calls.  Consecutive calls use different lanes, so the grouping, the
        key stores and the barriers of batch k + 1 run while the owners still
        serve batch k.  To keep that overlap, issue batch k + 1 BEFORE waiting
        for batch k: each call first makes its lane wait for everything
        already queued on the caller's stream (the producer of ``keys``, and
        the consumer of the lane's previous results)."""
        used = ctypes.c_uint32(0)
        self._chk_host(self.ops.lib.hkv_sharded_find_async(self._host, n, keys.data_ptr(), max_polls,
                                                           _stream_ptr(), ctypes.byref(used)))
        lane = used.value
        w = self.lanes[lane]
        result = LaneResult(self, lane, keys)
        self._pending[lane] = result
        return w.out_values[:n], w.out_founds[:n], result

    def join_lanes(self) -> None:
        """Makes the caller's stream wait for every lane's last find_fused_async."""
        for lane, r in enumerate(self._pending):
            if r is not None:
                r.wait()
                self._pending[lane] = None

    _ROUTED_OPS = {"insert_or_assign": 0, "find_or_insert": 1, "accum_or_assign": 2}

    def upsert_fused(self, op: str, n, keys, max_polls: int = 50_000_000,
                     reuse_route: bool = False):
        """insert_or_assign / find_or_insert / accum_or_assign over all shards
        with the update and the transfer fused (hkv_sharded_upsert).  The batch
        rows are the first n rows of this rank's peer-visible buffer
        ``peer.out_values`` (for accum_or_assign the flags are
        ``peer.out_founds[:n]``): the caller fills them before the call, the
        owners' kernels read new rows and deltas from them and --
        find_or_insert -- write the stored rows of the hits back into them, all
        over NVLink.  No NCCL call, no host synchronisation, no staging copy;
        two bounded peer barriers.

        A key that several ranks send in one step behaves as if those ranks had
        called the table one after the other, starting with rank owner + 1
        (wrapping).  Needs a score-free strategy (kLru / kEpochLru).

        ``reuse_route``: the keys are those of the previous upsert_fused call of
        every rank (the update that follows a find_or_insert of the same
        batch): the owners' inboxes still hold them and the routing is skipped;
        the barrier stays, it tells the owners that the ranks' buffers carry
        the new rows."""
        self._chk_host(self.ops.lib.hkv_sharded_upsert(self._host, self._ROUTED_OPS[op], n,
                                                       keys.data_ptr(), int(reuse_route), max_polls,
                                                       _stream_ptr()))
        return self.peer.out_values[:n]

    def insert_or_assign(self, n, keys, values, scores=None, stream=None) -> None:
        if n == 0:
            return
        if self.world == 1:
            self.local.insert_or_assign(n, keys, values, scores, stream)
            return
        route = self._route(n, keys)
        rows = self._rows_out(route, values[:n])
        sc = self._rows_out(route, scores[:n]) if scores is not None else None
        if route.recv_keys.numel():
            uniq, inverse, first = self._dedup(route.recv_keys)
            self.local.insert_or_assign(uniq.numel(), uniq, rows.index_select(0, first).contiguous(),
                                        sc.index_select(0, first).contiguous() if sc is not None else None,
                                        stream)

    def find_or_insert(self, n, keys, values, scores=None, stream=None) -> None:
        """Hits return the stored row, misses insert the caller's row; when the
        same new key arrives from several ranks the lowest rank's row is stored
        and every requester gets that row back."""
        if n == 0:
            return
        if self.world == 1:
            self.local.find_or_insert(n, keys, values, scores, stream)
            return
        route = self._route(n, keys)
        rows = self._rows_out(route, values[:n])
        sc = self._rows_out(route, scores[:n]) if scores is not None else None
        if route.recv_keys.numel():
            uniq, inverse, first = self._dedup(route.recv_keys)
            urows = rows.index_select(0, first).contiguous()
            self.local.find_or_insert(uniq.numel(), uniq, urows,
                                      sc.index_select(0, first).contiguous() if sc is not None else None,
                                      stream)
            served = urows.index_select(0, inverse).contiguous()
        else:
            served = rows
        self._rows_back(route, served, values)

    def accum_or_assign(self, n, keys, value_or_deltas, accum_or_assigns, scores=None,
                        stream=None) -> None:
        """Deltas for one key coming from several ranks are summed in rank order
        before the local accum_or_assign, so the fp32 result is reproducible."""
        if n == 0:
            return
        if self.world == 1:
            self.local.accum_or_assign(n, keys, value_or_deltas, accum_or_assigns, scores, stream)
            return
        route = self._route(n, keys)
        rows = self._rows_out(route, value_or_deltas[:n])
        flags = self._rows_out(route, accum_or_assigns[:n].view(torch.uint8)).view(torch.bool)
        sc = self._rows_out(route, scores[:n]) if scores is not None else None
        if not route.recv_keys.numel():
            return
        uniq, inverse, first = self._dedup(route.recv_keys)
        acc = torch.zeros((uniq.numel(),) + tuple(rows.shape[1:]), dtype=rows.dtype,
                          device=rows.device)
        at = 0
        for c in route.recv_counts:           # one source rank at a time: no collisions inside a call
            if c:
                seg = slice(at, at + c)
                is_acc = flags[seg]
                idx = inverse[seg]
                acc.index_add_(0, idx[is_acc], rows[seg][is_acc])
                # an assignment takes the first occurrence's row
                take = (~is_acc) & (first.index_select(0, idx) == torch.arange(at, at + c, device=rows.device))
                acc.index_copy_(0, idx[take], rows[seg][take])
            at += c
        uflags = flags.index_select(0, first).contiguous()
        usc = sc.index_select(0, first).contiguous() if sc is not None else None
        fn = getattr(self.local, "accum_or_assign_unique", self.local.accum_or_assign)
        fn(uniq.numel(), uniq, acc, uflags, usc, stream)

    def size(self, stream=None) -> int:
        s = self.local.size(stream)
        if self.world == 1:
            return s
        t = torch.tensor([s], dtype=torch.int64,
                         device="cuda" if self.dist.get_backend(self.group) == "nccl" else "cpu")
        self.dist.all_reduce(t, group=self.group)
        return int(t.item())

    def owner_of(self, keys: torch.Tensor) -> torch.Tensor:
        """Owner rank of each key (host-side check of the routing rule)."""
        k = keys.cpu().numpy().view("uint64").copy()
        import numpy as np

        k ^= k >> np.uint64(33)
        k *= np.uint64(0xFF51AFD7ED558CCD)
        k ^= k >> np.uint64(33)
        k *= np.uint64(0xC4CEB9FE1A85EC53)
        k ^= k >> np.uint64(33)
        return torch.from_numpy((k % np.uint64(self.world)).astype("int64"))
