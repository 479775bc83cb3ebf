"""Sharding of the page pool across the GPUs of one box by request ownership, and page migration between shards.

One process per GPU. A request's pages, block-table row and allocator state live on its owner; appends and gathers are
local and need no exchange. The only inter-GPU operation is migration: the destination allocates pages in its own pool,
pulls the payload of every layer page by page from the source's pool, and only then does the source release its pages.
The payload moves with `pkv_copy_pages` on the destination GPU, reading the source pool through a CUDA IPC mapping with
ordinary 16-byte loads over NVLink (no bulk/TMA copy ever touches peer memory). torch.distributed carries only the small
host-side messages (who moves where, which page ids); it is plumbing.

The reference has no sharded pool and no migration (parity unpinned). The rule fixed here: pages keep their logical
order; the destination takes fresh ids from its allocator exactly as alloc_pages would (src/engine/engine.cpp:437-444);
the source unreferences tail first (src/engine/engine.cpp:208-217); cached names are not carried over.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import numpy as np

from . import capi

i32p = C.POINTER(C.c_int32)


def owner(request: int, world: int) -> int:
    """Round-robin ownership of requests."""
    return request % world


@dataclass
class Move:
    request: int
    src: int
    dst: int
    length: int          # rows held by the sequence
    src_pages: list      # physical ids in the source pool, logical order


class PeerPools:
    """Every rank's pool base pointers, mapped into this process through CUDA IPC.

    local_ptrs: device pointers of this rank's pools (each the base of its own cudaMalloc allocation, e.g. from
    pkv_device_alloc). After construction `base(rank, i)` is a pointer valid on THIS device for pool i of `rank`.
    """

    def __init__(self, dist, rank: int, world: int, local_ptrs):
        self.lib, self.rank, self.world = capi.lib(), rank, world
        handles = []
        for p in local_ptrs:
            buf = (C.c_uint8 * 64)()
            capi.check(self.lib.pkv_ipc_export(C.c_void_p(p), buf))
            handles.append(bytes(buf))
        gathered = [None] * world
        dist.all_gather_object(gathered, handles)
        self._bases, self._opened = [], []
        for r in range(world):
            if r == rank:
                self._bases.append(list(local_ptrs))
                continue
            ptrs = []
            for h in gathered[r]:
                out = C.c_void_p()
                capi.check(self.lib.pkv_ipc_open((C.c_uint8 * 64).from_buffer_copy(h), C.byref(out)))
                ptrs.append(out.value)
                self._opened.append(out.value)
            self._bases.append(ptrs)

    def base(self, rank: int, i: int) -> int:
        return self._bases[rank][i]

    def close(self):
        for p in self._opened:
            self.lib.pkv_ipc_close(C.c_void_p(p))
        self._opened = []


class DevicePull:
    """Transport that pulls pages on the destination GPU from an IPC-mapped source pool (all pools in one launch)."""

    def __init__(self, torch, peers: PeerPools, page_bytes, num_pages: int):
        self.torch, self.peers, self.page_bytes, self.num_pages = torch, peers, list(page_bytes), num_pages
        self.lib = capi.lib()
        self.bytes_pulled = 0

    def pull(self, src_rank: int, src_ids, dst_ids, stream_ptr):
        n = len(src_ids)
        if n == 0:
            return
        descs = (capi.PkvPoolDesc * len(self.page_bytes))()
        for i, pb in enumerate(self.page_bytes):
            descs[i].src_base = self.peers.base(src_rank, i)
            descs[i].dst_base = self.peers.base(self.peers.rank, i)
            descs[i].page_bytes = pb
        ids = self.torch.tensor(np.concatenate([src_ids, dst_ids]).astype(np.int32), device="cuda")
        capi.check(self.lib.pkv_copy_pages(descs, len(self.page_bytes), ids.data_ptr(), ids.data_ptr() + 4 * n, n,
                                           self.num_pages, self.num_pages, stream_ptr))
        self._keep = ids
        self.bytes_pulled += n * sum(self.page_bytes)


def migrate(dist, rank: int, world: int, pool, seqs: dict, lengths: dict, outgoing, transport, stream_ptr=None,
            sync=lambda: None):
    """One migration event; every rank calls it (collectively) with its own outgoing list [(request, dst_rank)].

    pool: this rank's pkv_pool handle; seqs: request -> sequence handle in this pool; lengths: request -> rows held.
    Returns the moves that arrived here as [(request, new handle, length)]. `sync` must wait for the transport's copies
    (torch.cuda.synchronize on a GPU)."""
    lib = capi.lib()
    sync()                                       # this rank's own writes to the pages are complete before anyone pulls
    mine = []
    for request, dst in outgoing:
        h = seqs[request]
        n = lib.pkv_pool_seq_pages(pool, h, None, 0)
        pages = np.zeros(max(n, 1), np.int32)
        lib.pkv_pool_seq_pages(pool, h, pages.ctypes.data_as(i32p), n)
        mine.append(Move(request, rank, dst, lengths[request], pages[:n].tolist()))
    everyone = [None] * world
    dist.all_gather_object(everyone, mine)
    arrived = []
    for moves in everyone:                       # rank order, then each rank's own order: deterministic page ids
        for mv in moves:
            if mv.dst != rank:
                continue
            h = lib.pkv_pool_seq_open(pool)
            if lib.pkv_pool_assign_slot(pool, h) < 0 or lib.pkv_pool_alloc(pool, h, mv.length) != 1:
                raise RuntimeError(f"rank {rank}: no room for migrated request {mv.request} ({mv.length} rows)")
            n = lib.pkv_pool_seq_pages(pool, h, None, 0)
            dst_pages = np.zeros(max(n, 1), np.int32)
            lib.pkv_pool_seq_pages(pool, h, dst_pages.ctypes.data_as(i32p), n)
            assert n == len(mv.src_pages)
            transport.pull(mv.src, np.asarray(mv.src_pages, np.int32), dst_pages[:n], stream_ptr)
            arrived.append((mv.request, h, mv.length))
    sync()
    dist.barrier()                               # every payload has landed before any source page is released
    for mv in mine:
        capi.check(lib.pkv_pool_seq_close(pool, seqs.pop(mv.request)))
        lengths.pop(mv.request)
    for request, h, length in arrived:
        seqs[request] = h
        lengths[request] = length
    return arrived
