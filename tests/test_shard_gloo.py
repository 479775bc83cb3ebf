"""The sharded pool's host logic on the CPU: two `gloo` ranks, each with its own page pool and a pool of pages in
shared memory standing in for the IPC-mapped device pool. Requests are owned round-robin, written by their owner,
migrated back and forth by the collective protocol of unholy_b200/shard.py, and must read back unchanged through the
new owner's block table. The payload copy here is the CPU oracle's page move (the GPU path is covered by
tests/test_gpu_multi.py)."""
import os
import socket
from multiprocessing import shared_memory

import numpy as np
import pytest
import torch.distributed as dist
import torch.multiprocessing as mp

import pkv_testlib as tl

WORLD, PAGES, PPS, SLOTS = 2, 96, 24, 8


def content(request, length):
    g = tl.rng(1000 + request)
    return tl.normal_bf16(g, (length, tl.W))


def free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


class SharedPull:
    """Destination-side pull from the source rank's pool mapped through shared memory."""

    def __init__(self, pools, rank):
        self.pools, self.rank = pools, rank

    def pull(self, src_rank, src_ids, dst_ids, stream_ptr):
        from oracle import oracle_lib as orc
        orc.move_pages(self.pools[src_rank], self.pools[self.rank], tl.PAGE_BYTES, np.ascontiguousarray(src_ids),
                       np.ascontiguousarray(dst_ids))


def worker(rank, port, names, result):
    import ctypes as C

    from oracle import oracle_lib as orc
    from unholy_b200 import capi, shard
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=WORLD)
    lib = capi.lib()
    shms = [shared_memory.SharedMemory(name=n) for n in names]
    pools = [np.ndarray((PAGES * tl.RPP, tl.W), np.uint16, buffer=s.buf) for s in shms]
    pool = lib.pkv_pool_create(PAGES, tl.RPP, SLOTS, PPS, 1)
    seqs, lengths = {}, {}
    g = tl.rng(5)
    all_lengths = {r: int(n) for r, n in enumerate(g.integers(40, 700, size=8))}

    def table_of(h):
        t = np.ctypeslib.as_array(lib.pkv_pool_tables(pool), shape=(SLOTS, PPS))
        return t[lib.pkv_pool_seq_slot(pool, h)].copy()

    for r, n in all_lengths.items():
        if shard.owner(r, WORLD) != rank:
            continue
        h = lib.pkv_pool_seq_open(pool)
        assert lib.pkv_pool_assign_slot(pool, h) >= 0 and lib.pkv_pool_alloc(pool, h, n) == 1
        orc.store_rows(content(r, n), pools[rank], table_of(h), tl.RPP, tl.W, 0)
        seqs[r], lengths[r] = h, n
    transport = SharedPull(pools, rank)
    plan = [  # (request -> destination) per event; a request may come back
        {0: 1, 3: 0, 5: 0},
        {0: 0, 2: 1, 3: 1},
        {},
        {4: 1, 1: 0},
    ]
    for event in plan:
        outgoing = [(r, d) for r, d in event.items() if r in seqs and d != rank]
        shard.migrate(dist, rank, WORLD, pool, seqs, lengths, outgoing, transport)
    ok = True
    held = 0
    for r, h in seqs.items():
        n = lengths[r]
        idx = np.arange(n, dtype=np.int32).reshape(1, n)
        got = orc.gather_rows(pools[rank], table_of(h).reshape(1, -1), tl.RPP, tl.W, tl.W, idx, np.zeros(1, np.int32),
                              np.array([n], np.int32))[0]
        ok &= bool(np.array_equal(got, content(r, n)))
        held += -(-n // tl.RPP)
    ok &= lib.pkv_pool_available(pool) == PAGES - held          # nothing leaked on either side
    owners = [None] * WORLD
    dist.all_gather_object(owners, sorted(seqs))
    if rank == 0:
        ok &= sorted(owners[0] + owners[1]) == list(range(8))   # every request lives on exactly one shard
        result.put((ok, owners))
    else:
        result.put((ok, None))
    dist.barrier()
    dist.destroy_process_group()
    for s in shms:
        s.close()


def test_two_rank_ownership_and_migration():
    nbytes = PAGES * tl.RPP * tl.W * 2
    shms = [shared_memory.SharedMemory(create=True, size=nbytes) for _ in range(WORLD)]
    try:
        ctx = mp.get_context("spawn")
        result = ctx.Queue()
        port = free_port()
        procs = [ctx.Process(target=worker, args=(r, port, [s.name for s in shms], result)) for r in range(WORLD)]
        for p in procs:
            p.start()
        outs = [result.get(timeout=240) for _ in range(WORLD)]
        for p in procs:
            p.join(timeout=60)
            assert p.exitcode == 0
        assert all(o[0] for o in outs), outs
        owners = next(o[1] for o in outs if o[1] is not None)
        assert owners[0] == [0, 1, 5, 6] and owners[1] == [2, 3, 4, 7], owners
    finally:
        for s in shms:
            s.close()
            s.unlink()
