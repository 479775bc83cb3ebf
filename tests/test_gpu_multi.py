"""Migration between two GPUs: one process per GPU, each with its own page pool and cudaMalloc'd layer pools; pages
move by a pull kernel on the destination GPU that reads the source pool through a CUDA IPC mapping (ordinary loads over
NVLink). Requests written by their first owner must read back unchanged through the new owner's block table. Skipped
with fewer than two GPUs. Host messages go over gloo; no NCCL collective is involved in the data path."""
import os

import numpy as np
import pytest

import pkv_testlib as tl
from test_shard_gloo import content, free_port

pytestmark = pytest.mark.gpu
WORLD, PAGES, PPS, SLOTS, LAYERS = 2, 96, 24, 8, 2


def worker(rank, port, result):
    import ctypes as C

    import torch
    import torch.distributed as dist

    from unholy_b200 import capi, shard
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", rank=rank, world_size=WORLD)
    lib = capi.lib()
    sp = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    nbytes = PAGES * tl.PAGE_BYTES
    raw = []
    for _ in range(LAYERS):
        p = C.c_void_p()
        capi.check(lib.pkv_device_alloc(C.byref(p), nbytes))
        raw.append(p.value)
        z = torch.zeros(nbytes, dtype=torch.uint8, device="cuda")
        capi.check(lib.pkv_copy(p, z.data_ptr(), nbytes, sp))
    torch.cuda.synchronize()
    pool = lib.pkv_pool_create(PAGES, tl.RPP, SLOTS, PPS, 1)
    peers = shard.PeerPools(dist, rank, WORLD, raw)
    transport = shard.DevicePull(torch, peers, [tl.PAGE_BYTES] * LAYERS, PAGES)
    seqs, lengths = {}, {}
    g = tl.rng(5)
    all_lengths = {r: int(n) for r, n in enumerate(g.integers(40, 700, size=8))}

    def d_table(h):
        t = np.ctypeslib.as_array(lib.pkv_pool_tables(pool), shape=(SLOTS, PPS))
        return tl.dev(torch, t[lib.pkv_pool_seq_slot(pool, h)].copy())

    for r, n in all_lengths.items():
        if shard.owner(r, WORLD) != rank:
            continue
        h = lib.pkv_pool_seq_open(pool)
        assert lib.pkv_pool_assign_slot(pool, h) >= 0 and lib.pkv_pool_alloc(pool, h, n) == 1
        tab = d_table(h)
        for l in range(LAYERS):
            rows = tl.dev(torch, np.roll(content(r, n), l, axis=1))
            capi.check(lib.pkv_store_rows(rows.data_ptr(), n, tl.W, raw[l], tab.data_ptr(), tl.RPP, tl.W, 0, sp))
        torch.cuda.synchronize()
        seqs[r], lengths[r] = h, n
    plan = [{0: 1, 3: 0, 5: 0}, {0: 0, 2: 1, 3: 1}, {}, {4: 1, 1: 0}]
    for event in plan:
        outgoing = [(r, d) for r, d in event.items() if r in seqs and d != rank]
        shard.migrate(dist, rank, WORLD, pool, seqs, lengths, outgoing, transport, sp, torch.cuda.synchronize)
    ok = True
    for r, h in seqs.items():
        n = lengths[r]
        tab = d_table(h)
        idx = tl.dev(torch, np.arange(n, dtype=np.int32))
        vis = tl.dev(torch, np.array([n], np.int32))
        for l in range(LAYERS):
            out = torch.empty(n * tl.ROW_BYTES, dtype=torch.uint8, device="cuda")
            capi.check(lib.pkv_gather_rows(raw[l], tab.data_ptr(), tl.RPP, tl.W, tl.W, idx.data_ptr(), vis.data_ptr(), 1, n,
                                           out.data_ptr(), sp))
            torch.cuda.synchronize()
            ok &= bool(np.array_equal(tl.host(out, np.uint16, (n, tl.W)), np.roll(content(r, n), l, axis=1)))
    st = C.c_int(0)
    capi.check(lib.pkv_device_status(C.byref(st)))
    ok &= st.value == 0
    result.put((rank, ok, sorted(seqs), transport.bytes_pulled))
    dist.barrier()
    peers.close()
    dist.barrier()
    for p in raw:
        lib.pkv_device_free(C.c_void_p(p))
    dist.destroy_process_group()


def test_two_gpu_migration(cuda):
    if cuda.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    result = ctx.Queue()
    port = free_port()
    procs = [ctx.Process(target=worker, args=(r, port, result)) for r in range(WORLD)]
    for p in procs:
        p.start()
    outs = sorted(result.get(timeout=300) for _ in range(WORLD))
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    assert all(o[1] for o in outs), outs
    assert outs[0][2] == [0, 1, 5, 6] and outs[1][2] == [2, 3, 4, 7]
    assert outs[0][3] > 0 and outs[1][3] > 0
