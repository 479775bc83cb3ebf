"""The sharded pool's C++ host (pkv_shards_*): requests owned round-robin, decode steps issued by one host thread per
shard, and migration overlapped with the steps of the other requests — the destination pulls the pages of every layer
with plain loads from the source's pools and the request then decodes on its new owner. Two shards on ONE device (the
run that a single-GPU box can make: same code, same kernels, the "peer" pool is just another allocation) and, where the
box has two GPUs, two shards on two devices with the pull crossing NVLink. Every request, read back through its
current owner's block table, must equal what its owners wrote; the CPU oracle checks the gathered tiles of a step.
Sharding and migration have no reference counterpart (parity unpinned): the rule is the one of the allocator's
pkv_pool_migrate, which tests/test_page_pool_rules.py pins on the CPU."""
import ctypes as C

import numpy as np
import pytest

import pkv_testlib as tl
from oracle import oracle_lib as orc
from unholy_b200 import capi

pytestmark = pytest.mark.gpu
LAYERS, PAGES, SLOTS, PPS, K = 3, 160, 8, 40, 64


def content(request, n, layer):
    """Row p of a request before any decode step: a pattern of (request, position, layer)."""
    p = np.arange(n, dtype=np.int64)[:, None]
    c = np.arange(tl.W, dtype=np.int64)[None, :]
    return ((request * 40503 + p * 9973 + layer * 613 + c * 31) & 0x7FFF).astype(np.uint16)


def run_shards(pkv, torch, devices):
    G = len(devices)
    cfg = capi.PkvShardConfig(G, PAGES, tl.RPP, tl.W, tl.W, LAYERS, SLOTS, PPS, K, 0)
    devs = (C.c_int * G)(*devices)
    S = pkv.pkv_shards_create(C.byref(cfg), devs)
    assert S, pkv.pkv_last_error()
    g = tl.rng(77)
    lengths = {r: int(n) for r, n in enumerate(g.integers(70, 900, size=7))}
    written = {r: [content(r, n, l) for l in range(LAYERS)] for r, n in lengths.items()}
    keep = []

    def on(shard):
        torch.cuda.set_device(devices[shard])
        return C.c_void_p(pkv.pkv_shards_stream(S, shard))

    def dev(a):
        t = torch.from_numpy(np.ascontiguousarray(a).view(np.uint8).reshape(-1)).cuda()
        keep.append(t)
        return t

    try:
        for r, n in lengths.items():
            capi.check(pkv.pkv_shards_add(S, r, r % G, n))
        for r, n in lengths.items():      # the owners write their requests through the single-sequence entry point
            sh = pkv.pkv_shards_owner(S, r)
            st = on(sh)
            tab = pkv.pkv_shards_tables(S, sh) + pkv.pkv_shards_slot(S, r) * PPS * 4
            for l in range(LAYERS):
                capi.check(pkv.pkv_store_rows(dev(written[r][l]).data_ptr(), n, tl.W, pkv.pkv_shards_row_pool(S, sh, l), tab,
                                              tl.RPP, tl.W, 0, st))
        capi.check(pkv.pkv_shards_sync(S))

        def step(check_gather=False):
            """One decode step on every shard; each request appends a fresh random row per layer."""
            io = (capi.PkvShardIo * (G * LAYERS))()
            plan = []
            for sh in range(G):
                on(sh)
                ids = (C.c_int32 * SLOTS)()
                q = pkv.pkv_shards_local(S, sh, ids, SLOTS)
                order = list(ids[:q])
                for l in range(LAYERS):
                    rows = tl.normal_bf16(g, (max(q, 1), tl.W))
                    idx = np.full((max(q, 1), K), -1, np.int32)
                    for i, r in enumerate(order):
                        n = pkv.pkv_shards_length(S, r) + 1
                        m = min(K, n)
                        idx[i, :m] = np.sort(g.choice(n, size=m, replace=False))
                        idx[i, m - 1] = n - 1                 # the row appended in this very step is gathered too
                    out = torch.full((max(q, 1) * K * tl.W,), -1, dtype=torch.int16, device="cuda")
                    keep.append(out)
                    x = io[sh * LAYERS + l]
                    x.rows, x.idx, x.gathered = dev(rows).data_ptr(), dev(idx).data_ptr(), out.data_ptr()
                    plan.append((sh, l, order, rows, idx, out))
            capi.check(pkv.pkv_shards_step(S, io))
            for sh, l, order, rows, idx, out in plan:
                for i, r in enumerate(order):
                    written[r][l] = np.concatenate([written[r][l], rows[i:i + 1]])
            if check_gather:
                capi.check(pkv.pkv_shards_sync(S))
                for sh, l, order, rows, idx, out in plan:
                    torch.cuda.set_device(devices[sh])
                    got = out.cpu().numpy().view(np.uint16).reshape(-1, K, tl.W)
                    for i, r in enumerate(order):
                        want = np.zeros((K, tl.W), np.uint16)
                        sel = idx[i] >= 0
                        want[sel] = written[r][l][idx[i][sel]]
                        assert np.array_equal(got[i], want), (r, l)

        def read_back(requests):
            for r in requests:
                sh = pkv.pkv_shards_owner(S, r)
                st = on(sh)
                n = pkv.pkv_shards_length(S, r)
                tab = pkv.pkv_shards_tables(S, sh) + pkv.pkv_shards_slot(S, r) * PPS * 4
                d_idx, d_vis = dev(np.arange(n, dtype=np.int32)), dev(np.array([n], np.int32))
                for l in range(LAYERS):
                    out = torch.empty(n * tl.W, dtype=torch.int16, device="cuda")
                    capi.check(pkv.pkv_gather_rows(pkv.pkv_shards_row_pool(S, sh, l), tab, tl.RPP, tl.W, tl.W, d_idx.data_ptr(),
                                                   d_vis.data_ptr(), 1, n, out.data_ptr(), st))
                    torch.cuda.synchronize()
                    assert np.array_equal(out.cpu().numpy().view(np.uint16).reshape(n, tl.W), written[r][l]), (r, l)

        step(check_gather=True)
        step()
        # migration while the other requests keep stepping
        movers = np.array([0, 3, 4], np.int32)
        dsts = np.array([(pkv.pkv_shards_owner(S, int(r)) + 1) % G for r in movers], np.int32)
        free_before = [pkv.pkv_shards_free_pages(S, sh) for sh in range(G)]
        i32p = C.POINTER(C.c_int32)
        capi.check(pkv.pkv_shards_migrate_begin(S, movers.ctypes.data_as(i32p), dsts.ctypes.data_as(i32p), len(movers)))
        assert pkv.pkv_shards_migrate_pending(S) == len(movers)
        local_now = sum(pkv.pkv_shards_local(S, sh, None, 0) for sh in range(G))
        assert local_now == len(lengths) - len(movers)        # the movers sit out ...
        step(check_gather=True)                               # ... while everyone else steps (overlapping the pulls)
        assert pkv.pkv_shards_migrate_end(S, 1) == len(movers)
        for r, d in zip(movers, dsts):
            assert pkv.pkv_shards_owner(S, int(r)) == d
        if G > 1:
            assert sum(pkv.pkv_shards_free_pages(S, sh) for sh in range(G)) <= sum(free_before)   # nothing leaked, steps took pages
        nbytes, ms = C.c_double(0), (C.c_float * G)()
        capi.check(pkv.pkv_shards_migrate_stats(S, C.byref(nbytes), ms))
        want_bytes = sum(-(-pkv.pkv_shards_length(S, int(r)) // tl.RPP) for r in movers) * LAYERS * tl.PAGE_BYTES
        assert nbytes.value == want_bytes and sum(ms) > 0
        step(check_gather=True)                               # the migrated requests decode on their new owner
        step()
        capi.check(pkv.pkv_shards_sync(S))
        read_back(sorted(lengths))
        # a request that finishes gives its pages back; a full destination refuses a migration and nothing changes
        capi.check(pkv.pkv_shards_remove(S, 1))
        big = np.array([2], np.int32)
        filler = 100
        dst = (pkv.pkv_shards_owner(S, 2) + 1) % G if G > 1 else 0
        while pkv.pkv_shards_add(S, filler, dst, tl.RPP * 8) == capi.PKV_OK and filler < 100 + SLOTS:
            filler += 1
        if G > 1:
            rc = pkv.pkv_shards_migrate_begin(S, big.ctypes.data_as(i32p), np.array([dst], np.int32).ctypes.data_as(i32p), 1)
            assert rc == capi.PKV_ERR_LIMIT and pkv.pkv_shards_migrate_pending(S) == 0
            assert pkv.pkv_shards_owner(S, 2) != dst
        read_back([2])
        assert tl.device_status(pkv) == 0
    finally:
        torch.cuda.set_device(devices[0])
        pkv.pkv_shards_destroy(S)


def test_two_shards_on_one_device(pkv, cuda):
    run_shards(pkv, cuda, [cuda.cuda.current_device()] * 2)


def test_two_shards_on_two_devices(pkv, cuda):
    if cuda.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    run_shards(pkv, cuda, [0, 1])
    cuda.cuda.set_device(0)
