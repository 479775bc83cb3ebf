"""The snapshot store (unholy_b200/csrc/snapshot_store.{hpp,cpp}, pkv_snap_*): which snapshot slot a save goes into,
which one a prefix hit restores, eviction, and the disk tier. CPU only.

Part 1 — differential against the reference's own, unmodified engine (oracle/_ref/libref_engine.so): with few RAM
snapshot slots and no disk, the snapshot ids in every step's restore and save lists (StepInput::restore / save,
src/engine/step.hpp:67) and the snapshot counters after every iterate() must equal the reference's, through prefix
hits, decoding saves that supersede each other (rolling / stale), and eviction of the least recently used snapshot.

Part 2 — the disk tier by its rules (the I/O thread makes a step-for-step differential timing-dependent, so this part
checks the stated behaviour, the matrix of tools/sched_test/main.cpp:490-700,770-818): spill keeps a reserve of RAM
slots free, a boundary only the disk has is read back into a free RAM slot byte for byte, a stalled disk holds nothing
up, a file corrupted behind the store's back fails the read and turns the tier off once, a load whose sequence went
away settles by itself."""
import ctypes as C
import threading

import numpy as np
import pytest

import pkv_testlib as tl
from test_page_pool import Replay, refeng, u64p, u8p  # noqa: F401  (refeng is a fixture)
from unholy_b200 import capi


class SnapReplay(Replay):
    """Replay with the prefix-hit boundaries, restores and saves taken from a pkv_snap store instead of a set."""

    def __init__(self, pkv, refeng, ram_slots, **kw):
        super().__init__(pkv, refeng, snapshots=ram_slots, **kw)
        self.snap = pkv.pkv_snap_create(ram_slots, None, 0, None, 0, capi.SNAP_IO_HOOK(0), None)
        self.restore, self.rolling, self.n_prompt = {}, {}, {}
        self.slot_of = {}
        self.saves_checked = self.restores_checked = 0

    def close(self):
        super().close()
        self.pkv.pkv_snap_destroy(self.snap)

    def submit(self, prompt, max_tokens, images=None):
        rid = super().submit(prompt, max_tokens, images)
        self.n_prompt[rid] = len(prompt)
        return rid

    def hashes(self, toks, n):
        return np.array([self.pkv.pkv_page_hash_keys(toks.ctypes.data_as(u64p), self.pt, i) for i in range(n)], np.uint64)

    def boundaries(self, rid, toks, limit):
        ok = np.zeros(max(limit, 1), np.uint8)
        cached = self.pkv.pkv_pool_cached_prefix_keys(self.pool, toks.ctypes.data_as(u64p), len(toks))
        hit = capi.PkvSnapHit()
        hs = self.hashes(toks, cached)
        capi.check(self.pkv.pkv_snap_match(self.snap, hs.ctypes.data_as(u64p), cached, None, C.byref(hit)))
        assert hit.disk_slot < 0
        self.restore[rid] = hit.snap if hit.pages else -1
        if hit.pages:
            ok[hit.pages - 1] = 1
        return ok

    def on_admit_failed(self, rid):
        if self.restore.get(rid, -1) >= 0:
            self.pkv.pkv_snap_put(self.snap, self.restore.pop(rid))

    def on_step(self, chunks, save_ops, restore_ops):
        pkv = self.pkv
        slot_to_rid = {int(slot): int(seq) for seq, slot, s0, cn in chunks}
        end_of = {int(seq): int(s0 + cn) for seq, slot, s0, cn in chunks}
        want_restores = [(slot, self.restore[slot_to_rid[slot]]) for slot in (int(c[1]) for c in chunks)
                         if self.restore.get(slot_to_rid[slot], -1) >= 0]
        assert restore_ops == want_restores, "restored snapshot ids differ"
        self.restores_checked += len(restore_ops)
        taken = []
        for slot, ref_id in save_ops:                     # plan order: take_snapshot per saving chunk
            got = pkv.pkv_snap_take(self.snap)
            assert got == ref_id, f"save goes into snapshot {got}, the reference uses {ref_id}"
            taken.append((slot, got))
            self.saves_checked += 1
        # completion, in plan order: the restored snapshot is released, each save is committed under its boundary's name
        saves = dict(taken)
        for seq, slot, s0, cn in chunks:
            rid = int(seq)
            if self.restore.get(rid, -1) >= 0:
                pkv.pkv_snap_put(self.snap, self.restore.pop(rid))
            if int(slot) in saves:
                end = end_of[rid]
                toks = self.keys(rid)
                h = int(pkv.pkv_page_hash_keys(toks.ctypes.data_as(u64p), self.pt, end // self.pt - 1))
                rid_roll = self.rolling.setdefault(rid, [C.c_int(-1), C.c_uint64(0)])
                pkv.pkv_snap_commit(self.snap, saves[int(slot)], h, 1 if end > self.n_prompt[rid] else 0, C.byref(rid_roll[0]),
                                    C.byref(rid_roll[1]))

    def on_counters(self, snapshots, free_snapshots):
        c = capi.PkvSnapCounters()
        capi.check(self.pkv.pkv_snap_counters(self.snap, C.byref(c)))
        assert (c.cached, c.free_or_evictable) == (snapshots, free_snapshots), "snapshot counters differ"


@pytest.mark.parametrize("ram_slots", [3, 6, 24])
def test_snapshot_ids_match_reference_engine(pkv, refeng, ram_slots):
    g = tl.rng(600 + ram_slots)
    pt = 16
    r = SnapReplay(pkv, refeng, ram_slots, num_pages=512, page_tokens=pt, slots=4, pps=64, budget=256)
    try:
        bases = [g.integers(2, 500, size=int(n)).astype(np.int32) for n in g.integers(3 * pt, 14 * pt, size=5)]
        for rounds in range(4):
            for j in g.permutation(len(bases)):
                tail = g.integers(2, 500, size=int(g.integers(1, 3 * pt))).astype(np.int32)
                # decodes that cross several page boundaries: every completed page saves and supersedes the previous save
                r.submit(np.concatenate([bases[j], tail]) if rounds else bases[j], int(g.integers(1, 5 * pt if j % 2 else pt)))
                for _ in range(int(g.integers(0, 4))):
                    r.iterate()
            r.drain()
        assert r.saves_checked > 30
        assert r.restores_checked > (5 if ram_slots >= 24 else -1)   # few slots are recycled before most prompts return
        assert pkv.pkv_pool_available(r.pool) == 512
    finally:
        r.close()


# ---- part 2: the disk tier -----------------------------------------------------------------------------------------
SNAP_BYTES = 8192


class DiskStore:
    def __init__(self, pkv, tmp_path, ram_slots, disk_slots, hook=None):
        self.pkv = pkv
        raw = np.zeros(ram_slots * SNAP_BYTES + 4096, np.uint8)
        off = (-raw.ctypes.data) % 4096                       # 4096-aligned, as StepModel::snapshot_host promises
        self.mem = raw[off:off + ram_slots * SNAP_BYTES].reshape(ram_slots, SNAP_BYTES)
        self._raw = raw
        self.hook = capi.SNAP_IO_HOOK(hook) if hook else capi.SNAP_IO_HOOK(0)
        self.s = pkv.pkv_snap_create(ram_slots, self.mem.ctypes.data, SNAP_BYTES, str(tmp_path).encode(), disk_slots, self.hook, None)
        self.roll = [C.c_int(-1), C.c_uint64(0)]

    def save(self, name, past_prompt=False, fill=None):
        """A save: take a slot, write the state, commit it under `name`. Returns the slot or -1."""
        sid = self.pkv.pkv_snap_take(self.s)
        if sid >= 0:
            self.mem[sid] = np.frombuffer(np.random.default_rng(name).bytes(SNAP_BYTES), np.uint8) if fill is None else fill
            self.pkv.pkv_snap_commit(self.s, sid, name, 1 if past_prompt else 0, C.byref(self.roll[0]), C.byref(self.roll[1]))
        return sid

    def expected(self, name):
        return np.frombuffer(np.random.default_rng(name).bytes(SNAP_BYTES), np.uint8)

    def match(self, names):
        hit = capi.PkvSnapHit()
        hs = np.array(names, np.uint64)
        capi.check(self.pkv.pkv_snap_match(self.s, hs.ctypes.data_as(u64p), len(names), None, C.byref(hit)))
        return hit

    def settle_io(self):
        self.pkv.pkv_snap_wait_idle(self.s)
        done = (capi.PkvSnapDone * 64)()
        n = self.pkv.pkv_snap_poll(self.s, done, 64)
        return [(d.write, d.ok, d.snap, d.load_id) for d in done[:max(n, 0)]]

    def counters(self):
        c = capi.PkvSnapCounters()
        capi.check(self.pkv.pkv_snap_counters(self.s, C.byref(c)))
        return c

    def close(self):
        self.pkv.pkv_snap_destroy(self.s)


def test_spill_and_load_round_trip(pkv, tmp_path):
    d = DiskStore(pkv, tmp_path, ram_slots=4, disk_slots=8)
    try:
        assert pkv.pkv_snap_disk_on(d.s) == 1
        names = list(range(101, 113))
        for nm in names:                                      # twelve prefixes through four RAM slots
            assert d.save(nm) >= 0                            # a slot is always found: spills keep two free
            pkv.pkv_snap_spill(d.s)
            d.settle_io()
            pkv.pkv_snap_spill(d.s)
            d.settle_io()
        c = d.counters()
        assert c.spills == 10 and c.on_disk == 8 and c.disk_write_bytes == c.spills * SNAP_BYTES   # 111 and 112 stay in RAM
        assert c.free_or_evictable == 4 and c.io_pending == 0
        # the oldest two were pushed out of the eight disk slots (least recently used first); 103 is only on disk
        assert d.match([101]).pages == 0 and d.match([102]).pages == 0
        hit = d.match([103])
        assert hit.pages == 1 and hit.disk_slot >= 0 and hit.snap >= 0
        d.mem[hit.snap] = 0
        lid = pkv.pkv_snap_start_load(d.s, C.byref(hit))
        assert lid > 0 and d.counters().io_pending == 1
        assert d.settle_io() == [(0, 1, hit.snap, lid)]
        assert np.array_equal(d.mem[hit.snap], d.expected(103))      # the bytes that were saved, checksum verified
        assert d.counters().disk_hits == 1 and d.counters().disk_read_bytes == SNAP_BYTES
        again = d.match([103])                                        # now cached in RAM as well: no second read
        assert again.pages == 1 and again.disk_slot < 0 and again.snap == hit.snap
        pkv.pkv_snap_put(d.s, hit.snap)
        pkv.pkv_snap_put(d.s, hit.snap)
        # the deepest boundary wins; a RAM hit is preferred unless the disk one is deeper
        deep = d.match([112, 104])
        assert deep.pages == 2 and deep.hash == 104
        if deep.disk_slot >= 0:
            pkv.pkv_snap_cancel_load(d.s, C.byref(deep))              # given up before the read was started
        pkv.pkv_snap_put(d.s, deep.snap)
        assert d.counters().io_pending == 0
    finally:
        d.close()
    assert not (tmp_path / "snapshots.bin").exists()                  # entries do not outlive the store


def test_stalled_disk_holds_nothing_up(pkv, tmp_path):
    gate = threading.Event()
    d = DiskStore(pkv, tmp_path, ram_slots=3, disk_slots=4, hook=lambda write, user: gate.wait(5))
    try:
        assert d.save(1) >= 0 and d.save(2) >= 0
        pkv.pkv_snap_spill(d.s)                                       # one slot free, reserve is two: a write is queued ...
        assert d.counters().io_pending == 1
        assert d.save(3) >= 0                                         # ... and stalls; the last free slot is still usable
        assert pkv.pkv_snap_take(d.s) == -1                           # nothing droppable while the disk holds the write:
        assert pkv.pkv_snap_spare(d.s) == 0                           # a save is skipped rather than losing a prefix
        assert d.match([2]).pages == 1                                # prefix hits go on
        pkv.pkv_snap_put(d.s, d.match([2]).snap)
        pkv.pkv_snap_put(d.s, d.match([2]).snap)
        pkv.pkv_snap_put(d.s, d.match([2]).snap)
        gate.set()
        assert [x[:2] for x in d.settle_io()] == [(1, 1)]
        assert d.counters().on_disk == 1 and pkv.pkv_snap_take(d.s) >= 0
    finally:
        gate.set()
        d.close()


def test_corrupt_file_fails_the_read_and_turns_the_tier_off(pkv, tmp_path):
    d = DiskStore(pkv, tmp_path, ram_slots=3, disk_slots=4)
    try:
        for nm in (11, 12, 13, 14):
            assert d.save(nm) >= 0
            pkv.pkv_snap_spill(d.s)
            d.settle_io()
        pkv.pkv_snap_spill(d.s)
        d.settle_io()
        hit = d.match([11])
        assert hit.pages == 1 and hit.disk_slot >= 0
        with open(tmp_path / "snapshots.bin", "r+b") as f:            # someone scribbles over the slot
            f.seek(hit.disk_slot * SNAP_BYTES + 100)
            f.write(b"\\xff\\x00\\xff\\x00")
        lid = pkv.pkv_snap_start_load(d.s, C.byref(hit))
        assert d.settle_io() == [(0, 0, hit.snap, lid)]               # the read fails its checksum ...
        assert pkv.pkv_snap_disk_on(d.s) == 0                         # ... and the tier is off from now on
        pkv.pkv_snap_put(d.s, hit.snap)                               # the sequence recomputes; its empty slot is free again
        assert d.match([11]).pages == 0
        assert d.save(15) >= 0                                        # RAM-only bookkeeping continues (plain LRU)
        pkv.pkv_snap_spill(d.s)
        assert d.counters().io_pending == 0
    finally:
        d.close()


def test_load_whose_sequence_went_away_settles_itself(pkv, tmp_path):
    gate = threading.Event()
    d = DiskStore(pkv, tmp_path, ram_slots=3, disk_slots=4, hook=lambda write, user: gate.wait(5) if not write else None)
    try:
        for nm in (21, 22, 23):
            assert d.save(nm) >= 0
            pkv.pkv_snap_spill(d.s)
            d.settle_io()
        pkv.pkv_snap_spill(d.s)
        d.settle_io()
        hit = d.match([21])
        assert hit.disk_slot >= 0
        before = d.counters().free_or_evictable
        pkv.pkv_snap_start_load(d.s, C.byref(hit))                    # the read stalls ...
        pkv.pkv_snap_put(d.s, hit.snap)                               # ... and the request is aborted meanwhile
        assert d.counters().free_or_evictable == before               # the slot stays out until the read is over
        gate.set()
        assert [x[:2] for x in d.settle_io()] == [(0, 1)]
        c = d.counters()
        assert c.free_or_evictable == before + 1 and c.io_pending == 0
        assert d.match([21]).disk_slot < 0                            # the read made it a RAM snapshot after all
    finally:
        gate.set()
        d.close()


def test_rolling_saves_go_stale_and_are_dropped_not_spilled(pkv, tmp_path):
    d = DiskStore(pkv, tmp_path, ram_slots=4, disk_slots=4)
    try:
        for nm in (31, 32, 33):                                       # a decoding sequence saves at every page it completes
            assert d.save(nm, past_prompt=True) >= 0
        # Each superseded save went to the FRONT of the eviction order: 32, then 31, then the live 33. One slot is free,
        # the reserve is two: the stale 32 is dropped, not written.
        pkv.pkv_snap_spill(d.s)
        assert d.counters().io_pending == 0 and d.counters().spills == 0
        assert d.match([32]).pages == 0 and d.match([33]).pages == 1 and d.match([31]).pages == 1
    finally:
        d.close()
