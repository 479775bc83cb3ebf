"""The snapshot store (unholy_b200/csrc/snapshot_store.{hpp,cpp}, pkv_snap_*): which snapshot slot a save goes into,
which one a prefix hit restores, eviction, and the disk tier. CPU only.

Part 1 — differential against the reference's own, unmodified engine (oracle/_ref/libref_engine.so): with few RAM
snapshot slots and no disk, the snapshot ids in every step's restore and save lists (StepInput::restore / save,
src/engine/step.hpp:67) and the snapshot counters after every iterate() must equal the reference's, through prefix
hits, decoding saves that supersede each other (rolling / stale), and eviction of the least recently used snapshot.

Part 1b — the same differential with the disk tier of both sides on. Every disk operation is held at a gate in the I/O
hook and let through between two iterate() calls, a fixed number of calls after it was queued, so both sides see their
completions at the same points: spills, reads of prefixes only the disk has, recycled disk slots, a corrupted file
(tools/sched_test/main.cpp:490-700) and aborts while a read is out (:770-818) must leave the same snapshot ids, block
tables and counters as the reference after every iterate().

Part 2 — the disk tier by its rules, where bytes matter (the recording model's snapshot contents are not compared in
part 1b): a boundary only the disk has is read back into a free RAM slot byte for byte, a stalled disk holds nothing
up, a file corrupted behind the store's back fails the read and turns the tier off once, a load whose sequence went
away settles by itself."""
import ctypes as C
import threading

import numpy as np
import pytest

import pkv_testlib as tl
from test_page_pool import Replay, refeng, u64p, u8p  # noqa: F401  (refeng is a fixture)
from unholy_b200 import capi


SNAP_BYTES = 8192


class SnapReplay(Replay):
    """Replay with the prefix-hit boundaries, restores and saves taken from a pkv_snap store instead of a set."""

    def __init__(self, pkv, refeng, ram_slots, **kw):
        super().__init__(pkv, refeng, snapshots=ram_slots, **kw)
        self.snap = self.make_store(ram_slots)
        self.restore, self.rolling, self.n_prompt = {}, {}, {}
        self.slot_of = {}
        self.saves_checked = self.restores_checked = 0

    def make_store(self, ram_slots):
        return self.pkv.pkv_snap_create(ram_slots, None, 0, None, 0, capi.SNAP_IO_HOOK(0), None)

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
        self.on_hit(rid, hit)
        self.restore[rid] = hit.snap if hit.pages else -1
        if hit.pages:
            ok[hit.pages - 1] = 1
        return ok

    def on_hit(self, rid, hit):
        assert hit.disk_slot < 0

    def on_admit_failed(self, rid):
        if self.restore.get(rid, -1) >= 0:
            self.pkv.pkv_snap_put(self.snap, self.restore.pop(rid))

    def on_finished(self, rid):                           # a request that ends before its restore was used (an abort)
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
        for slot, ref_id in self.take_order(chunks, save_ops):   # take_snapshot per saving chunk
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

    def take_order(self, chunks, save_ops):
        return save_ops                                   # plan order

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


# ---- part 1b: the same differential with the disk tier on ----------------------------------------------------------
class Gate:
    """The store's I/O hook under the test's control, the twin of the reference driver's gate: operation number i waits
    until `released` exceeds i; release(n, more, idle) returns when those n operations have completed: with `more`
    operations queued behind them, when the next one has reached the gate; with none, when idle() (the store's own
    wait for an empty queue) returns."""

    def __init__(self):
        self.cv = threading.Condition()
        self.started = self.released = 0
        self.open = False

    def hook(self, write, user):
        with self.cv:
            i = self.started
            self.started += 1
            self.cv.notify_all()
            self.cv.wait_for(lambda: self.open or self.released > i, timeout=20)

    def release(self, n, more, idle):
        with self.cv:
            self.released += n
            target = self.released
            self.cv.notify_all()
            assert self.cv.wait_for(lambda: self.started >= target + (1 if more else 0), timeout=10), \
                "a released disk operation never started"
        if not more:
            idle()

    def open_for_good(self):
        with self.cv:
            self.open = True
            self.cv.notify_all()


class DiskReplay(SnapReplay):
    """SnapReplay with both disk tiers on. Disk operations complete between iterate() calls, `delay` calls after they
    were queued, on both sides alike; what is compared is everything SnapReplay compares plus, after every iterate(),
    the snapshots on disk, the operations in flight, the spill and the disk-hit counts."""

    def __init__(self, pkv, refeng, ram_slots, tmp_path, disk_slots, delay, **kw):
        self.gate, self.delay, self.disk_slots = Gate(), delay, disk_slots
        self.dir_mine = tmp_path / "mine"
        self.dir_mine.mkdir()
        raw = np.zeros(ram_slots * SNAP_BYTES + 4096, np.uint8)
        off = (-raw.ctypes.data) % 4096
        self._raw, self.mem = raw, raw[off:off + ram_slots * SNAP_BYTES].reshape(ram_slots, SNAP_BYTES)
        self.hook = capi.SNAP_IO_HOOK(self.gate.hook)
        (tmp_path / "ref").mkdir()
        super().__init__(pkv, refeng, ram_slots, disk=(tmp_path / "ref", disk_slots), **kw)
        self.hits, self.loading, self.ages, self.cut = {}, {}, [], {}
        self.saves = 0
        self.loads_done = self.loads_failed = self.spills_seen = self.max_in_flight = 0
        self.expect_failure = False

    def make_store(self, ram_slots):
        s = self.pkv.pkv_snap_create(ram_slots, self.mem.ctypes.data, SNAP_BYTES, str(self.dir_mine).encode(), self.disk_slots,
                                     self.hook, None)
        assert self.pkv.pkv_snap_disk_on(s) == 1
        return s

    def close(self):
        self.gate.open_for_good()
        super().close()

    def on_hit(self, rid, hit):
        if hit.pages and hit.disk_slot >= 0:
            self.hits[rid] = capi.PkvSnapHit.from_buffer_copy(hit)

    def on_admit_failed(self, rid):
        if rid in self.hits:                                  # not started: the disk slot goes back, then the RAM slot
            self.pkv.pkv_snap_cancel_load(self.snap, C.byref(self.hits.pop(rid)))
        super().on_admit_failed(rid)

    def on_admitted(self, rid):
        # the prompt's last page boundary, where its prefill stops to save (set_cut, src/engine/engine.cpp:411-416)
        cut = (self.n_prompt[rid] - 1) // self.pt * self.pt
        self.cut[rid] = cut if cut > self.computed[rid] else 0
        if rid in self.hits:
            self.loading[int(self.pkv.pkv_snap_start_load(self.snap, C.byref(self.hits.pop(rid))))] = rid

    def on_iterate_begin(self):
        done = (capi.PkvSnapDone * 64)()
        n = self.pkv.pkv_snap_poll(self.snap, done, 64)
        for d in done[:max(n, 0)]:
            assert d.ok or self.expect_failure, "a disk operation failed"
            if d.write:
                continue
            rid = self.loading.pop(int(d.load_id))
            self.loads_done += 1
            if not d.ok and rid in self.running:          # drop_prefix (src/engine/engine.cpp:419-425): start over
                self.loads_failed += 1
                capi.check(self.pkv.pkv_pool_drop_prefix(self.pool, self.handle[rid]))
                self.pkv.pkv_snap_put(self.snap, self.restore.pop(rid))
                self.computed[rid] = 0
                self.cut[rid] = (self.n_prompt[rid] - 1) // self.pt * self.pt

    def on_step(self, chunks, save_ops, restore_ops):
        for seq, slot, s0, cn in chunks:
            assert int(seq) not in self.loading.values(), "a sequence whose prefix is still being read was scheduled"
            assert int(seq) not in self.aborted
        for slot, sid in save_ops:                            # a save changes the snapshot's bytes (they are checksummed)
            self.saves += 1
            self.mem[sid] = np.frombuffer(np.random.default_rng(self.saves).bytes(SNAP_BYTES), np.uint8)
        super().on_step(chunks, save_ops, restore_ops)

    def take_order(self, chunks, save_ops):
        """With the disk tier the saves at a prompt's last boundary take their slots before the others do
        (src/engine/engine.cpp:704-707); within each group, plan order."""
        musts = set()
        if not self.pkv.pkv_snap_disk_on(self.snap):
            return save_ops
        for seq, slot, s0, cn in chunks:
            if self.cut.get(int(seq), 0) == int(s0 + cn) != 0:
                musts.add(int(slot))
                self.cut[int(seq)] = 0
        return [op for op in save_ops if op[0] in musts] + [op for op in save_ops if op[0] not in musts]

    def on_iterate_end(self):
        self.pkv.pkv_snap_spill(self.snap)

    def on_disk_counters(self, disk_snapshots, snapshot_io, spills, disk_hits):
        c = capi.PkvSnapCounters()
        capi.check(self.pkv.pkv_snap_counters(self.snap, C.byref(c)))
        assert (c.on_disk, c.io_pending, c.spills, c.disk_hits) == (disk_snapshots, snapshot_io, spills, disk_hits), \
            "disk counters differ"
        self.spills_seen = spills
        self.max_in_flight = max(self.max_in_flight, snapshot_io)
        # Operations released after the previous iterate() were completed before this one and taken by its poll; the rest
        # of snapshot_io is still at the gate. Those queued `delay` iterate() calls ago are let through now, in order.
        new = snapshot_io - len(self.ages)
        assert new >= 0
        self.ages = [a + 1 for a in self.ages] + [0] * new
        n = sum(1 for a in self.ages if a >= self.delay)
        if n:
            more = len(self.ages) > n
            self.ref.refeng_io_release(self.eng, n, 1 if more else 0)
            self.gate.release(n, more, lambda: self.pkv.pkv_snap_wait_idle(self.snap))
            self.ages = self.ages[n:]

    def settle(self):
        """Runs the engine until no disk operation is queued or in flight."""
        for _ in range(10 * (self.delay + 2)):
            self.iterate()
            if not self.ages:
                self.iterate()                                # the poll that takes the last completions
                return
        raise AssertionError("disk operations never settled")


    def corrupt_files(self):
        """Someone scribbles over every slot of both snapshot files (as tools/sched_test/main.cpp:503-508 does)."""
        for path, size in ((self.dir_mine / "snapshots.bin", SNAP_BYTES), (self.dir_mine.parent / "ref" / "snapshots.bin", 4096)):
            with open(path, "r+b") as f:
                for d in range(self.disk_slots):
                    f.seek(d * size + 16)
                    f.write(b"\xff" * 8)


@pytest.mark.parametrize("ram_slots,disk_slots,delay", [(4, 24, 0), (3, 16, 1), (6, 12, 3), (5, 32, 2), (4, 5, 1)])
def test_disk_tier_matches_reference_engine(pkv, refeng, tmp_path, ram_slots, disk_slots, delay):
    """Prompts that return after their snapshot was pushed out of RAM: spills that keep the reserve free, prefixes read
    back from the file while other requests run, disk slots recycled least recently used first, stale rolling saves
    dropped instead of written. The reference's unmodified engine and the store see the same calls and the same
    completion points; every snapshot id and every counter must agree after every iterate()."""
    g = tl.rng(700 + 10 * ram_slots + delay)
    pt = 16
    r = DiskReplay(pkv, refeng, ram_slots, tmp_path, disk_slots, delay, num_pages=768, page_tokens=pt, slots=4, pps=64, budget=256)
    try:
        bases = [g.integers(2, 500, size=int(n)).astype(np.int32) for n in g.integers(3 * pt, 12 * pt, size=9)]
        for rounds in range(4):
            for j in g.permutation(len(bases)):
                tail = g.integers(2, 500, size=int(g.integers(1, 3 * pt))).astype(np.int32)
                r.submit(np.concatenate([bases[j], tail]) if rounds else bases[j], int(g.integers(1, 3 * pt if j % 2 else pt // 2)))
                for _ in range(int(g.integers(0, 5))):
                    r.iterate()
            r.drain()
            r.settle()
        assert r.spills_seen >= 6 and r.saves_checked > 30
        assert disk_slots < 12 or (r.loads_done >= 3 and r.restores_checked >= 3), (r.loads_done, r.restores_checked)
        assert delay == 0 or r.max_in_flight >= 2
        assert pkv.pkv_pool_available(r.pool) == 768
    finally:
        r.close()


# ---- part 2: the disk tier -----------------------------------------------------------------------------------------
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


def disk_scenario(pkv, refeng, tmp_path, seed, delay, ram_slots=4, disk_slots=24):
    """Nine prompts run once (their snapshots end up on disk), ready to return with a tail."""
    g = tl.rng(seed)
    pt = 16
    r = DiskReplay(pkv, refeng, ram_slots, tmp_path, disk_slots, delay, num_pages=768, page_tokens=pt, slots=4, pps=64, budget=256)
    bases = [g.integers(2, 500, size=int(n)).astype(np.int32) for n in g.integers(3 * pt, 12 * pt, size=9)]
    for b in bases:
        r.submit(b, 2)
        r.iterate()
    r.drain()
    r.settle()
    return r, g, bases


@pytest.mark.parametrize("delay", [0, 2])
def test_disk_tier_corrupt_file_matches_reference_engine(pkv, refeng, tmp_path, delay):
    """The snapshot file is corrupted behind both engines' backs: the next read fails its checksum, the request starts
    over from position 0 (its matched pages given back), the tier turns itself off, and everything after that runs on
    RAM snapshots alone. Same snapshot ids, tables and counters as the reference throughout."""
    r, g, bases = disk_scenario(pkv, refeng, tmp_path, 801 + delay, delay)
    try:
        r.corrupt_files()
        r.expect_failure = True
        for rounds in range(2):
            for j in g.permutation(len(bases)):
                r.submit(np.concatenate([bases[j], g.integers(2, 500, size=20).astype(np.int32)]), int(g.integers(1, 24)))
                for _ in range(int(g.integers(0, 4))):
                    r.iterate()
            r.drain()
            r.settle()
        assert r.loads_failed >= 1 and pkv.pkv_snap_disk_on(r.snap) == 0
        assert r.restores_checked >= 1                        # RAM hits go on after the tier went off
        assert pkv.pkv_pool_available(r.pool) == 768
    finally:
        r.close()


def test_disk_tier_abort_while_loading_matches_reference_engine(pkv, refeng, tmp_path):
    """Requests aborted while their prefix is being read from disk (the read is held at the gate for three iterate()
    calls): the slot and pages go back at once, the RAM snapshot slot and the disk slot only when the read completes
    (src/engine/engine.cpp:219-226, 1207-1224); a later request finds the prefix in RAM."""
    r, g, bases = disk_scenario(pkv, refeng, tmp_path, 901, delay=3, ram_slots=6)
    try:
        aborted = 0
        for n, j in enumerate(g.permutation(len(bases))):
            rid = r.submit(np.concatenate([bases[j], g.integers(2, 500, size=20).astype(np.int32)]), 8)
            r.iterate()
            if rid in r.loading.values() and aborted < 4:     # its read is at the gate
                r.abort(rid)
                aborted += 1
                if aborted % 2:                               # the same prefix again while the orphaned read is still out
                    r.submit(np.concatenate([bases[j], g.integers(2, 500, size=9).astype(np.int32)]), 3)
            for _ in range(1 + n % 5):
                r.iterate()
        r.drain()
        r.settle()
        assert aborted >= 3
        for j in range(len(bases)):                           # everything is still consistent afterwards
            r.submit(np.concatenate([bases[j], g.integers(2, 500, size=5).astype(np.int32)]), 2)
        r.drain()
        r.settle()
        assert pkv.pkv_pool_available(r.pool) == 768
    finally:
        r.close()
