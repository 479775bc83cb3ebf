"""Slot-state snapshots (ResidentModel::state_copies, src/engine/resident.hip:545-557): save copies every segment's
slice of a slot into the snapshot at the segment's offset, restore copies it back; an op outside the snapshot or slot
range is the reference's "step: bad state op". The CUDA path does all (op, segment) pairs of a call in one launch and
is compared byte for byte with the oracle's loop of copies, with the snapshots in device memory and in pinned host
memory (where the reference keeps them, resident.hip:538-541)."""
import ctypes as C

import numpy as np
import pytest

import pkv_testlib as tl
from oracle import oracle_lib as orc
from unholy_b200 import capi

SLOTS, SNAPSHOTS = 6, 5


def layout(g, sizes):
    """Segments as the reference lays them out (resident.hip:519-537): offsets accumulate, the snapshot is rounded up to
    4 KiB."""
    off, offs = 0, []
    for b in sizes:
        offs.append(off)
        off += b
    snap_bytes = (off + 4095) // 4096 * 4096
    bufs = [g.integers(0, 256, size=(SLOTS, b), dtype=np.uint8) for b in sizes]
    return bufs, offs, snap_bytes


def test_oracle_state_copies_round_trip():
    g = tl.rng(90)
    bufs, offs, snap_bytes = layout(g, [4096, 100, 131072, 48])
    snap = np.zeros(SNAPSHOTS * snap_bytes, np.uint8)
    before = [b.copy() for b in bufs]
    orc.state_copies(bufs, offs, [(2, 4), (0, 1)], snap, snap_bytes, True)
    for b, o in zip(before, offs):
        assert np.array_equal(snap[4 * snap_bytes + o: 4 * snap_bytes + o + b.shape[1]], b[2])
        assert np.array_equal(snap[1 * snap_bytes + o: 1 * snap_bytes + o + b.shape[1]], b[0])
    assert not snap[:snap_bytes].any()                                   # snapshot 0 untouched
    orc.state_copies(bufs, offs, [(5, 4)], snap, snap_bytes, False)       # restore snapshot 4 into slot 5
    for b, was in zip(bufs, before):
        assert np.array_equal(b[5], was[2]) and np.array_equal(b[:5], was[:5])


def seg_array(d_bufs, sizes, offs):
    segs = (capi.PkvStateSeg * len(sizes))()
    for i, (t, b, o) in enumerate(zip(d_bufs, sizes, offs)):
        segs[i] = capi.PkvStateSeg(t.data_ptr(), b, o)
    return segs


def op_array(ops):
    arr = (capi.PkvStateOp * len(ops))()
    for i, (slot, snapshot) in enumerate(ops):
        arr[i] = capi.PkvStateOp(slot, snapshot)
    return arr


@pytest.mark.gpu
@pytest.mark.parametrize("where", ["device", "pinned"])
def test_state_copies_gpu(pkv, cuda, where):
    g = tl.rng(91)
    # window rows, rings, a ragged size (byte path), more than 256 segments (two launches per call)
    sizes = [131072, 24576, 24576, 100, 4096 + 16] + [2048] * 260
    bufs, offs, snap_bytes = layout(g, sizes)
    snap = g.integers(0, 256, size=SNAPSHOTS * snap_bytes, dtype=np.uint8)
    d_bufs = [tl.dev(cuda, b) for b in bufs]
    if where == "device":
        d_snap = tl.dev(cuda, snap)
    else:
        d_snap = cuda.from_numpy(snap.copy()).pin_memory()
    segs = seg_array(d_bufs, sizes, offs)
    sp = tl.stream_ptr(cuda)
    save_ops, restore_ops = [(1, 0), (4, 3), (2, 2)], [(0, 3), (5, 0)]
    capi.check(pkv.pkv_state_copies(segs, len(sizes), op_array(save_ops), len(save_ops), d_snap.data_ptr(), snap_bytes,
                                    SNAPSHOTS, SLOTS, 1, sp))
    capi.check(pkv.pkv_state_copies(segs, len(sizes), op_array(restore_ops), len(restore_ops), d_snap.data_ptr(), snap_bytes,
                                    SNAPSHOTS, SLOTS, 0, sp))
    cuda.cuda.synchronize()
    orc.state_copies(bufs, offs, save_ops, snap, snap_bytes, True)
    orc.state_copies(bufs, offs, restore_ops, snap, snap_bytes, False)
    got_snap = tl.host(d_snap, np.uint8) if where == "device" else d_snap.numpy()
    assert np.array_equal(got_snap, snap)
    for t, b in zip(d_bufs, bufs):
        assert np.array_equal(tl.host(t, np.uint8, b.shape), b)


def test_state_copies_argument_errors(pkv):
    segs = (capi.PkvStateSeg * 1)(capi.PkvStateSeg(16, 64, 0))
    assert pkv.pkv_state_copies(segs, 1, op_array([(0, 0)]), 0, 16, 4096, 4, 4, 1, None) == capi.PKV_OK      # no ops
    for bad in ((0, 4), (4, 0), (-1, 0), (0, -1)):
        assert pkv.pkv_state_copies(segs, 1, op_array([bad]), 1, 16, 4096, 4, 4, 1, None) == capi.PKV_ERR_ARG
        assert pkv.pkv_last_error() == b"step: bad state op"
    assert pkv.pkv_state_copies(segs, 1, op_array([(0, 0)]), 1, 16, 32, 4, 4, 1, None) == capi.PKV_ERR_ARG   # segment past the end
    assert pkv.pkv_state_copies(segs, 1, op_array([(0, 0)]), 1, None, 4096, 4, 4, 1, None) == capi.PKV_ERR_ARG
