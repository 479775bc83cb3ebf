#!/usr/bin/env python
"""Benchmark of the paged KV-cache hot path: one batched decode step over 43 layers.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--variant bulk|vec]

Workload ("decode43", benchmark configuration 2): 64 sequences at 128k context on every GPU, page size 64, a pool of
131,072 pages (8,388,608 tokens) that is exactly full, block tables shuffled. Per layer and step: append one bf16
576-wide row and one 128-wide MXFP4 key row per sequence, then gather 2048 distinct sorted positions per sequence out
of the scattered pages. A step is all 43 layers, one library call per layer (the call pattern of a real model, where
layer l+1's rows do not exist before layer l has run).

43 full-size layer pools (10.2 GB each) do not fit one GPU, so R resident pools are allocated (as many as fit) and
layer l uses pool l mod R; the traffic per step is unchanged and the working set stays far larger than L2.

Prints ONE JSON line (rank 0). `value` = algorithmic GB/s over all ranks with inputs resident in HBM; `e2e` = the same
metric with the step's host inputs copied in from pinned memory and a result sample copied back inside the timed
region; `roofline` compares the dominant kernel with the measured HBM copy peak; `cpu_baseline` times the CPU oracle
(a scalar C++ port of the reference's arithmetic) on the host cores on a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
for _p in (ROOT, ROOT / "tests"):
    if str(_p) not in sys.path:
        sys.path.insert(0, str(_p))

W, KEY_DIM, RPP, K_SEL, LAYERS, NSEQ = 576, 128, 64, 2048, 43, 64
CONTEXT = 131072                      # rows per sequence after the step's append
PAGES_PER_SEQ = CONTEXT // RPP        # 2048
NUM_PAGES = NSEQ * PAGES_PER_SEQ      # 131,072
ROW_BYTES = W * 2
PAGE_BYTES = RPP * ROW_BYTES          # 73,728
FP4_PAGE_BYTES = RPP * 68             # 4,352
# Algorithmic bytes (read + write) per sequence and layer.
APPEND_BYTES = 2 * ROW_BYTES + (KEY_DIM * 2 + 68)      # 2304 + 324
GATHER_BYTES = K_SEL * 2 * ROW_BYTES                   # 2048 rows read and written
STEP_BYTES_PER_GPU = LAYERS * NSEQ * (APPEND_BYTES + GATHER_BYTES)
# dram__bytes_read.sum + dram__bytes_write.sum of one per-layer launch (ncu capture summarised under profiles/).
NCU_TRAFFIC_BYTES_PER_LAUNCH = 248_560_000
WORKLOAD_NAME = "decode43: 64 seq x 128k ctx per GPU, page 64, 43 layers, bf16 576 rows + MXFP4 128 keys, top-2048 gather"


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--variant", choices=["bulk", "vec"], default=os.environ.get("PKV_BENCH_VARIANT", "bulk"))
    ap.add_argument("--layers-per-launch", type=int, default=1)
    ap.add_argument("--resident-layers", type=int, default=0, help="0 = as many pools as fit")
    ap.add_argument("--small", action="store_true", help="a reduced pool (for profiler captures and quick checks)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    return ap.parse_args()


def load_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


class ClockSampler(threading.Thread):
    """Reads SM clocks and throttle reasons through NVML while the timed region runs (read-only queries)."""

    def __init__(self, index: int, period=0.02):
        super().__init__(daemon=True)
        self.index, self.period = index, period
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._halt = threading.Event()
        self.ok = False
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
            self.ok = True
        except Exception:
            self.ok = False

    def run(self):
        if not self.ok:
            return
        nv = self.nv
        names = {
            getattr(nv, "nvmlClocksThrottleReasonHwSlowdown", 0x8): "hw_slowdown",
            getattr(nv, "nvmlClocksThrottleReasonHwThermalSlowdown", 0x40): "hw_thermal_slowdown",
            getattr(nv, "nvmlClocksThrottleReasonSwThermalSlowdown", 0x20): "sw_thermal_slowdown",
            getattr(nv, "nvmlClocksThrottleReasonSwPowerCap", 0x4): "sw_power_cap",
        }
        while not self._halt.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, name in names.items():
                    if r & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._halt.wait(self.period)

    def stop(self):
        self._halt.set()
        if self.is_alive():
            self.join(timeout=2)
        med = float(np.median(self.samples)) if self.samples else None
        return {"sm_mhz": med, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": len(self.samples)}


class Workload:
    """The decode43 step on one GPU: device pools, block tables, the step's inputs and the prepared library calls."""

    def __init__(self, torch, args, rank: int):
        from unholy_b200 import capi
        self.torch, self.capi, self.lib = torch, capi, capi.lib()
        self.context = 8192 if args.small else CONTEXT
        self.pps = self.context // RPP
        self.num_pages = NSEQ * self.pps
        self.variant = capi.PKV_VARIANT_BULK if args.variant == "bulk" else 0
        self.lpl = max(1, min(args.layers_per_launch, capi.PKV_MAX_LAYERS))
        dev = torch.device("cuda", torch.cuda.current_device())
        g = torch.Generator(device=dev)
        g.manual_seed(2 + 1000 * rank)
        pool_bytes = self.num_pages * PAGE_BYTES
        fp4_bytes = self.num_pages * FP4_PAGE_BYTES
        out_bytes = NSEQ * K_SEL * ROW_BYTES
        free, _total = torch.cuda.mem_get_info()
        fixed = LAYERS * (out_bytes + NSEQ * (ROW_BYTES + KEY_DIM * 2 + K_SEL * 4)) + (6 << 30)
        fit = int((free - fixed) // (pool_bytes + fp4_bytes))
        self.resident = max(1, min(LAYERS, args.resident_layers or (4 if args.small else fit)))
        if fit < 1:
            raise RuntimeError(f"not enough device memory for one layer pool ({free >> 30} GiB free)")
        # Block tables: a seeded permutation of all physical pages dealt to the sequences in order.
        perm = torch.randperm(self.num_pages, generator=g, device=dev).to(torch.int32)
        self.tables = perm.view(NSEQ, self.pps).contiguous()
        s0 = self.context - 1  # the appended row fills the last row of each sequence's last page
        self.chunks = torch.tensor([[s, s0, 1, s] for s in range(NSEQ)], dtype=torch.int32, device=dev)
        self.q_chunk = torch.arange(NSEQ, dtype=torch.int32, device=dev)
        self.q_visible = torch.full((NSEQ,), self.context, dtype=torch.int32, device=dev)
        # Pools: bf16 N(0,1) rows; MXFP4 key pools start as arbitrary bytes (only the appended rows are defined).
        self.pools, self.fp4 = [], []
        for _ in range(self.resident):
            p = torch.empty(pool_bytes // 2, dtype=torch.bfloat16, device=dev)
            p.normal_(generator=g)
            self.pools.append(p)
            self.fp4.append(torch.randint(0, 256, (fp4_bytes,), dtype=torch.uint8, device=dev, generator=g))
        # The step's inputs, per layer.
        self.rows = torch.randn(LAYERS, NSEQ, W, generator=g, device=dev).to(torch.bfloat16)
        mag = torch.ldexp(torch.ones(LAYERS, NSEQ, 1, device=dev),
                          torch.randint(-3, 4, (LAYERS, NSEQ, 1), generator=g, device=dev))
        self.keys = (torch.randn(LAYERS, NSEQ, KEY_DIM, generator=g, device=dev) * mag).to(torch.bfloat16)
        self.idx = torch.empty(LAYERS, NSEQ, K_SEL, dtype=torch.int32, device=dev)
        for l in range(LAYERS):  # 2048 distinct positions uniform in [0, context), sorted
            r = torch.rand(NSEQ, self.context, generator=g, device=dev)
            self.idx[l] = r.topk(K_SEL, dim=1).indices.sort(dim=1).values.to(torch.int32)
            del r
        self.out = torch.empty(LAYERS, NSEQ, K_SEL, W, dtype=torch.bfloat16, device=dev)
        self.out.fill_(float("nan"))
        # Prepared calls: one pkv_step_run per group of `lpl` layers.
        st = capi.PkvStep()
        st.width = st.row_stride = W
        st.rows_per_page, st.max_pages_per_seq, st.num_pages, st.fp8_block = RPP, self.pps, self.num_pages, 64
        st.nchunks = st.T = st.Q = NSEQ
        st.k = K_SEL
        st.tables, st.chunks = self.tables.data_ptr(), self.chunks.data_ptr()
        st.q_chunk, st.q_visible = self.q_chunk.data_ptr(), self.q_visible.data_ptr()
        self.step = st
        self.layers = (capi.PkvLayer * LAYERS)()
        for l in range(LAYERS):
            y = self.layers[l]
            y.rows, y.row_pool = self.rows[l].data_ptr(), self.pools[l % self.resident].data_ptr()
            y.keys, y.key_pool_fp4 = self.keys[l].data_ptr(), self.fp4[l % self.resident].data_ptr()
            y.idx, y.gathered = self.idx[l].data_ptr(), self.out[l].data_ptr()
        self.flags = capi.PKV_DO_ROWS | capi.PKV_DO_KEYS_FP4 | capi.PKV_DO_GATHER | self.variant
        self.groups = [(l, min(self.lpl, LAYERS - l)) for l in range(0, LAYERS, self.lpl)]
        self.group_ptrs = [C.cast(C.byref(self.layers, l * C.sizeof(capi.PkvLayer)), C.POINTER(capi.PkvLayer))
                           for l, _ in self.groups]
        fused = self.variant and (NSEQ + 1) // 2 * self.lpl <= 148   # the decode append rides in the gather launch
        self.kernels_per_call = 2 if (self.variant and not fused) else 1
        # Layers that share a resident pool and run in ONE launch write the same appended row in no defined order.
        self.unordered_alias = self.lpl > self.resident or (self.lpl > 1 and self.resident < LAYERS)
        self.step_ref = C.byref(self.step)

    def run_step(self, stream_ptr):
        run, check, flags, ref = self.lib.pkv_step_run, self.capi.check, self.flags, self.step_ref
        for ptr, (_, n) in zip(self.group_ptrs, self.groups):
            check(run(ref, ptr, n, flags, stream_ptr))

    @property
    def launches_per_step(self):
        return len(self.groups) * self.kernels_per_call

    def verify(self):
        """Size-independent check at full size: for sampled (layer, sequence) pairs the gathered tile equals the pool
        rows the block table names (torch indexing as the checker), and the appended row landed in its page."""
        torch = self.torch
        torch.cuda.synchronize()
        st = C.c_int(0)
        self.capi.check(self.lib.pkv_device_status(C.byref(st)))
        if st.value:
            return False, f"device status {st.value:#x}"
        for l in (0, 1, LAYERS // 2, LAYERS - 1):
            pool = self.pools[l % self.resident].view(-1, W)
            for s in (0, 17, NSEQ - 1):
                # a later layer that shares this pool overwrote the appended row: compare it only where it is the last writer
                last_writer = max(x for x in range(LAYERS) if x % self.resident == l % self.resident)
                pos = self.idx[l, s].long()
                phys = self.tables[s].long()[pos // RPP] * RPP + pos % RPP
                want = pool[phys]
                got = self.out[l, s]
                fresh = pos == self.context - 1
                want = want.clone()
                want[fresh] = self.rows[l, s]  # an entry inside the step's own chunk reads the row being appended
                if not torch.equal(got.view(torch.int16), want.view(torch.int16)):
                    return False, f"gathered tile differs at layer {l} sequence {s}"
                if l == last_writer and not self.unordered_alias:
                    ph = int(self.tables[s, self.pps - 1]) * RPP + RPP - 1
                    if not torch.equal(pool[ph].view(torch.int16), self.rows[l, s].view(torch.int16)):
                        return False, f"appended row differs at layer {l} sequence {s}"
        return True, "sampled tiles and appended rows match"


class CpuWorkload:
    """The CPU oracle on a bounded sample of the workload: ONE layer of the step (64 sequences at full context, block
    tables shuffled over a full-size host pool when host memory allows, else the largest power-of-two context that
    fits). layer_step() runs the layer's appends and gathers once with fresh index lists and returns the seconds."""

    def __init__(self, threads: int):
        import psutil

        from oracle import oracle_lib as orc
        self.orc, self.threads = orc, threads
        avail = psutil.virtual_memory().available
        context = CONTEXT
        while NSEQ * (context // RPP) * (PAGE_BYTES + FP4_PAGE_BYTES) * 1.3 > avail * 0.5 and context > 4096:
            context //= 2
        self.context, self.pps = context, context // RPP
        self.num_pages = NSEQ * self.pps
        g = self.g = np.random.Generator(np.random.MT19937(2))
        self.pool = np.empty((self.num_pages * RPP, W), np.uint16)
        block = orc.f32_to_bf16_bits(g.standard_normal((1 << 16, W), dtype=np.float32))
        for o in range(0, self.pool.shape[0], block.shape[0]):  # N(0,1) rows, tiled: a copy loop never reads values
            self.pool[o:o + block.shape[0]] = block[:self.pool.shape[0] - o]
        self.fp4 = np.zeros(self.num_pages * FP4_PAGE_BYTES, np.uint8)
        self.tables = g.permutation(self.num_pages).astype(np.int32).reshape(NSEQ, self.pps)
        self.chunks = np.array([[s, context - 1, 1, s] for s in range(NSEQ)], np.int32)
        self.q_slot = np.arange(NSEQ, dtype=np.int32)
        self.q_vis = np.full(NSEQ, context, np.int32)
        self.rows = orc.f32_to_bf16_bits(g.standard_normal((NSEQ, W), dtype=np.float32))
        self.keys = orc.f32_to_bf16_bits(g.standard_normal((NSEQ, KEY_DIM), dtype=np.float32))
        self.out = np.empty((NSEQ, K_SEL, W), np.uint16)
        self.layer_bytes = NSEQ * (APPEND_BYTES + GATHER_BYTES)
        self.layer_step()  # warm: first touch of the fresh allocations

    def layer_step(self) -> float:
        orc, g = self.orc, self.g
        idx = np.empty((NSEQ, K_SEL), np.int32)
        for s in range(NSEQ):
            idx[s] = np.sort(g.choice(self.context, size=K_SEL, replace=False))
        t0 = time.perf_counter()
        orc.store_rows_chunks(self.rows, self.pool, self.tables, RPP, W, self.chunks, self.threads)
        orc.store_rows_fp4_chunks(self.keys, self.fp4, self.tables, RPP, self.chunks, self.threads)
        orc.lib().orc_gather_rows(self.pool.ctypes.data, self.tables.ctypes.data, self.pps, RPP, W, W, idx.ctypes.data,
                                  self.q_slot.ctypes.data, self.q_vis.ctypes.data, NSEQ, K_SEL, self.out.ctypes.data,
                                  self.threads)
        return time.perf_counter() - t0

    def describe(self, n: int) -> str:
        return (f"{n} layer-steps of the decode43 step (64 sequences x [1 bf16 row + 1 MXFP4 key append, 2048-row "
                f"gather] = {self.layer_bytes / 1e6:.0f} MB each) at context {self.context} on a {self.num_pages}-page "
                f"host pool, {self.threads} thread(s)")


def cpu_baseline(threads: int, seconds_target: float = 10.0):
    wl = CpuWorkload(threads)
    times = []
    while sum(times) < seconds_target and len(times) < 86:
        times.append(wl.layer_step())
    gbs = wl.layer_bytes * len(times) / sum(times) / 1e9
    return gbs, wl.describe(len(times))


def run_reference_arm(args):
    """The reference arm: the reference's path on the host cores. The reference's kernels are HIP-only and have no CPU
    build, so this is its arithmetic restated in C++ (oracle/pkv_oracle.cpp, kind "port") on all host threads. Each
    step is a bounded sample: 2 of the 43 layers; ms_per_step extrapolates the sample's rate to the full step."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    from oracle import oracle_lib as orc
    threads = max(1, orc.hardware_threads())
    wl = CpuWorkload(threads)
    sample_layers = 2
    times = []
    for i in range(args.warmup + args.steps):
        dt = sum(wl.layer_step() for _ in range(sample_layers))
        if i >= args.warmup:
            times.append(dt)
    v = wl.layer_bytes * sample_layers * len(times) / sum(times) / 1e9 if times else 0.0
    ms_step = STEP_BYTES_PER_GPU / (v * 1e9) * 1e3 if v > 0 else None
    line = {
        "impl": "reference", "metric": "paged_kv_gather_append_GBps", "value": round(v, 3), "unit": "GB/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "u16/u8 moves, f32 quantisation",
        "data": "synthetic", "config": {"workload": WORKLOAD_NAME,
                                        "note": "each step is a bounded sample (2 of 43 layers); ms_per_step "
                                                "extrapolates the sample rate to the full step"},
        "cpu_baseline": {"value": round(v, 3), "unit": "GB/s", "cores": threads, "kind": "port",
                         "sample": wl.describe(sample_layers * len(times))},
        "e2e": {"value": round(v, 3), "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def run_ours(args):
    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device: the library has no CPU path (use --impl reference for the CPU arm)")
    torch.cuda.set_device(local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    wl = Workload(torch, args, rank)
    stream = torch.cuda.current_stream()
    sp = C.c_void_p(stream.cuda_stream)
    step_bytes = STEP_BYTES_PER_GPU

    # ---- device-resident timing: W warm-up steps, then exactly K steps between two events ----
    for _ in range(max(args.warmup, 3)):
        wl.run_step(sp)
    barrier()
    sampler = ClockSampler(local)
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record(stream)
    for _ in range(args.steps):
        wl.run_step(sp)
    e1.record(stream)
    barrier()
    ms = e0.elapsed_time(e1)
    clocks = sampler.stop()
    ok, why = wl.verify()

    # ---- end to end: the step's host inputs come from pinned memory, a sample of the result goes back ----
    e2e = None
    if not args.no_e2e:
        host = {k: getattr(wl, k).cpu().pin_memory() for k in ("rows", "keys", "idx", "tables", "chunks", "q_chunk", "q_visible")}
        sample = torch.empty_like(wl.out[LAYERS - 1, 0], device="cpu").pin_memory()
        h2d = sum(t.numel() * t.element_size() for t in host.values())
        d2h = sample.numel() * sample.element_size()

        def e2e_step():
            for k, t in host.items():
                getattr(wl, k).copy_(t, non_blocking=True)
            wl.run_step(sp)
            sample.copy_(wl.out[LAYERS - 1, 0], non_blocking=True)

        for _ in range(3):
            e2e_step()
        barrier()
        f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        f0.record(stream)
        for _ in range(args.steps):
            e2e_step()
        f1.record(stream)
        barrier()
        e2e_ms = f0.elapsed_time(f1)
        e2e = (e2e_ms, h2d, d2h)

    times = torch.tensor([ms, e2e[0] if e2e else 0.0], dtype=torch.float64, device="cuda")
    oks = torch.tensor([1 if ok else 0], dtype=torch.int32, device="cuda")
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
        dist.all_reduce(oks, op=dist.ReduceOp.MIN)
    ms_max, e2e_ms_max = float(times[0]), float(times[1])
    all_ok = bool(int(oks[0]))

    if rank == 0:
        peak, peak_kind = load_peaks()
        total_bytes = step_bytes * world * args.steps
        value = total_bytes / (ms_max * 1e-3) / 1e9
        per_gpu = value / world
        launches = wl.launches_per_step * args.steps
        # Dominant kernel = the per-layer gather. Its average duration is taken as the timed region divided by the
        # number of layer calls (an upper bound: it charges the small append kernel and launch gaps to it).
        calls = len(wl.groups) * args.steps
        call_bytes = step_bytes / len(wl.groups)
        achieved = call_bytes / (ms * 1e-3 / calls) / 1e9
        line = {
            "metric": "paged_kv_gather_append_GBps", "value": round(value, 1), "unit": "GB/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": round(ms_max / args.steps, 4),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "u16/u8 moves, f32 quantisation",
            "data": "synthetic",
            "config": {"workload": WORKLOAD_NAME if not args.small else "SMALL decode43 (8k context): not the benchmark configuration",
                       "gather_variant": args.variant, "layers_per_launch": wl.lpl, "resident_layer_pools": wl.resident,
                       "pool_GB_per_layer": round(wl.num_pages * (PAGE_BYTES + FP4_PAGE_BYTES) / 1e9, 2),
                       "l2": "inputs larger than L2 (pools %.0f GB, outputs %.1f GB per step)" % (
                           wl.resident * wl.num_pages * PAGE_BYTES / 1e9, LAYERS * NSEQ * K_SEL * ROW_BYTES / 1e9),
                       "step_GB_per_gpu": round(step_bytes / 1e9, 3)},
            "decode_step_us": round(ms_max / args.steps * 1e3, 1),
            "pct_of_8TBps_per_gpu": round(per_gpu / 8000 * 100, 2),
            "pct_of_measured_peak_per_gpu": round(per_gpu / peak * 100, 2),
            "bit_exact_check": {"ok": all_ok, "what": why},
            "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peak, "unit": "GB/s",
                         "frac": round(achieved / peak, 4),
                         "traffic": NCU_TRAFFIC_BYTES_PER_LAUNCH if (args.variant == "bulk" and wl.lpl == 1) else None,
                         "traffic_source": "profiles/gather_bulk_kernel_decode43_small.md (ncu dram__bytes_read+write, one launch)",
                         "peak_kind": "of " + peak_kind,
                         "kernel": "gather_bulk_kernel" if args.variant == "bulk" else "step_vec_kernel",
                         "algorithmic_bytes_per_launch": int(call_bytes)},
            "gpu_launches": launches, "clocks": clocks,
        }
        if e2e:
            line["e2e"] = {"value": round(total_bytes / (e2e_ms_max * 1e-3) / 1e9, 1), "unit": "GB/s",
                           "h2d_bytes_per_step": int(e2e[1]), "d2h_bytes_per_step": int(e2e[2]),
                           "note": "host rows, keys, index lists, block tables and chunk lists copied in from pinned "
                                   "memory every step; one sequence's gathered tile of the last layer copied back"}
        if world == 1 and not args.no_cpu_baseline:
            from oracle import oracle_lib as orc
            threads = max(1, orc.hardware_threads())
            gbs, desc = cpu_baseline(threads)
            line["cpu_baseline"] = {"value": round(gbs, 3), "unit": "GB/s", "cores": threads, "kind": "port", "sample": desc}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if not all_ok:
        sys.exit(3)


def main():
    args = parse_args()
    if args.impl == "reference":
        run_reference_arm(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
