#!/usr/bin/env python
"""Benchmark of the quantized-FC decode path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (the configuration the headline metric is quoted on): the Q4_1
group-128 decode GEMV sweep over the Llama-7B FC shapes
(K,N) in {(4096,4096), (4096,11008), (11008,4096), (4096,32000)} at
M in {1,2,4,8}.  One "step" = one pass over those 16 FC calls.  Every
(shape, M) pair has its own packed weight tensor (506 MB of distinct weights
per step, four times the L2), so no call finds its weights in cache.  Weights
~ N(0, 0.02), activations ~ N(0, 1), seeded, synthetic.

value  packed weight GB/s (packed bytes / time, 1 GB = 1e9 B: the reference's
       own "Bound: GB/s" figure of ops/perf_ops.py:243-245), inputs (fp32
       activations, packed weights) resident in HBM.  The 16 calls of a step
       are independent, so a step quantizes the 16 inputs (four launches of
       q4fc_quant_x_q8_batch) and runs the FCs as four launches of
       q4fc_fc_decode_batch (one per row count each), replayed as
       one CUDA graph.  The timed region runs every step `inner` times so that
       it lasts about half a second; ms_per_step is per single step.
roofline  the dominant kernel (fc_decode_ring_kernel) alone: a second timed
       pass over the same FC launches with the inputs already quantized;
       achieved = algorithmic bytes per launch / average launch duration.
       `in_order_single_calls` has the 16 calls as 16 single launches in
       order, and every (shape, M) by itself as ops/perf_ops.py:190-245
       measures it (rotating distinct weights).
e2e    the same sweep through host.HostFCBatch: host buffers in and out over
       one pinned block each way, copies pipelined with the launches, inside
       the timed region.

With --gpus N > 1 every FC weight is split along N over the ranks (strong
scaling: the job is the same sweep, each rank streams 1/N of every weight).
--tp fused (default): the FC kernel stores its columns, stamped with the
step number, into every rank's output buffer over NVLink.  The same sweep
joined by an NCCL all-gather after every FC is timed beside it (`tp_nccl`).

--impl reference times the reference's own CPU FC (compiled from its sources
into oracle/_ref when that was possible, else the C restatement in oracle/)
on all host cores, on the same sweep.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

SHAPES = [(4096, 4096), (4096, 11008), (11008, 4096), (4096, 32000)]  # (K, N)
MS = [1, 2, 4, 8]
QTYPE, GROUP_K = 1, 128
BS = 16 * GROUP_K + 128
# DRAM bytes per launch of the dominant kernel from one ncu capture of the four-launch step (profiles/), against
# the algorithmic bytes of those launches
DECODE_TRAFFIC_RATIO = 1.03
METRIC = "Q4_1 FC decode weight GB/s"
UNIT = "GB/s"
TIMED_REGION_S = 0.5


def packed_bytes(K: int, N: int) -> int:
    return ((N + 31) // 32) * ((K + GROUP_K - 1) // GROUP_K) * BS


def algorithmic_bytes(K: int, N: int, M: int) -> int:
    """Packed weights read once + fp32 activations in + fp32 outputs out."""
    return packed_bytes(K, N) + 4 * M * K + 4 * M * N


STEP_WEIGHT_BYTES = sum(packed_bytes(K, N) for K, N in SHAPES) * len(MS)
STEP_ALGO_BYTES = sum(algorithmic_bytes(K, N, M) for K, N in SHAPES for M in MS)
CONFIG = {
    "workload": "Q4_1 group-128 decode GEMV sweep, Llama-7B FC shapes (K,N)=(4096,4096),(4096,11008),"
                "(11008,4096),(4096,32000) x M=1,2,4,8; one step = 16 FC calls",
    "qtype": "q4_1", "group_k": GROUP_K,
    "cache": "every (shape, M) has its own packed weights: 506 MB distinct per step, inputs larger than L2",
    "weights": "N(0,0.02) seeded", "activations": "N(0,1) seeded",
}


def load_peaks() -> tuple[float, str]:
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(p) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


_emit = print  # replaced in main() by a writer bound to the real stdout


# --------------------------------------------------------------------- clocks
class ClockSampler:
    """Samples SM clock and throttle reasons through NVML while the timed region runs."""

    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}

    def __init__(self, index: int) -> None:
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml

            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM))
        except Exception:
            self.nv = None

    def _poll(self) -> None:
        nv = self.nv
        while not self._stop.is_set():
            try:
                self.samples.append(int(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)))
                try:
                    mask = int(nv.nvmlDeviceGetCurrentClocksEventReasons(self.h))
                except Exception:
                    mask = int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h))
                for bit, name in self.REASONS.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.004)

    def start(self) -> None:
        if self.nv is not None:
            self._thread = threading.Thread(target=self._poll, daemon=True)
            self._thread.start()

    def stop(self) -> dict:
        self._stop.set()
        if self._thread is not None:
            self._thread.join()
        s = sorted(self.samples)
        return {"sm_mhz": (s[len(s) // 2] if s else None), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(s),
                "note": "sampled by NVML every 4 ms inside the timed region"}


# ------------------------------------------------------------- reference arm
def host_cpu_info() -> tuple[str, int]:
    model = "unknown"
    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:
        n = os.cpu_count() or 1
    try:
        with open("/proc/cpuinfo") as f:
            for line in f:
                if line.startswith("model name"):
                    model = line.split(":", 1)[1].strip()
                    break
    except OSError:
        pass
    return model, n


def cpu_sweep_setup(shapes, ms):
    """Seeded inputs and packed weights for the CPU legs, packed by the CPU checker itself; the OpenMP team is set
    to the cores this process may run on (a launcher may have exported OMP_NUM_THREADS=1 for its children)."""
    import numpy as np

    from oracle import build_oracle, cpu

    build_oracle.build_restatement()
    use_ref = cpu.have_compiled_reference(QTYPE, GROUP_K)
    impl = cpu.compiled_reference(QTYPE, GROUP_K) if use_ref else None
    _, ncpu = host_cpu_info()
    rng = np.random.default_rng(0)
    work = []
    for K, N in shapes:
        W = (rng.standard_normal((N, K), dtype=np.float32) * np.float32(0.02))
        wq = cpu.restated.pack(W, QTYPE, GROUP_K)
        del W
        for M in ms:
            x = rng.standard_normal((1, M, K), dtype=np.float32)
            work.append((x, wq.copy(), N))  # a clone per M, as ops/perf_ops.py:234-236 rotates clones
    if use_ref:
        cores = impl.set_threads(ncpu)
        run = lambda x, wq, N: impl.fc(x, wq, N)  # noqa: E731
        kind = "reference"
    else:
        run = lambda x, wq, N: cpu.restated.fc(x, wq, N)  # noqa: E731
        kind, cores = "port", cpu.restated.threads()
    return work, run, kind, cores


def time_cpu_sweep(work, run, passes: int, warm: int) -> float:
    """Seconds per pass over the sweep (mean over `passes` timed passes)."""
    for _ in range(warm):
        for x, wq, N in work:
            run(x, wq, N)
    t0 = time.perf_counter()
    for _ in range(passes):
        for x, wq, N in work:
            run(x, wq, N)
    return (time.perf_counter() - t0) / passes


def reference_arm(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    work, run, kind, cores = cpu_sweep_setup(SHAPES, MS)
    warm = max(args.warmup, 3)
    # bound the run to about a minute of CPU work
    t_probe = time_cpu_sweep(work, run, 1, 1)
    warm = max(1, min(warm, int(10.0 / max(t_probe, 1e-6))))
    steps = max(1, min(args.steps, int(60.0 / max(t_probe, 1e-6))))
    sec = time_cpu_sweep(work, run, steps, warm)
    value = STEP_WEIGHT_BYTES / sec / 1e9
    model, ncpu = host_cpu_info()
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": steps,
        "warmup": warm, "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "int8xuint4->int32, fp32 scaling", "data": "synthetic", "config": CONFIG,
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": kind,
                         "sample": f"the whole 16-call sweep, {steps} timed passes; host CPU {model}, "
                                   f"{ncpu} usable logical CPUs, {cores} OpenMP threads"},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    _emit(json.dumps(line))


# ------------------------------------------------------------------- our arm
def our_arm(args) -> int:
    import torch
    import torch.distributed as dist

    import llama_cl_b200 as pkg
    from llama_cl_b200 import tp
    from llama_cl_b200.host import HostFCBatch
    from llama_cl_b200.stack import DecodeFCStack

    ops = pkg.llmops
    sections = set(args.sections.split(","))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device: the FC path has no CPU fallback")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    distributed = world > 1
    if distributed:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    pkg._cabi.lib()
    peak, peak_kind = load_peaks()
    warmup = max(args.warmup, 3)

    def barrier() -> None:
        if distributed:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms: float) -> float:
        if not distributed:
            return ms
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def capture(fn):
        """Two eager runs (kernel attributes, lazy look-ups), then one CUDA graph of fn."""
        for _ in range(2):
            fn()
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            fn()
        torch.cuda.synchronize()
        return g.replay

    def timed(run, n: int, warm: int = 3, sample_clocks: bool = False):
        """(ms per run, clocks) over n runs on the device, max over ranks; every rank makes the same n runs."""
        for _ in range(warm):
            run()
        sampler = ClockSampler(local_rank) if sample_clocks else None
        barrier()
        if sampler:
            sampler.start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            run()
        e1.record()
        barrier()
        clocks = sampler.stop() if sampler else None
        return max_over_ranks(e0.elapsed_time(e1)) / n, clocks

    # ---- how the ranks' column slices meet
    arena, tp_mode, tp_note = None, ("none" if not distributed else args.tp), None
    if distributed and tp_mode == "fused":
        try:
            arena = tp.TPArena(160 << 20, dev)
        except Exception as e:  # no peer mapping on this box: the collective-library form still works
            tp_note = f"peer-mapped arena unavailable ({e}); joined by NCCL all-gather instead"
            print(f"[bench] {tp_note}", file=sys.stderr)
            tp_mode = "nccl"
        flag = torch.tensor([1 if tp_mode == "fused" else 0], device=dev)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)  # all ranks take the same route
        if int(flag.item()) == 0 and tp_mode == "fused":
            tp_mode, tp_note = "nccl", "another rank could not map the arena; joined by NCCL all-gather instead"
    fused = tp_mode == "fused"
    status_words: dict = {}

    def section_status(name: str) -> None:
        """Reads and clears the status word of the peer-store path after a section: non-zero means a bounded wait on
        another rank ran out, and everything timed in that section is void."""
        if not fused:
            return
        st = arena.status()
        t = torch.tensor([st], device=dev, dtype=torch.int64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        status_words[name] = int(t.item())
        arena.tensor(arena.STATUS, (1,), torch.int32).zero_()
        torch.cuda.synchronize()

    # ---- inputs: one packed weight per (shape, M); with TP each rank packs only its rows
    gen = torch.Generator(device=dev)
    calls = []
    sweep_sched = tp.TPSchedule(arena) if fused else None
    for si, (K, N) in enumerate(SHAPES):
        for M in MS:
            gen.manual_seed(1000 * si + M)
            n0, n1 = tp.shard_rows(N, world, rank) if distributed else (0, N)
            W = torch.randn((N, K), generator=gen, device=dev, dtype=torch.float32) * 0.02
            wq = ops.offline_FC_quant_Q4A(W[n0:n1].contiguous(), qtype="q4_1", group_k=GROUP_K)
            del W
            x = torch.randn((1, M, K), generator=gen, device=dev, dtype=torch.float32)
            c = {"x": x, "wq": wq, "N": N, "n_local": n1 - n0, "M": M, "K": K}
            if fused:
                c["layer"] = tp.FusedTPLinearQ4(sweep_sched, wq, N, max_rows=8, pdl=True)
                c["xq"] = ops.QuantizedActivations(1, M, K, GROUP_K, False, dev)
                c["y_full"] = torch.empty((1, M, N), device=dev, dtype=torch.float32)
            elif distributed:
                c["layer"] = tp.TPLinearQ4(wq, N, pdl=True, path="decode")
            else:
                c["xq"] = ops.QuantizedActivations(1, M, K, GROUP_K, False, dev)
                c["y"] = torch.empty((1, M, N), device=dev, dtype=torch.float32)
            calls.append(c)
    torch.cuda.synchronize()
    per_rank_weight = sum(packed_bytes(c["K"], c["n_local"]) for c in calls)
    per_rank_algo = sum(packed_bytes(c["K"], c["n_local"]) + 4 * c["M"] * c["K"] + 4 * c["M"] * c["n_local"]
                        for c in calls)

    # ---- the step
    n_fc_launches = len(calls)
    if not distributed:
        # one launch per row count: calls of a launch then share the size of their code buffers
        groups = [[c for c in calls if c["M"] == M] for M in reversed(MS)]  # largest first: the step ends on the smallest launch
        batches = [ops.FCBatch([(c["xq"], c["wq"], c["N"], c["y"]) for c in g_], pdl=True) for g_ in groups]
        qbatches = [ops.QuantizeBatch([(c["x"], c["xq"]) for c in g_]) for g_ in groups]
        n_fc_launches = len(batches)
        side = torch.cuda.Stream(dev)

        def step_device() -> None:
            # the quantizers (one launch per group) run on a side branch of the graph: all but the first group's hide
            # behind the FCs of the group before
            cur = torch.cuda.current_stream(dev)
            start = torch.cuda.Event()
            start.record(cur)
            side.wait_event(start)
            done = []
            with torch.cuda.stream(side):
                for qb in qbatches:
                    qb.run()  # the group's four quantizers as one launch
                    ev = torch.cuda.Event()
                    ev.record(side)
                    done.append(ev)
            for b, ev in zip(batches, done):
                cur.wait_event(ev)
                b.run()

        def step_fc_only() -> None:
            for b in batches:
                b.run()

        launches_per_step = len(qbatches) + len(batches)
    elif fused:
        groups = [[c for c in calls if c["M"] == M] for M in reversed(MS)]  # largest first: the step ends on the smallest launch
        tbatches = [tp.FusedTPBatch([c["layer"] for c in g_], [c["xq"] for c in g_]) for g_ in groups]
        qbatches = [ops.QuantizeBatch([(c["x"], c["xq"]) for c in g_]) for g_ in groups]
        side = torch.cuda.Stream(dev)

        def step_device() -> None:
            # step barrier, the quantizers on a side branch group by group, one N-split launch per row count, and
            # ONE unpacking launch that waits for the other ranks' columns of all 16 outputs: the step ends when
            # every rank holds every full output
            cur = torch.cuda.current_stream(dev)
            start = torch.cuda.Event()
            start.record(cur)
            side.wait_event(start)
            done = []
            with torch.cuda.stream(side):
                for qb in qbatches:
                    qb.run()  # the group's four quantizers as one launch
                    ev = torch.cuda.Event()
                    ev.record(side)
                    done.append(ev)
            sweep_sched.step_begin()
            outs = []
            for b, ev in zip(tbatches, done):
                cur.wait_event(ev)
                outs += b.run()
            tp.collect_many(outs, [c["y_full"] for g_ in groups for c in g_])

        step_fc_only = step_device
        n_fc_launches = len(tbatches)
        launches_per_step = len(qbatches) + len(tbatches) + 2  # quantizers, N-split launches, step barrier, unpacking
    else:
        def step_device() -> None:
            for c in calls:
                c["layer"](c["x"])

        step_fc_only = step_device
        launches_per_step = len(calls)

    run_step = capture(step_device)
    # the timed region: args.steps steps, each replayed `inner` times so that the region lasts about half a second
    probe_ms, _ = timed(run_step, 20, warm=warmup)
    inner = max(1, int(round(args.region_s * 1e3 / max(probe_ms * args.steps, 1e-6))))
    if distributed:
        t = torch.tensor([inner], device=dev, dtype=torch.int64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)  # the same count on every rank: the step holds a cross-rank barrier
        inner = int(t.item())

    def run_steps() -> None:
        for _ in range(inner):
            run_step()

    ms_outer, clocks = timed(run_steps, args.steps, warm=1, sample_clocks=True)
    ms_step = ms_outer / inner
    value = STEP_WEIGHT_BYTES / (ms_step * 1e-3) / 1e9
    section_status("sweep")

    # ---- the dominant kernel alone: the FC launches of a step with their inputs already quantized
    if not distributed:
        run_fc = capture(step_fc_only)
        n_fc = max(20, min(2000, int(0.4 * args.region_s * 1e3 / max(probe_ms, 1e-3))))
        ms_fc, _ = timed(run_fc, n_fc)
    else:
        ms_fc = ms_step
    achieved = per_rank_algo / (ms_fc * 1e-3) / 1e9

    # ---- every (shape, M) as a single call in order, on rotating distinct weights (ops/perf_ops.py:190-245)
    per_call = None
    ms_in_order = None
    if not distributed and "percall" in sections:
        ws = ops.Workspace(int(pkg._cabi.lib().q4fc_fc_workspace_bytes(8, 11008, 32000, QTYPE, GROUP_K)), dev)
        per_call = {}
        for pdl in (False, True):
            def in_order() -> None:
                for c in calls:
                    ops.fc_Q4A(c["x"], c["wq"], c["N"], out=c["y"], workspace=ws, pdl=pdl, path="decode")
            ms, _ = timed(capture(in_order), 200)
            per_call["sweep_in_order_pdl_ms" if pdl else "sweep_in_order_plain_ms"] = ms
        ms_in_order = per_call["sweep_in_order_pdl_ms"]
        # every (shape, M) by itself: the same call repeated over enough distinct copies of the packed weights that
        # none is found in L2 (at least 300 MB in turn), one graph of programmatic launches in order
        table = {}
        for K, N in SHAPES:
            src = next(c for c in calls if c["K"] == K and c["N"] == N)
            ncopies = max(2, -(-300_000_000 // packed_bytes(K, N)))
            copies = [src["wq"]] + [src["wq"].clone() for _ in range(ncopies - 1)]
            row = {}
            for c in (c for c in calls if c["K"] == K and c["N"] == N):
                def one_shape(c=c) -> None:
                    for w in copies:
                        ops.fc_Q4A(c["x"], w, N, out=c["y"], workspace=ws, pdl=True, path="decode")
                ms, _ = timed(capture(one_shape), 20)
                us = ms * 1e3 / ncopies
                nb = algorithmic_bytes(K, N, c["M"])
                row[f"M{c['M']}"] = {"us": us, "gb_s": nb / (us * 1e-6) / 1e9, "frac": nb / (us * 1e-6) / 1e9 / peak}
            table[f"K{K}_N{N}"] = row
            del copies
        per_call["single_call_in_a_chain_of_its_own_kind"] = table

    # ---- end to end: host buffers in, host buffers out, one copy each way per step (public API)
    e2e = None
    if "e2e" in sections:
        if not distributed:
            hb = HostFCBatch([(c["wq"], c["N"], c["M"]) for c in calls])
            for i, c in enumerate(calls):
                hb.x_staging(i).copy_(c["x"].cpu())

            def step_e2e() -> None:
                hb(None, sync=True)

            h2d, d2h = hb.h2d_bytes(), hb.d2h_bytes()
        else:
            if fused:
                hbt = tp.HostFusedBatch(arena, [(c["wq"], c["N"], c["M"]) for c in calls])
                for i, c in enumerate(calls):
                    hbt.x_staging(i).copy_(c["x"].cpu())

                def step_e2e() -> None:
                    hbt(None, sync=True, check=False)  # the status word is read once after the section

                h2d, d2h = hbt.h2d_bytes(), hbt.d2h_bytes()
            else:
                xs_host = [c["x"].cpu().pin_memory() for c in calls]
                ys_host = [torch.empty((1, c["M"], c["N"]), dtype=torch.float32).pin_memory() for c in calls]

                def step_e2e() -> None:
                    for c, xh, yh in zip(calls, xs_host, ys_host):
                        c["x"].copy_(xh, non_blocking=True)
                        yh.copy_(c["layer"](c["x"]), non_blocking=True)
                    torch.cuda.current_stream(dev).synchronize()

                h2d = sum(4 * c["M"] * c["K"] for c in calls)
                d2h = sum(4 * c["M"] * c["N"] for c in calls)
        n_e2e = max(3, min(args.steps * inner, 300))
        for _ in range(3):
            step_e2e()
        barrier()
        wall0 = time.perf_counter()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        for _ in range(n_e2e):
            step_e2e()
        t1.record()
        barrier()
        wall = (time.perf_counter() - wall0) * 1e3
        ms_e2e = max_over_ranks(max(t0.elapsed_time(t1), wall)) / n_e2e  # the host waits for every result
        e2e = {"value": STEP_WEIGHT_BYTES / (ms_e2e * 1e-3) / 1e9, "unit": UNIT, "h2d_bytes_per_step": h2d,
               "d2h_bytes_per_step": d2h, "ms_per_step": ms_e2e, "steps": n_e2e,
               "api": "host.HostFCBatch: one pinned block each way; per FC launch (row count) one copy up and one down, pipelined with the kernels" if not distributed else
                      ("tp.HostFusedBatch: one pinned block each way; per N-split launch one copy up and one down, pipelined with the kernels, every rank" if fused
                       else "TPLinearQ4 with explicit copies")}
        section_status("e2e")

    # ---- per-token pass through the FC stack of a 32-layer Llama-7B (225 FCs, batch 1)
    stack = None
    if "stack" in sections:
        try:
            H, I, V, L = 4096, 11008, 32000, 32

            def shard_pack(N, K, seed):
                gen.manual_seed(seed)
                n0, n1 = tp.shard_rows(N, world, rank) if distributed else (0, N)
                Wf = torch.randn((N, K), generator=gen, device=dev, dtype=torch.float32) * 0.02
                w = ops.offline_FC_quant_Q4A(Wf[n0:n1].contiguous(), qtype="q4_1", group_k=GROUP_K)
                del Wf
                return w

            names = [("q", H, H), ("k", H, H), ("v", H, H), ("o", H, H), ("gate", I, H), ("up", I, H), ("down", H, I)]
            layers = [{nm: shard_pack(N_, K_, 50000 + li * 16 + j) for j, (nm, N_, K_) in enumerate(names)}
                      for li in range(L)]
            lm_head = shard_pack(V, H, 49999)
            full_bytes = sum(packed_bytes(K_, N_) for _, N_, K_ in names) * L + packed_bytes(H, V)
            gen.manual_seed(7)
            h0 = torch.randn((1, 1, H), generator=gen, device=dev, dtype=torch.float32)
            stack = {"packed_weight_bytes": full_bytes, "fc_calls": 7 * L + 1,
                     "what": "Q4_1 group-128 FC stack of a random-init 32-layer Llama-7B (hidden 4096, intermediate "
                             "11008, vocab 32000 lm_head), batch 1"}
            if not distributed:
                for glue, chain in (("none", False), ("llama", False), ("none", True), ("llama", True)):
                    st = DecodeFCStack(layers, lm_head, hidden=H, intermediate=I, vocab=V, rows=1, glue=glue, chain=chain)
                    st.forward(h0, sync=True)
                    n_tok = max(3, min(args.steps * inner, 100))
                    with torch.cuda.stream(st.stream):
                        for _ in range(3):
                            st.forward()
                        a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                        a0.record()
                        for _ in range(n_tok):
                            st.forward()
                        a1.record()
                    st.stream.synchronize()
                    ms_tok = a0.elapsed_time(a1) / n_tok
                    if chain:
                        # the same schedule as ONE persistent launch (q4fc_fc_chain_*): reported beside the graph of
                        # launches, whichever is faster
                        st.check()
                        stack.setdefault("one_persistent_launch", {})[
                            "ms_per_token" if glue == "none" else "ms_per_token_with_norms_and_mlp_glue"] = ms_tok
                        del st
                        continue
                    key = "ms_per_token" if glue == "none" else "ms_per_token_with_norms_and_mlp_glue"
                    stack[key] = ms_tok
                    stack["launches_per_token" if glue == "none" else "launches_per_token_with_glue"] = \
                        st.launches_per_token
                    if glue == "none":
                        stack["weight_gb_s"] = full_bytes / (ms_tok * 1e-3) / 1e9
                        stack["frac_of_hbm_peak"] = stack["weight_gb_s"] / peak
                    del st
                stack["launch"] = ("stack.DecodeFCStack: one CUDA graph per token; ms_per_token is the FC-only chain "
                                   "(q/k/v and gate/up one launch each), the second figure adds rmsnorm, residual adds "
                                   "and silu*up between the FCs")
            else:
                if fused:
                    from llama_cl_b200.stack import FusedTPDecodeFCStack

                    tst = FusedTPDecodeFCStack(arena, layers, lm_head, hidden=H, intermediate=I, vocab=V, rows=1)
                    tst.forward(h0, sync=True)

                    def run_tok() -> None:
                        # the stack replays on a stream of its own: tie it to the stream the timing events are on
                        cur = torch.cuda.current_stream(dev)
                        tst.stream.wait_stream(cur)
                        tst.forward()
                        cur.wait_stream(tst.stream)

                else:
                    def mk(w, N_):
                        return tp.TPLinearQ4(w, N_, pdl=True, path="decode")

                    lay = [{nm: mk(l[nm], N_) for nm, N_, _ in names} for l in layers]
                    head = mk(lm_head, V)

                    def run_tok() -> None:
                        # the seven FCs of chatllama/main.py:348-370 with their data dependences; the non-FC ops
                        # between them are not part of this path
                        h = h0
                        for f in lay:
                            q = f["q"](h)
                            f["k"](h)
                            f["v"](h)
                            o = f["o"](q)
                            g_ = f["gate"](o)
                            f["up"](o)
                            h = f["down"](g_)
                        head(h)

                ms_tok, _ = timed(run_tok, max(3, min(args.steps * inner, 60)))
                stack["ms_per_token"] = ms_tok
                stack["weight_gb_s"] = full_bytes / (ms_tok * 1e-3) / 1e9
                stack["launch"] = ("stack.FusedTPDecodeFCStack: cuda graph of one token (225 fused N-split FCs in 129 "
                                   "launches + step barrier + one unpacking launch)" if fused
                                   else "eager, NCCL all-gather per FC")
            del layers, lm_head
        except Exception as e:
            stack = {"error": str(e)}
        section_status("fc_stack")

    # ---- the NCCL all-gather join named by the task, timed beside the fused form (short pass)
    tp_nccl = None
    if distributed and fused and "nccl" in sections:
        try:
            lay = [tp.TPLinearQ4(c["wq"], c["N"], pdl=True, path="decode") for c in calls]

            def step_nccl() -> None:
                for c, l in zip(calls, lay):
                    l(c["x"])

            ms_n, _ = timed(step_nccl, 30)
            tp_nccl = {"ms_per_step": ms_n, "value": STEP_WEIGHT_BYTES / (ms_n * 1e-3) / 1e9, "unit": UNIT,
                       "what": "the same sweep with every FC's column slices joined by an NCCL all-gather (eager launches)"}
            # prefill under the N-split: M = 512, K = 4096, N = 11008, Q4_1 group 128, all-gather of [M, N/g] tiles
            gen.manual_seed(4243)
            Wp = torch.randn((11008, 4096), generator=gen, device=dev, dtype=torch.float32) * 0.02
            lp = tp.TPLinearQ4.from_full_weight(Wp, qtype="q4_1", group_k=GROUP_K)
            xp = torch.randn((1, 512, 4096), generator=gen, device=dev, dtype=torch.float32)
            ms_p, _ = timed(lambda: lp(xp), 10)
            tp_nccl["prefill_M512_K4096_N11008_ms"] = ms_p
            tp_nccl["prefill_M512_tops"] = 2.0 * 512 * 11008 * 4096 / (ms_p * 1e-3) / 1e12
            del Wp, lp
        except Exception as e:
            tp_nccl = {"error": str(e)}

    # ---- the other configurations of the path, reported beside the headline (single GPU only)
    extras = None
    if not distributed and "extras" in sections:
        try:
            extras = {}
            gen.manual_seed(4242)
            Wp = torch.randn((11008, 4096), generator=gen, device=dev, dtype=torch.float32) * 0.02

            def time_fn(fn, reps):
                fn()
                torch.cuda.synchronize()
                t0_, t1_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                t0_.record()
                for _ in range(reps):
                    fn()
                t1_.record()
                torch.cuda.synchronize()
                return t0_.elapsed_time(t1_) / reps

            # prefill: K=4096, N=11008, M=512 and 2048 (int8 tensor-core kernel + quantizer), Q4_0 g32 (the baseline's
            # configuration) and Q4_1 g128 (the format of the decode configurations)
            int8_peak_tops = 2.0 * 1641.8
            try:
                with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
                    int8_peak_tops = 2.0 * float(json.load(f)["bf16_tflops"])
            except Exception:
                pass
            for qname, G_ in (("q4_0", 32), ("q4_1", 128)):
                wq0 = ops.offline_FC_quant_Q4A(Wp, qtype=qname, group_k=G_)
                pre = {}
                for M_ in (512, 2048):
                    xp = torch.randn((1, M_, 4096), generator=gen, device=dev, dtype=torch.float32)
                    yp = torch.empty((1, M_, 11008), device=dev, dtype=torch.float32)
                    wsp = ops.fc_workspace(M_, 4096, 11008, 0 if qname == "q4_0" else 1, G_, dev)
                    ms_ = time_fn(lambda: ops.fc_Q4A(xp, wq0, 11008, out=yp, workspace=wsp), 10)
                    wsp.check()
                    tops = 2.0 * M_ * 11008 * 4096 / (ms_ * 1e-3) / 1e12
                    pre[f"M{M_}"] = {"ms": ms_, "tops": tops, "frac_of_int8_peak": tops / int8_peak_tops}
                pre["int8_peak_tops"] = int8_peak_tops
                pre["int8_peak_kind"] = "2 x the measured dense bf16 burst figure (no int8 figure is measured on this pool)"
                extras[f"prefill_{qname}_g{G_}_K4096_N11008"] = pre
            # packer over a whole Llama-7B FC weight set: 32 layers x {q, k, v, o: 4096x4096; gate, up: 11008x4096;
            # down: 4096x11008}, one matrix after the other (every fp32 matrix is 64-180 MB: nothing stays in L2)
            shapes_ = {(4096, 4096): 4 * 32, (11008, 4096): 2 * 32, (4096, 11008): 1 * 32}
            mats_ = {sh: torch.randn(sh, generator=gen, device=dev, dtype=torch.float32) * 0.02 for sh in shapes_}
            full = {}
            for G_ in (32, 128):
                outs_ = {sh: torch.empty(((sh[0] + 31) // 32, sh[1] // G_, 16 * G_ + 128), dtype=torch.int8, device=dev)
                         for sh in shapes_}

                def pack_all():
                    for sh, cnt in shapes_.items():
                        for _ in range(cnt):
                            ops.offline_FC_quant_Q4A(mats_[sh], qtype="q4_1", group_k=G_, out=outs_[sh])

                ms_ = time_fn(pack_all, 3)
                nbytes = sum(cnt * (mats_[sh].numel() * 4 + outs_[sh].numel()) for sh, cnt in shapes_.items())
                full[f"g{G_}"] = {"ms": ms_, "gb_s": nbytes / (ms_ * 1e-3) / 1e9,
                                  "weights": sum(cnt * mats_[sh].numel() for sh, cnt in shapes_.items()),
                                  "frac_of_hbm_peak": nbytes / (ms_ * 1e-3) / 1e9 / peak}
            extras["pack_q4_1_llama7b_fc_set_224_matrices"] = full
            del mats_
            # per-channel int8 weights of the reference's older extension (FC_evaluate_Q8C) and its quantized
            # embedding table: lm_head-sized FC at M = 1 and 8 (each call = quantizer + FC launch, six packed copies
            # of the weights in turn so that none stays in L2, replayed as one graph), packer, table look-up
            q8 = {}
            Wl = torch.randn((32000, 4096), generator=gen, device=dev, dtype=torch.float32) * 0.02
            packs_ = [ops.FC_quant_Q8C(Wl) for _ in range(6)]
            for M_ in (1, 8):
                xq_ = torch.randn((1, M_, 4096), generator=gen, device=dev, dtype=torch.float32)
                yq_ = torch.empty((1, M_, 32000), device=dev, dtype=torch.float32)
                st_ = torch.cuda.Stream(dev)
                with torch.cuda.stream(st_):
                    ops.FC_evaluate_Q8C(xq_, packs_[0][0], packs_[0][1], 32000, out=yq_)
                    st_.synchronize()
                    g_ = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(g_, stream=st_):
                        for wq_, ws_ in packs_:
                            ops.FC_evaluate_Q8C(xq_, wq_, ws_, 32000, out=yq_)
                    ms_ = time_fn(g_.replay, 20) / len(packs_)
                nb_ = 32000 * 4096 + 32000 * 4 + M_ * 4096 * 4 + M_ * 32000 * 4
                q8[f"fc_M{M_}_K4096_N32000"] = {"us_per_call": ms_ * 1e3, "gb_s": nb_ / (ms_ * 1e-3) / 1e9,
                                                "frac_of_hbm_peak": nb_ / (ms_ * 1e-3) / 1e9 / peak,
                                                "launches_per_call": 2}
            ms_ = time_fn(lambda: ops.FC_quant_Q8C(Wl), 5)
            nb_ = Wl.numel() * 5
            q8["pack_K4096_N32000"] = {"ms": ms_, "gb_s": nb_ / (ms_ * 1e-3) / 1e9, "launches_per_call": 2,
                                       "frac_of_hbm_peak": nb_ / (ms_ * 1e-3) / 1e9 / peak}
            ms_ = time_fn(lambda: ops.embedding_q8c_quant_w(Wl), 5)
            q8["embedding_quant_V32000_E4096"] = {"ms": ms_, "gb_s": nb_ / (ms_ * 1e-3) / 1e9,
                                                  "frac_of_hbm_peak": nb_ / (ms_ * 1e-3) / 1e9 / peak}
            codes_, scales_ = ops.embedding_q8c_quant_w(Wl)
            ids_ = torch.randint(0, 32000, (1, 2048), generator=gen, device=dev)
            oe_ = torch.empty((1, 2048, 4096), device=dev, dtype=torch.float32)
            ms_ = time_fn(lambda: ops.embedding_q8c(oe_, ids_, codes_, scales_), 20)
            q8["embedding_lookup_2048_ids_E4096"] = {"us": ms_ * 1e3, "gb_s": 2048 * 4096 * 5 / (ms_ * 1e-3) / 1e9}
            ops.check_device_status(dev)
            extras["q8c"] = q8
            del Wl, packs_, Wp
        except Exception as e:
            extras = {"error": str(e)}

    # ---- parity spot check of what was just timed (not timed itself)
    check = None
    y_tp = None
    if distributed:
        c = calls[0]
        if fused:
            step_device()
            torch.cuda.synchronize()
            y_tp = c["y_full"].reshape(c["M"], c["N"]).clone()
        else:
            y_tp = c["layer"](c["x"]).reshape(c["M"], c["N"]).clone()
        lo, hi = y_tp.clone(), y_tp.clone()
        dist.all_reduce(lo, op=dist.ReduceOp.MIN)
        dist.all_reduce(hi, op=dist.ReduceOp.MAX)
        ranks_agree = bool(torch.equal(lo, hi))
        section_status("spot_check")
    if rank == 0:
        import numpy as np

        from oracle import cpu

        if not distributed:
            run_step()
            torch.cuda.synchronize()
            check = True
            for c in (calls[0], calls[7], calls[15]):
                want = cpu.restated.fc(c["x"].cpu().numpy(), c["wq"].cpu().numpy(), c["N"])
                check = check and bool(np.allclose(c["y"].cpu().numpy(), want, rtol=1e-3, atol=1e-4))
        else:
            c = calls[0]
            n0, _ = tp.shard_rows(c["N"], world, rank)
            want = cpu.restated.fc(c["x"].cpu().numpy(), c["wq"].cpu().numpy(), c["n_local"])
            mine = y_tp[:, n0: n0 + c["n_local"]].cpu().numpy().reshape(want.shape)
            check = bool(np.allclose(mine, want, rtol=1e-3, atol=1e-4)) and ranks_agree

    bad_status = {k: v for k, v in status_words.items() if v != 0}
    if rank == 0:
        cpu_baseline = None
        if not distributed and "cpu" in sections:
            try:
                work, run, kind, cores = cpu_sweep_setup(SHAPES, MS)
                t_probe = time_cpu_sweep(work, run, 1, 1)
                passes = max(1, min(50, int(15.0 / max(t_probe, 1e-6))))
                sec = time_cpu_sweep(work, run, passes, 0)
                model, ncpu = host_cpu_info()
                cpu_baseline = {"value": STEP_WEIGHT_BYTES / sec / 1e9, "unit": UNIT, "cores": cores, "kind": kind,
                                "sample": f"the whole 16-call sweep, {passes} passes (~{sec * passes:.0f} s); "
                                          f"host CPU {model}, {ncpu} usable logical CPUs", "ms_per_step": sec * 1e3}
            except Exception as e:
                cpu_baseline = {"value": None, "unit": UNIT, "cores": 0, "kind": "port", "sample": f"failed: {e}"}
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": warmup, "ms_per_step": ms_step, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None,
            "dtype": "int8xuint4->int32, fp32 scaling", "data": "synthetic", "config": CONFIG,
            "launch": {
                "parallelism": (
                    "single GPU" if world == 1 else
                    f"N-split tp{world}, columns stored into every rank's buffer by the FC kernel (epoch-stamped "
                    f"64-bit words, NVLink peer stores)" if fused else f"N-split tp{world} + NCCL all-gather"),
                **({"tp_note": tp_note} if tp_note else {}),
                "step": ("cuda graph: 4 quantizer launches (q4fc_quant_x_q8_batch, one per row count) on a side branch + 4 launches of q4fc_fc_decode_batch "
                         "(one per row count)" if not distributed else
                         "cuda graph: step barrier, 4 quantizer launches (one per row count) on a side branch, 4 launches of "
                         "q4fc_fc_decode_tp_batch (one per row count), one unpacking launch" if fused else "eager"),
                "inner_repeats_per_step": inner, "timed_region_ms": ms_outer * args.steps},
            "clocks": clocks, "e2e": e2e, "gpu_launches": launches_per_step * args.steps * inner,
            "gpu_launches_per_step": launches_per_step,
            **({"tp_status": max(status_words.values()) if status_words else 0, "tp_status_sections": status_words}
               if fused else {}),
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak,
                         "traffic": (DECODE_TRAFFIC_RATIO * per_rank_algo / n_fc_launches) if not distributed else None,
                         "traffic_source": "ncu dram__bytes_read.sum + dram__bytes_write.sum of the step's FC launches "
                                           "(summary under profiles/), per launch",
                         "peak_kind": peak_kind, "kernel": "fc_decode_ring_kernel<128,1,false,ROWS,false,true> (ROWS = 1 for the one-row launch, 8 for the others)",
                         "algorithmic_bytes_per_step": per_rank_algo, "launches_per_step": n_fc_launches,
                         "algorithmic_bytes_per_launch": per_rank_algo / n_fc_launches,
                         "avg_launch_ms": ms_fc / n_fc_launches,
                         "timed_as": "the step's FC launches alone (inputs already quantized), replayed as a graph; "
                                     "average launch duration = pass time / launches",
                         **({"in_order_single_calls": {
                             "what": "the 16 calls as 16 single q4fc_fc_decode launches in order on one stream",
                             "frac_pdl": per_rank_algo / (ms_in_order * 1e-3) / 1e9 / peak,
                             "frac_plain": per_rank_algo / (per_call["sweep_in_order_plain_ms"] * 1e-3) / 1e9 / peak,
                             **per_call}} if per_call else {})},
            "cpu_baseline": cpu_baseline, "parity_spot_check": check, "fc_stack": stack,
            **({"tp_nccl": tp_nccl} if tp_nccl is not None else {}),
            "other_configs": extras,
        }
        _emit(json.dumps(line))
    rc = 0
    if bad_status or (rank == 0 and check is False):
        print(f"[bench] INVALID RUN: status words {bad_status}, parity spot check {check}", file=sys.stderr)
        rc = 1
    if distributed:
        # Captured graphs hold NCCL work; tearing the process group down under them has been seen to
        # block.  Every collective of this run is behind us: drain the GPU and leave without the
        # interpreter's teardown.
        torch.cuda.synchronize()
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(rc)
    return rc


def main() -> None:
    # The checker libraries (the compiled reference prints a banner per thread pool) and any
    # library chatter must not reach stdout: the one JSON line goes to the real stdout, the
    # rest of the process writes to stderr.
    real_stdout = os.fdopen(os.dup(1), "w")
    os.dup2(2, 1)
    global _emit
    _emit = lambda line: (real_stdout.write(line + "\n"), real_stdout.flush())  # noqa: E731
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--tp", default="fused", choices=["fused", "nccl"],
                    help="with --gpus N > 1: how the ranks' output columns meet")
    ap.add_argument("--region-s", type=float, default=TIMED_REGION_S,
                    help="length of the timed region in seconds: every step is replayed as often as it takes "
                         "(a profiler run asks for 0: every step once)")
    ap.add_argument("--sections", default="e2e,stack,extras,cpu,percall,nccl",
                    help="optional legs beside the timed sweep (a profiler run asks for none of them: --sections none)")
    args = ap.parse_args()
    if args.impl == "reference":
        # a launcher may have exported OMP_NUM_THREADS=1 for its children: the reference arm uses every core it may
        os.environ.pop("OMP_NUM_THREADS", None)
        reference_arm(args)
        sys.exit(0)
    sys.exit(our_arm(args))


if __name__ == "__main__":
    main()
