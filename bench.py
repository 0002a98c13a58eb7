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
       own "Bound: GB/s" figure of ops/perf_ops.py:243-245), inputs resident
       in HBM, the 16 calls of a step replayed as one CUDA graph.  The calls
       are independent, so the graph runs them on --lanes parallel branches
       (default 4); the roofline figure is taken from a second timed pass with
       the same launches strictly one after the other.
e2e    the same metric through the host-buffer API (HostFC / HostFCGroup):
       activations copied from pinned host memory, results copied back to
       pinned host memory, every call, the step's calls submitted together.

With --gpus N > 1 every FC weight is split along N over the ranks (strong
scaling: the job is the same sweep, each rank streams 1/N of every weight).
--tp fused (default): the FC kernel stores its columns, stamped with the
step number, into every rank's output buffer over NVLink; consumers wait
word by word for the current stamp.
--tp nccl: the slices are joined by an NCCL all-gather after every FC.

--impl reference times the reference's own CPU FC (compiled from its sources
into oracle/_ref when that was possible, else the C restatement in oracle/)
on the host cores, on the same sweep.
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
# DRAM bytes per decode launch of this sweep from one ncu capture (3,561,665,024 B over 113 launches), against
# 31.89 MB of algorithmic bytes per launch
DECODE_TRAFFIC_PER_LAUNCH = 31.52e6
METRIC = "Q4_1 FC decode weight GB/s"
UNIT = "GB/s"


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
                "reasons": sorted(self.reasons), "samples": len(s)}


# ------------------------------------------------------------- reference arm
def host_cpu_info() -> tuple[str, int]:
    model, n = "unknown", os.cpu_count() or 1
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
    """Seeded inputs and packed weights for the CPU legs, packed by the CPU checker itself."""
    import numpy as np

    from oracle import build_oracle, cpu

    build_oracle.build_restatement()
    use_ref = cpu.have_compiled_reference(QTYPE, GROUP_K)
    impl = cpu.compiled_reference(QTYPE, GROUP_K) if use_ref else None
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
        run = lambda x, wq, N: impl.fc(x, wq, N)  # noqa: E731
        kind, cores = "reference", impl.threads()
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
    warm = max(1, min(args.warmup, 3))
    # bound the run to about a minute of CPU work
    t_probe = time_cpu_sweep(work, run, 1, 1)
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
                                   f"{ncpu} logical CPUs, {cores} OpenMP threads"},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    _emit(json.dumps(line))


# ------------------------------------------------------------------- our arm
def our_arm(args) -> None:
    import torch
    import torch.distributed as dist

    import llama_cl_b200 as pkg
    from llama_cl_b200 import tp
    from llama_cl_b200.host import HostFC

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

    # ---- how the ranks' column slices meet
    arena, tp_mode, tp_note = None, ("none" if not distributed else args.tp), None
    if distributed and tp_mode == "fused":
        try:
            arena = tp.TPArena(128 << 20, dev)
        except Exception as e:  # no peer mapping on this box: the collective-library form still works
            tp_note = f"peer-mapped arena unavailable ({e}); joined by NCCL all-gather instead"
            print(f"[bench] {tp_note}", file=sys.stderr)
            tp_mode = "nccl"
        flag = torch.tensor([1 if tp_mode == "fused" else 0], device=dev)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)  # all ranks take the same route
        if int(flag.item()) == 0 and tp_mode == "fused":
            tp_mode, tp_note = "nccl", "another rank could not map the arena; joined by NCCL all-gather instead"
    fused = tp_mode == "fused"
    # a schedule is a set of FCs that always run together: the sweep is one, the token pass another,
    # and each call of the host-buffer leg stands alone
    sweep_sched = tp.TPSchedule(arena) if fused else None

    def make_layer(sched, wq_, N_, max_rows=8, prequant=False):
        if fused:
            return tp.FusedTPLinearQ4(sched, wq_, N_, max_rows=max_rows, pdl=True, prequant=prequant)
        return tp.TPLinearQ4(wq_, N_, pdl=True, workspace=ws, path="decode")

    # ---- inputs: one packed weight per (shape, M); with TP each rank packs only its rows
    ws = pkg.llmops.fc_workspace(8, 11008, 32000, QTYPE, GROUP_K, dev)
    gen = torch.Generator(device=dev)
    calls = []
    for si, (K, N) in enumerate(SHAPES):
        for M in MS:
            gen.manual_seed(1000 * si + M)
            n0, n1 = tp.shard_rows(N, world, rank) if distributed else (0, N)
            W = torch.randn((N, K), generator=gen, device=dev, dtype=torch.float32) * 0.02
            wq = pkg.llmops.offline_FC_quant_Q4A(W[n0:n1].contiguous(), qtype="q4_1", group_k=GROUP_K)
            del W
            x = torch.randn((1, M, K), generator=gen, device=dev, dtype=torch.float32)
            layer = make_layer(sweep_sched, wq, N, prequant=args.lanes > 1) if distributed else None
            calls.append({"x": x, "wq": wq, "N": N, "n_local": n1 - n0, "M": M, "K": K, "layer": layer,
                          "y_full": torch.empty((1, M, N), device=dev, dtype=torch.float32) if fused else None,
                          "y": torch.empty((1, M, n1 - n0), device=dev, dtype=torch.float32)})
    torch.cuda.synchronize()

    # The 16 calls of a step are independent of one another, so a step may run them side by side: they are
    # dealt over `lanes` streams (longest first, each to the least loaded lane) that become parallel
    # branches of the step's CUDA graph.  While one call is in its short latency-bound phases (activation
    # quantization, the cluster reduction) the others keep HBM busy.  lanes = 1 is the plain one-after-the-
    # other order, timed as well: the per-launch roofline figure comes from that pass.
    n_lanes = 1 if tp_mode == "nccl" else max(1, args.lanes)  # one communicator: its collectives stay in order
    lane_streams = [torch.cuda.Stream(dev) for _ in range(n_lanes)]
    # calls that may overlap on the GPU need separate workspaces
    lane_ws = [pkg.llmops.Workspace(ws.nbytes, dev) for _ in range(n_lanes)]

    def deal(n: int):
        load, plan = [0.0] * n, [[] for _ in range(n)]
        for c in sorted(calls, key=lambda c: -packed_bytes(c["K"], c["n_local"])):
            i = load.index(min(load))
            plan[i].append(c)
            load[i] += packed_bytes(c["K"], c["n_local"]) / 5e12 + 4e-6 * (1 + c["M"] / 8)
        return plan

    def run_calls(cs, pdl: bool = True, wsp=None, side_by_side: bool = False) -> None:
        outs = []
        wsp = ws if wsp is None else wsp
        for c in cs:
            if fused:
                outs.append((c, c["layer"](c["x"])))
            elif distributed:
                c["layer"](c["x"])
            else:
                pkg.llmops.fc_Q4A(c["x"], c["wq"], c["N"], out=c["y"], workspace=wsp, pdl=pdl, path="decode",
                                  prequant=side_by_side)
        # fused: unpack to plain fp32 behind the lane's FCs (each unpacking kernel waits for the other ranks'
        # columns), so that the step ends when every rank holds every full output
        for c, o in outs:
            o.tensor(out=c["y_full"])

    def step_device(lanes: int = n_lanes) -> None:
        cur = torch.cuda.current_stream(dev)
        if fused:
            sweep_sched.step_begin()
        if lanes == 1:
            # plain launches, each after the one before has finished: nothing of one launch hides in another
            run_calls(calls, pdl=distributed or n_lanes == 1)
            return
        start = torch.cuda.Event()
        start.record(cur)
        for st, cs, wsp in zip(lane_streams, deal(lanes), lane_ws):
            st.wait_event(start)
            with torch.cuda.stream(st):
                run_calls(cs, wsp=wsp, side_by_side=True)
        for st in lane_streams[:lanes]:
            cur.wait_stream(st)

    def capture(fn):
        """Two eager runs (kernel attributes, TP buffers), then one CUDA graph of fn; fn itself if capture fails."""
        for _ in range(2):
            fn()
        torch.cuda.synchronize()
        try:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                fn()
            torch.cuda.synchronize()
            return g.replay, True
        except Exception as e:  # capture is an optimisation; eager launches still measure the same kernels
            print(f"[bench] CUDA graph capture failed, timing eager launches: {e}", file=sys.stderr)
            torch.cuda.synchronize()
            return fn, False

    run_step, graphed = capture(step_device)

    def barrier() -> None:
        if distributed:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        run_step()
    sampler = ClockSampler(local_rank)
    barrier()
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        run_step()
    e1.record()
    barrier()
    clocks = sampler.stop()
    if clocks["samples"] < 5:
        # the timed region was shorter than a few NVML polls: keep replaying the same graph (untimed)
        # for about a second and sample the clocks under that identical load
        sampler = ClockSampler(local_rank)
        sampler.start()
        t_end = time.perf_counter() + 1.0
        while time.perf_counter() < t_end:
            for _ in range(50):
                run_step()
            torch.cuda.synchronize()
        more = sampler.stop()
        more["note"] = "sampled during an untimed one-second replay of the timed graph (timed region too short to poll)"
        clocks = more
    ms_total = e0.elapsed_time(e1)
    if distributed:
        t = torch.tensor([ms_total], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_total = float(t.item())
    ms_step = ms_total / args.steps
    value = STEP_WEIGHT_BYTES / (ms_step * 1e-3) / 1e9

    # ---- the same 16 launches one after the other on one stream: the per-launch figure of the roofline
    ms_serial, serial_graphed = ms_step, graphed
    if n_lanes > 1:
        run_serial, serial_graphed = capture(lambda: step_device(1))
        n_serial = max(3, min(args.steps, 500))
        for _ in range(3):
            run_serial()
        barrier()
        s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s0.record()
        for _ in range(n_serial):
            run_serial()
        s1.record()
        barrier()
        ms_serial = s0.elapsed_time(s1)
        if distributed:
            t = torch.tensor([ms_serial], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms_serial = float(t.item())
        ms_serial /= n_serial

    # ---- end to end: host buffers in, host buffers out, every call (eager, public API)
    e2e = None
    if "e2e" in sections:
        hosts = []
        for c in calls:
            if fused:
                hosts.append(tp.HostFusedFC(arena, c["wq"], c["N"], max_rows=8, pdl=True, prequant=n_lanes > 1,
                                            stream=lane_streams[len(hosts) % n_lanes]))
            elif distributed:
                hosts.append(None)
            else:
                hosts.append(HostFC(c["wq"], c["N"], max_rows=8, workspace=lane_ws[len(hosts) % n_lanes],
                                    path="decode", prequant=n_lanes > 1, stream=lane_streams[len(hosts) % n_lanes]))
        # the activations sit in the pinned input buffer of the call's host front end
        xs_host = [c["x"].cpu().pin_memory() if h is None else h.x_staging(c["M"]).copy_(c["x"].cpu())
                   for c, h in zip(calls, hosts)]
        ys_host = [torch.empty((1, c["M"], c["N"]), dtype=torch.float32).pin_memory() for c in calls]

        from llama_cl_b200.host import HostFCGroup

        group = HostFCGroup(hosts) if all(h is not None for h in hosts) else None

        def step_e2e() -> None:
            if group is not None:
                # the step's 16 calls as one submission: copies in, kernels, copies out on the lanes' streams
                group(xs_host, sync=True)
                return
            for c, xh, yh in zip(calls, xs_host, ys_host):  # NCCL form: eager, call by call
                c["x"].copy_(xh, non_blocking=True)
                y = c["layer"](c["x"])
                yh.copy_(y, non_blocking=True)
            torch.cuda.current_stream(dev).synchronize()

        n_e2e = max(3, min(args.steps, 200))
        for _ in range(3):
            step_e2e()
        barrier()
        t0 = torch.cuda.Event(enable_timing=True)
        t1 = torch.cuda.Event(enable_timing=True)
        wall0 = time.perf_counter()
        t0.record()
        for _ in range(n_e2e):
            step_e2e()
        t1.record()
        barrier()
        wall = (time.perf_counter() - wall0) * 1e3
        ms_e2e = max(t0.elapsed_time(t1), 0.0)
        if distributed:
            t = torch.tensor([ms_e2e], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms_e2e = float(t.item())
        e2e = {"value": STEP_WEIGHT_BYTES / (ms_e2e / n_e2e * 1e-3) / 1e9, "unit": UNIT,
               "h2d_bytes_per_step": sum(4 * c["M"] * c["K"] for c in calls),
               "d2h_bytes_per_step": sum(4 * c["M"] * c["N"] for c in calls),
               "ms_per_step": ms_e2e / n_e2e, "steps": n_e2e, "wall_ms_per_step": wall / n_e2e}

    # ---- per-token pass through the FC stack of a 32-layer Llama-7B (225 FCs, batch 1)
    stack = None
    try:
        if "stack" not in sections:
            raise RuntimeError("section not requested")
        H, I, V, L = 4096, 11008, 32000, 32

        def make_fc(N, K, seed):
            """-> (fn(x) -> y, packed bytes on this rank)"""
            gen.manual_seed(seed)
            n0, n1 = tp.shard_rows(N, world, rank) if distributed else (0, N)
            Wf = torch.randn((N, K), generator=gen, device=dev, dtype=torch.float32) * 0.02
            wq_ = pkg.llmops.offline_FC_quant_Q4A(Wf[n0:n1].contiguous(), qtype="q4_1", group_k=GROUP_K)
            del Wf
            if fused:
                return make_layer(tok_sched, wq_, N, max_rows=1), wq_.numel()
            if distributed:
                return make_layer(None, wq_, N), wq_.numel()
            return _LocalFC(wq_, N), wq_.numel()

        ws_of_stream: dict = {}

        class _LocalFC:
            """One FC of the stack on this GPU: on fp32 activations, or on activations quantized beforehand."""

            def __init__(self, wq_, N_):
                self.wq, self.N = wq_, N_
                self.out = torch.empty((1, 1, N_), device=dev, dtype=torch.float32)

            def __call__(self, x_):
                return pkg.llmops.fc_Q4A(x_, self.wq, self.N, out=self.out, workspace=stream_ws(), pdl=True,
                                         path="decode")

            def q8(self, xq_):
                return pkg.llmops.fc_Q4A_q8(xq_, self.wq, self.N, out=self.out, pdl=True)

        def stream_ws():
            """One workspace per stream: FCs running side by side must not share scratch."""
            key = torch.cuda.current_stream(dev).cuda_stream
            if key not in ws_of_stream:
                ws_of_stream[key] = pkg.llmops.Workspace(ws.nbytes, dev)
            return ws_of_stream[key]

        tok_sched = tp.TPSchedule(arena) if fused else None
        layers, stack_bytes_rank = [], 0
        for li in range(L):
            fcs = {}
            for j, (name, N_, K_) in enumerate([("q", H, H), ("k", H, H), ("v", H, H), ("o", H, H),
                                                ("gate", I, H), ("up", I, H), ("down", H, I)]):
                fcs[name], nb = make_fc(N_, K_, 50000 + li * 16 + j)
                stack_bytes_rank += nb
            layers.append(fcs)
        lm_head, nb = make_fc(V, H, 49999)
        logits = torch.empty((1, 1, V), device=dev, dtype=torch.float32)
        stack_bytes_rank += nb
        gen.manual_seed(7)
        h0 = torch.randn((1, 1, H), generator=gen, device=dev, dtype=torch.float32)

        side = [torch.cuda.Stream(dev), torch.cuda.Stream(dev)]

        def fork(fns, x_):
            """Run independent FCs of one input side by side: the first on the current stream, the rest on side
            streams (they become parallel branches of the captured graph); returns their outputs after the join."""
            cur = torch.cuda.current_stream(dev)
            start = torch.cuda.Event()
            start.record(cur)
            outs = [None] * len(fns)
            for i_, f_ in enumerate(fns[1:]):
                with torch.cuda.stream(side[i_]):
                    side[i_].wait_event(start)
                    outs[i_ + 1] = f_(x_)
            outs[0] = fns[0](x_)
            for i_ in range(len(fns) - 1):
                cur.wait_stream(side[i_])
            return outs

        def token() -> None:
            # the seven FCs of chatllama/main.py:348-370 with their data dependences: q, k, v read the same
            # input, as do gate and up; the non-FC ops between them are not part of this path
            h = h0
            if fused:
                tok_sched.step_begin()
            for f in layers:
                q, _, _ = fork([f["q"], f["k"], f["v"]], h)
                o = f["o"](q)
                g_, _ = fork([f["gate"], f["up"]], o)
                h = f["down"](g_)
            y = lm_head(h)
            if fused:
                y.tensor(out=logits)  # the token is done when every rank holds the whole logits row

        def time_token(fn):
            run, graphed_ = capture(fn)
            n_ = max(3, min(args.steps, 100))
            for _ in range(3):
                run()
            barrier()
            a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a0.record()
            for _ in range(n_):
                run()
            a1.record()
            barrier()
            return a0.elapsed_time(a1), n_, graphed_

        ms_tok, n_tok, tok_graphed = time_token(token)
        if distributed:
            t = torch.tensor([ms_tok], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms_tok = float(t.item())
        ms_tok /= n_tok
        full_bytes = sum(packed_bytes(K_, N_) for N_, K_ in
                         [(H, H)] * 4 + [(I, H)] * 2 + [(H, I)]) * L + packed_bytes(H, V)
        stack = {"ms_per_token": ms_tok, "weight_gb_s": full_bytes / (ms_tok * 1e-3) / 1e9,
                 "packed_weight_bytes": full_bytes, "fc_calls": 7 * L + 1, "tokens_timed": n_tok,
                 "launch": "cuda graph of one token" if tok_graphed else "eager",
                 "what": "Q4_1 group-128 FC stack of a random-init 32-layer Llama-7B (hidden 4096, intermediate "
                         "11008, vocab 32000 lm_head), batch 1; FC kernels only"}
        if not distributed:
            # the same pass with every shared input quantized once (q/k/v read one quantized copy, gate/up
            # another) instead of once per FC as the reference does
            xq_a = pkg.llmops.QuantizedActivations(1, 1, H, GROUP_K, False, dev)
            xq_b = pkg.llmops.QuantizedActivations(1, 1, H, GROUP_K, False, dev)

            def token_quantize_once() -> None:
                h = h0
                for f in layers:
                    xa = pkg.llmops.quantize_activations(h, GROUP_K, pdl=True, out=xq_a)
                    q, _, _ = fork([f["q"].q8, f["k"].q8, f["v"].q8], xa)
                    o = f["o"](q)
                    xb = pkg.llmops.quantize_activations(o, GROUP_K, pdl=True, out=xq_b)
                    g_, _ = fork([f["gate"].q8, f["up"].q8], xb)
                    h = f["down"](g_)
                lm_head(h)

            ms_once, n_once, _ = time_token(token_quantize_once)
            stack["ms_per_token_quantize_once"] = ms_once / n_once
        del layers, lm_head
    except Exception as e:
        stack = {"error": str(e)}

    # ---- the other configurations of the path, reported beside the headline (single GPU only)
    extras = None
    if not distributed and "extras" in sections:
        try:
            extras = {}
            gen.manual_seed(4242)
            Wp = torch.randn((11008, 4096), generator=gen, device=dev, dtype=torch.float32) * 0.02

            def timed(fn, reps):
                fn()
                torch.cuda.synchronize()
                t0_, t1_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                t0_.record()
                for _ in range(reps):
                    fn()
                t1_.record()
                torch.cuda.synchronize()
                return t0_.elapsed_time(t1_) / reps

            # prefill: Q4_0 group 32, K=4096, N=11008, M=512 and 2048 (int8 tensor-core kernel + quantizer)
            wq0 = pkg.llmops.offline_FC_quant_Q4A(Wp, qtype="q4_0", group_k=32)
            pre = {}
            for M_ in (512, 2048):
                xp = torch.randn((1, M_, 4096), generator=gen, device=dev, dtype=torch.float32)
                yp = torch.empty((1, M_, 11008), device=dev, dtype=torch.float32)
                wsp = pkg.llmops.fc_workspace(M_, 4096, 11008, 0, 32, dev)
                ms_ = timed(lambda: pkg.llmops.fc_Q4A(xp, wq0, 11008, out=yp, workspace=wsp), 10)
                wsp.check()
                pre[f"M{M_}"] = {"ms": ms_, "tops": 2.0 * M_ * 11008 * 4096 / (ms_ * 1e-3) / 1e12}
            extras["prefill_q4_0_g32_K4096_N11008"] = pre
            # packer: fp32 -> Q4_1, one 11008x4096 matrix (algorithmic bytes = 4 B read + packed bytes written per weight)
            pk = {}
            for G_ in (32, 128):
                outp = torch.empty(((11008 + 31) // 32, 4096 // G_, 16 * G_ + 128), dtype=torch.int8, device=dev)
                ms_ = timed(lambda: pkg.llmops.offline_FC_quant_Q4A(Wp, qtype="q4_1", group_k=G_, out=outp), 20)
                nbytes = Wp.numel() * 4 + outp.numel()
                pk[f"g{G_}"] = {"ms": ms_, "gb_s": nbytes / (ms_ * 1e-3) / 1e9, "frac_of_hbm_peak": nbytes / (ms_ * 1e-3) / 1e9 / load_peaks()[0]}
            extras["pack_q4_1_11008x4096"] = pk
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
                            pkg.llmops.offline_FC_quant_Q4A(mats_[sh], qtype="q4_1", group_k=G_, out=outs_[sh])

                ms_ = timed(pack_all, 3)
                nbytes = sum(cnt * (mats_[sh].numel() * 4 + outs_[sh].numel()) for sh, cnt in shapes_.items())
                full[f"g{G_}"] = {"ms": ms_, "gb_s": nbytes / (ms_ * 1e-3) / 1e9, "weights": sum(
                    cnt * mats_[sh].numel() for sh, cnt in shapes_.items()),
                    "frac_of_hbm_peak": nbytes / (ms_ * 1e-3) / 1e9 / load_peaks()[0]}
            extras["pack_q4_1_llama7b_fc_set_224_matrices"] = full
            del mats_
            del Wp
        except Exception as e:
            extras = {"error": str(e)}

    # ---- parity spot check of what was just timed (not timed itself)
    check = None
    y_tp = None
    if distributed:
        # one more untimed step; every rank must now hold the same full output of the first call
        c = calls[0]
        if fused:
            step_device()
            y_tp = c["y_full"].reshape(c["M"], c["N"]).clone()
        else:
            y_tp = c["layer"](c["x"]).reshape(c["M"], c["N"]).clone()
        lo, hi = y_tp.clone(), y_tp.clone()
        dist.all_reduce(lo, op=dist.ReduceOp.MIN)
        dist.all_reduce(hi, op=dist.ReduceOp.MAX)
        ranks_agree = bool(torch.equal(lo, hi))
    if rank == 0:
        import numpy as np

        from oracle import cpu

        c = calls[0]
        if not distributed:
            y = pkg.llmops.fc_Q4A(c["x"], c["wq"], c["N"], workspace=ws).cpu().numpy()
            want = cpu.restated.fc(c["x"].cpu().numpy(), c["wq"].cpu().numpy(), c["N"])
            check = bool(np.allclose(y, want, rtol=1e-3, atol=1e-4))
        else:
            # this rank's own columns against the CPU restatement of its shard, and all ranks bit-equal
            want = cpu.restated.fc(c["x"].cpu().numpy(), c["wq"].cpu().numpy(), c["n_local"])
            mine = y_tp[:, : c["n_local"]].cpu().numpy().reshape(want.shape)
            check = bool(np.allclose(mine, want, rtol=1e-3, atol=1e-4)) and ranks_agree

    tp_status = arena.status() if fused else 0  # non-zero: a bounded wait on another rank ran out
    # this library's kernels per timed step: the FC kernel of every call, plus -- side by side on one GPU --
    # the quantizing launch in front of each, or -- N-split -- the step barrier and one unpacking kernel per call
    if fused:
        launches_per_step = (3 if n_lanes > 1 else 2) * len(calls) + 1
    elif distributed:
        launches_per_step = len(calls)
    elif n_lanes > 1:
        launches_per_step = 2 * len(calls)
    else:
        launches_per_step = len(calls) + sum(1 for c in calls if c["M"] * c["K"] >= 40 * 1024)
    if rank == 0:
        peak, peak_kind = load_peaks()
        # per launch: the step's algorithmic bytes and time divided by its 16 launches
        per_rank_algo = sum(packed_bytes(c["K"], c["n_local"]) + 4 * c["M"] * c["K"] + 4 * c["M"] * c["n_local"]
                            for c in calls)
        achieved = per_rank_algo / (ms_serial * 1e-3) / 1e9
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
                                          f"host CPU {model}, {ncpu} logical CPUs", "ms_per_step": sec * 1e3}
            except Exception as e:
                cpu_baseline = {"value": None, "unit": UNIT, "cores": 0, "kind": "port", "sample": f"failed: {e}"}
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None,
            "dtype": "int8xuint4->int32, fp32 scaling", "data": "synthetic",
            "config": dict(CONFIG, parallelism=(
                "single GPU" if world == 1 else
                f"N-split tp{world}, columns stored into every rank's buffer by the FC kernel (epoch-stamped 64-bit "
                f"words, NVLink peer stores)" if fused else f"N-split tp{world} + NCCL all-gather"),
                           **({"tp_note": tp_note} if tp_note else {}),
                           launch=(f"cuda graph of one step, the 16 independent calls on {n_lanes} parallel branches"
                                   if graphed else "eager"),
                           lanes=n_lanes),
            "clocks": clocks, "e2e": e2e, "gpu_launches": launches_per_step * args.steps, "gpu_launches_per_step": launches_per_step,
            **({"tp_status": tp_status} if fused else {}),
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak, "traffic": DECODE_TRAFFIC_PER_LAUNCH if not distributed else None,
                         "traffic_source": "ncu dram__bytes_read.sum + dram__bytes_write.sum, average over the decode "
                                           "launches of this sweep (launch-list summary under profiles/)",
                         "peak_kind": peak_kind,
                         "kernel": "fc_decode_cluster_kernel<128,1,false,ROWS>",
                         "algorithmic_bytes_per_step": per_rank_algo, "launches_per_step": len(calls),
                         "timed_as": "the 16 launches one after the other on one stream, plain stream order (a "
                                     "second timed pass); average launch duration = pass time / 16",
                         "ms_per_step_serial": ms_serial,
                         "value_serial": STEP_WEIGHT_BYTES / (ms_serial * 1e-3) / 1e9},
            "cpu_baseline": cpu_baseline, "parity_spot_check": check, "fc_stack": stack, "other_configs": extras,
        }
        _emit(json.dumps(line))
    if distributed:
        # Captured graphs hold NCCL work; tearing the process group down under them has been seen to
        # block.  Every collective of this run is behind us (the last one was the all-reduce of the
        # timings): drain the GPU and leave without the interpreter's teardown.
        torch.cuda.synchronize()
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)


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
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--lanes", type=int, default=4,
                    help="parallel graph branches the 16 independent calls of a step are dealt over (1: in order)")
    ap.add_argument("--tp", default="fused", choices=["fused", "nccl"],
                    help="with --gpus N > 1: how the ranks' output columns meet")
    ap.add_argument("--sections", default="e2e,stack,extras,cpu",
                    help="optional legs beside the timed sweep (a profiler run asks for none of them: --sections none)")
    args = ap.parse_args()
    if args.impl == "reference":
        reference_arm(args)
    else:
        our_arm(args)


if __name__ == "__main__":
    main()
