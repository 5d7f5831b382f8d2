"""Benchmark of the quantized decode GEMV hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload llama8b|llama70b] [--batch M] [--mode q8|f32] [--layers L]

Workload (default `llama8b`, BASELINE configs[1]): the Llama-3-8B-shaped FFN GEMVs -- per layer the
fused gate||up projection [28672 x 4096] in Q4_K and the down projection [4096 x 14336] in Q6_K,
fp32 N(0,1) activations at batch M -- over L = 32 layers with distinct weights (3.66 GB), so every
launch streams its matrix from HBM rather than from the 126 MB L2.  A "step" is one pass over all
layers.  Weights are N(0, 0.02) drawn on the device and quantised on the device by the library's
own TensorQuantizer kernels; there is no dataset involved.

One JSON line is printed by rank 0:
  value     whole-job algorithmic GB/s (weights counted once + fp32 activations in + fp32 outputs),
            inputs resident in HBM, steps replayed from a CUDA graph, timed with CUDA events;
  e2e       the same metric through the host-pointer C ABI (smc_qmatmul_host): host buffers in and
            out, H2D/D2H inside the timed region -- this is how a SharpMind slot would call it;
  roofline  the dominant kernel (the Q4_K gate||up GEMV) timed alone over all layers against the
            measured HBM copy bandwidth in MEASURED_PEAKS.json;
  cpu_baseline  the reference's AVX2/FMA tier (C port, oracle/sm_cpu_fma.c) on the host cores, on a
            bounded sample of the same workload.
With --gpus N > 1 (launched under torchrun) every matrix is row-split across the ranks and the
output slices are all-gathered over NCCL; total work is fixed ("strong" scaling).
`--impl reference` times the CPU port alone on a bounded sample per step.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

Q4_K, Q6_K = 12, 14
WORKLOADS = {
    # name: (hidden, ffn, default layers, BASELINE config it stands for)
    "llama8b": (4096, 14336, 32, "configs[1] Llama-3-8B-shaped FFN GEMVs: gate||up 28672x4096 Q4_K, down 4096x14336 Q6_K"),
    "llama70b": (8192, 28672, 80, "configs[4] Llama-3-70B FFN GEMV stack: gate||up 57344x8192 Q4_K, down 8192x28672 Q4_K"),
}


# DRAM traffic per algorithmic byte of the one-row TMA GEMV, from the ncu captures summarised under profiles/
# (Q4_K 28672x4096: 66.116 MB read + 0.48 MB written for 66.191 MB algorithmic; Q6_K 4096x14336: 48.23 MB read +
# 0.1 MB written for 48.243 MB).  Traffic grows with the rows a launch covers, so other shapes scale it.
NCU_TRAFFIC_PER_ALGORITHMIC_BYTE = {Q4_K: (66.116e6 + 0.48e6) / 66191360.0, Q6_K: (48.23e6 + 0.1e6) / 48242688.0}


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="llama8b", choices=sorted(WORKLOADS))
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--mode", default="q8", choices=["q8", "f32"])
    ap.add_argument("--layers", type=int, default=0)
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--gather", default="peer", choices=["peer", "nccl"],
                    help="N > 1: exchange inside the GEMV kernel over peer memory, or a library all-gather per matmul")
    ap.add_argument("--no-extras", action="store_true", help="skip the batch sweep / e2e / cpu baseline")
    ap.add_argument("--cpu-seconds", type=float, default=12.0)
    return ap.parse_args()


def matrices(workload: str):
    """[(name, dtype, N, K)] of one layer."""
    H, F, _, _ = WORKLOADS[workload]
    down_dtype = Q6_K if workload == "llama8b" else Q4_K
    return [("gate_up", Q4_K, 2 * F, H), ("down", down_dtype, H, F)]


def raw_bytes(dtype, n, k):
    return n * k // 256 * (144 if dtype == Q4_K else 210)


def algorithmic_bytes(mats, M):
    """Weights once + fp32 activations in + fp32 outputs, per layer."""
    return sum(raw_bytes(dt, n, k) + 4 * M * k + 4 * M * n for _, dt, n, k in mats)


# ------------------------------------------------------------------------------------------ clocks
class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.gpu)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons, power = [], [], set(), []
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            p = [t.strip() for t in ln.split(",")]
            if len(p) < 9:
                continue
            try:
                sm.append(float(p[1]))
                mx.append(float(p[2]))
                power.append(float(p[3]))
            except ValueError:
                continue
            for name, val in zip(names, p[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(power) if power else None, "samples": len(sm), "reasons": sorted(reasons)}


# ------------------------------------------------------------------------------------------ CPU arm
def cpu_port_time(workload: str, M: int, seconds: float, layers_hint: int = 1):
    """Times the AVX2/FMA port on `layers_hint` layer(s) of the workload, repeated for ~`seconds`."""
    from oracle import sm_oracle as oracle
    from sharpmind_b200 import synth

    oracle.build()
    mats = matrices(workload)
    host = []
    for name, dt, n, k in mats:
        # one layer of weights; block contents do not change the CPU kernels' speed, so the sample
        # tiles a 64-row quantised slab instead of spending minutes in the scalar quantiser
        slab_rows = 64
        slab = oracle.quantize(dt, synth.normal("bench-cpu", name, (slab_rows, k), 0.02))
        raw = np.tile(slab, n // slab_rows)
        x = synth.normal("bench-cpu", name + ".x", (M, k))
        host.append((dt, n, k, raw, x))
    threads = int(oracle.fma_lib().smf_num_threads())

    def one_layer():
        for dt, n, k, raw, x in host:
            oracle.qmatmul_fma(dt, x, raw, M, k, n)

    one_layer()
    t0 = time.perf_counter()
    one_layer()
    t1 = time.perf_counter() - t0
    reps = max(1, min(200, int(seconds / max(t1, 1e-6))))
    t0 = time.perf_counter()
    for _ in range(reps):
        one_layer()
    dt_s = (time.perf_counter() - t0) / reps
    gbs = algorithmic_bytes(mats, M) / dt_s / 1e9
    return {"value": gbs, "unit": "GB/s", "cores": threads, "kind": "port",
            "sample": f"1 of the workload's layers (gate||up + down, batch {M}), {reps} repetitions, "
                      f"{dt_s * 1e3:.1f} ms per layer; C port of the reference's AVX2/FMA tier with its "
                      f"DecodeParallel chunking on {threads} threads"}, dt_s


def run_reference(args):
    """The reference arm: the reference's own CPU implementation of the path (C port of its FMA tier;
    the C# original cannot be compiled on this image), all host threads, bounded sample per step."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    mats = matrices(args.workload)
    M = args.batch
    base, per_layer = cpu_port_time(args.workload, M, seconds=2.0)
    from oracle import sm_oracle as oracle
    from sharpmind_b200 import synth

    host = []
    for name, dt, n, k in mats:
        slab = oracle.quantize(dt, synth.normal("bench-cpu", name, (64, k), 0.02))
        host.append((dt, n, k, np.tile(slab, n // 64), synth.normal("bench-cpu", name + ".x", (M, k))))

    def step():
        for dt, n, k, raw, x in host:
            oracle.qmatmul_fma(dt, x, raw, M, k, n)

    for _ in range(args.warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    el = time.perf_counter() - t0
    ms = el / args.steps * 1e3
    val = algorithmic_bytes(mats, M) * args.steps / el / 1e9
    base["value"] = val
    base["sample"] = f"each step = 1 layer of the workload (gate||up + down, batch {M}) on {base['cores']} host threads"
    out = {"metric": "quant GEMV HBM GB/s", "value": val, "unit": "GB/s", "impl": "reference", "n_gpus": args.gpus,
           "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
           "scaling": "strong", "vs_baseline": None, "dtype": "f32 activations x dequantised int4/int6 weights",
           "data": "synthetic", "config": {"workload": WORKLOADS[args.workload][3], "batch": M,
                                           "sample_layers_per_step": 1},
           "cpu_baseline": base,
           "e2e": {"value": val, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
           "gpu_launches": 0}
    print(json.dumps(out), flush=True)


# ------------------------------------------------------------------------------------------ GPU arm
def run_ours(args):
    import torch

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        import torch.distributed as dist

        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    else:
        dist = None
        torch.cuda.set_device(local)
    from sharpmind_b200 import ops
    from sharpmind_b200.sharded import PeerGather, RowSplit

    ctx = ops.CudaContext(local)
    dev = ops.DeviceOps(ctx)
    mode = ops.Mode.ACT_Q8 if args.mode == "q8" else ops.Mode.ACT_F32
    H, F, Ldef, desc = WORKLOADS[args.workload]
    L = args.layers or Ldef
    mats = matrices(args.workload)
    split = RowSplit(world, rank)

    # ---- weights: generated and quantised on the device, one slice per rank
    weights, host_raw = [], []
    for layer in range(L):
        row = []
        for mi, (name, dt, n, k) in enumerate(mats):
            parts = 2 if name == "gate_up" else 1  # gate and up are split separately
            rows_local = split.rows(n // parts) * parts
            g = torch.Generator(device="cuda").manual_seed(1_000_003 * layer + 101 * mi + 7 * rank + 1)
            wf = torch.randn((rows_local, k), generator=g, device="cuda", dtype=torch.float32) * 0.02
            raw_d = dev.quantize_weights(dt, wf)
            del wf
            if world == 1 and not args.no_extras:
                raw_h = raw_d.cpu().numpy()  # the host-pointer path registers from host memory
                w = ctx.register(raw_h, dt, rows_local, k, repack=True, keep_raw=False)
                host_raw.append(raw_h)
            else:
                w = ctx.register_dev(raw_d, dt, rows_local, k, repack=True, keep_raw=False)
            del raw_d
            row.append(w)
        weights.append(row)
    torch.cuda.synchronize()

    def make_inputs(M):
        return [torch.from_numpy(np.random.default_rng(17 + i).standard_normal((M, k), dtype=np.float32)).cuda()
                for i, (_, _, _, k) in enumerate(mats)]

    def make_state(M):
        xs = make_inputs(M)
        acts = [ops.Q8Act(ctx, M, k) for (_, _, _, k) in mats]
        outs = [torch.empty((M, w.N), device="cuda", dtype=torch.float32) for w in weights[0]]
        gathered = [torch.empty((world, M, w.N), device="cuda", dtype=torch.float32) for w in weights[0]] if world > 1 else None
        return xs, acts, outs, gathered

    comm_stream = torch.cuda.Stream() if world > 1 else None
    peer = world > 1 and args.gather == "peer"
    gathers = {}

    def gather_for(M, mi):
        # one receive buffer per (batch, matrix): the exchange runs inside the GEMV kernel over peer memory
        if (M, mi) not in gathers:
            gathers[(M, mi)] = PeerGather(ctx, split, world * M * weights[0][mi].N, dist)
        return gathers[(M, mi)]

    def step(state, M):
        xs, acts, outs, gathered = state
        for layer in range(L):
            for mi, w in enumerate(weights[layer]):
                if peer:
                    gather_for(M, mi).matmul(xs[mi], w, mode)
                    continue
                if mode == ops.Mode.ACT_Q8 and M > 1:
                    dev.quantize_q8(xs[mi], acts[mi], w.K)
                    dev.qmatmul_q8(acts[mi], w, out=outs[mi])
                else:
                    # one row: the Q8_0 quantisation of the activations happens inside the GEMV kernel
                    dev.qmatmul(xs[mi], w, mode, out=outs[mi])
                if world > 1:
                    # the exchange step of the row-split: every rank receives every slice
                    ev = torch.cuda.Event()
                    ev.record()
                    with torch.cuda.stream(comm_stream):
                        comm_stream.wait_event(ev)
                        dist.all_gather_into_tensor(gathered[mi].view(world * M, -1), outs[mi])
                    # the next launch that overwrites outs[mi] must wait for this gather
                    done = torch.cuda.Event()
                    done.record(comm_stream)
                    torch.cuda.current_stream().wait_event(done)

    def launches_per_step(M):
        # M = 1 rows up to K = 8192 are quantised inside the GEMV kernel; otherwise a quantiser launch precedes it
        per = sum(2 if (mode == ops.Mode.ACT_Q8 and (M > 1 or k > 8192)) else 1 for _, _, _, k in mats)
        if peer and not (mode == ops.Mode.ACT_Q8 and M == 1):
            per += len(mats)  # the exchange is a launch of its own unless it rides in the one-row GEMV's tail
        return L * per

    def timed(M, steps, warmup, use_graph, preload_s=0.0):
        state = make_state(M)
        runner = lambda: step(state, M)  # noqa: E731
        graph = None
        if peer:
            for mi in range(len(mats)):
                gather_for(M, mi)  # created (and peers mapped) on every rank before anything is timed or captured
        if use_graph and (world == 1 or peer):
            s = torch.cuda.Stream()
            s.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(s):
                step(state, M)  # warm-up outside capture (first calls may allocate)
            torch.cuda.current_stream().wait_stream(s)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                step(state, M)
            runner = graph.replay
        for _ in range(max(warmup, 3)):
            runner()
        torch.cuda.synchronize()
        # The timed region of a few dozen steps lasts tens of milliseconds, too short for the 200 ms clock sampler:
        # the same step is replayed (untimed) for `preload_s` first, so that the clocks and throttle reasons that are
        # sampled are those of the GPU under this very load.  The number of replays is fixed on rank 0 and broadcast.
        if preload_s > 0:
            t_one = time.perf_counter()
            runner()
            torch.cuda.synchronize()
            reps = int(min(5000, max(1, preload_s / max(time.perf_counter() - t_one, 1e-5))))
            if dist is not None:
                rt = torch.tensor([reps], device="cuda")
                dist.broadcast(rt, 0)
                reps = int(rt.item())
            for _ in range(reps):
                runner()
            torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            runner()
        e1.record()
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        if dist is not None:
            t = torch.tensor([ms], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms / steps, graph is not None

    M = args.batch
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    ms_step, graphed = timed(M, args.steps, args.warmup, not args.no_graph, preload_s=1.2)
    clocks = sampler.stop() if rank == 0 else None

    # whole-job bytes: the full matrices (all ranks' slices) + activations and outputs once
    step_bytes = algorithmic_bytes(mats, M) * L
    value = step_bytes / (ms_step * 1e-3) / 1e9

    result = {
        "metric": "quant GEMV HBM GB/s", "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "int8 x int4/int6 dp4a, fp32 scale" if mode == ops.Mode.ACT_Q8 else "f32",
        "data": "synthetic",
        "config": {"workload": desc, "layers": L, "batch": M, "activations": "q8_0 on device" if mode == ops.Mode.ACT_Q8 else "fp32",
                   "weight_bytes": sum(raw_bytes(dt, n, k) for _, dt, n, k in mats) * L,
                   "l2": f"{L} distinct layers ({step_bytes / 1e9:.2f} GB per step) >> 126 MB L2",
                   "cuda_graph": graphed,
                   "parallelism": "single GPU" if world == 1 else (
                       f"row-split x{world}, slices exchanged by the GEMV kernel over NVLink peer memory" if peer
                       else f"row-split x{world} + NCCL all-gather")},
        "pct_of_8TBs_nominal": value / 8000.0 * 100.0 / world,
        "gpu_launches": launches_per_step(M) * args.steps,
        "clocks": clocks,
    }

    if rank == 0 and not args.no_extras:
        peaks = {}
        try:
            peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        except (OSError, ValueError):
            pass
        peak = float(peaks.get("hbm_gbs", 6650.0))
        peak_src = "measured (MEASURED_PEAKS.json hbm_gbs)" if "hbm_gbs" in peaks else "fallback 6650 GB/s"
        # ---- roofline of the dominant kernel: the gate||up GEMV alone over all layers
        name, dt, n, k = mats[0]
        xs, acts, outs, _ = make_state(M)
        if mode == ops.Mode.ACT_Q8 and M > 1:
            dev.quantize_q8(xs[0], acts[0], k)
        def graph_time_us(fn, reps=10):
            """Average duration of one launch of `fn`'s L launches, replayed from a CUDA graph (no host gaps)."""
            st = torch.cuda.Stream()
            st.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(st):
                fn()
            torch.cuda.current_stream().wait_stream(st)
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                fn()
            for _ in range(3):
                g.replay()
            torch.cuda.synchronize()
            t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0.record()
            for _ in range(reps):
                g.replay()
            t1.record()
            torch.cuda.synchronize()
            return t0.elapsed_time(t1) * 1e3 / (reps * L)

        def dom():
            for layer in range(L):
                if mode == ops.Mode.ACT_Q8 and M > 1:
                    dev.qmatmul_q8(acts[0], weights[layer][0], out=outs[0])
                else:
                    dev.qmatmul(xs[0], weights[layer][0], mode, out=outs[0])
        us_launch = graph_time_us(dom)
        n_local = weights[0][0].N
        kbytes = raw_bytes(dt, n_local, k) + 4 * M * k + 4 * M * n_local
        achieved = kbytes / (us_launch * 1e-6) / 1e9
        result["roofline"] = {"bound": "hbm", "kernel": "gemv_tma_kernel<MathQ4K> (gate||up, Q4_K)", "achieved": achieved,
                              "peak": peak, "unit": "GB/s", "frac": achieved / peak, "peak_source": peak_src,
                              "us_per_launch": us_launch, "algorithmic_bytes_per_launch": kbytes,
                              "traffic": (NCU_TRAFFIC_PER_ALGORITHMIC_BYTE.get(dt, 0) * kbytes) or None,
                              "traffic_source": "ncu dram__bytes_read+write of one launch of this kernel on the single-GPU "
                                                "shape (profiles/gemv_tma_q4k_llama8b_gate_up.md), scaled by rows"}
        # ---- the other matrix, for the record
        xs2 = xs[1]
        if mode == ops.Mode.ACT_Q8 and M > 1:
            dev.quantize_q8(xs2, acts[1], mats[1][3])
        def dom2():
            for layer in range(L):
                if mode == ops.Mode.ACT_Q8 and M > 1:
                    dev.qmatmul_q8(acts[1], weights[layer][1], out=outs[1])
                else:
                    dev.qmatmul(xs2, weights[layer][1], mode, out=outs[1])
        us2 = graph_time_us(dom2)
        b2 = raw_bytes(mats[1][1], weights[0][1].N, mats[1][3]) + 4 * M * mats[1][3] + 4 * M * weights[0][1].N
        result["kernels"] = {"gate_up": {"us": us_launch, "GBps": achieved},
                             "down": {"us": us2, "GBps": b2 / (us2 * 1e-6) / 1e9}}

        if world == 1:
            # ---- batch sweep and the other activation mode (fewer steps)
            sweep = {}
            for m2 in (1, 8, 32):
                for md, label in ((ops.Mode.ACT_Q8, "q8"), (ops.Mode.ACT_F32, "f32")):
                    if m2 == M and md == mode:
                        sweep[f"{label}_b{m2}"] = value
                        continue
                    if md == ops.Mode.ACT_F32 and m2 > 8:
                        continue  # CUDA-core bound by construction; not a bandwidth number
                    saved = mode
                    mode = md
                    try:
                        ms2, _ = timed(m2, max(2, args.steps // 4), 3, not args.no_graph)
                        sweep[f"{label}_b{m2}"] = algorithmic_bytes(mats, m2) * L / (ms2 * 1e-3) / 1e9
                    finally:
                        mode = saved
            result["sweep_GBps"] = sweep

            # ---- the 70B-shaped stack of configs[4] on this GPU (12 of its 80 layers: 4.8 GB per step >> L2), batch 1
            if args.workload == "llama8b":
                try:
                    mats70 = matrices("llama70b")
                    w70 = []
                    for layer in range(12):
                        row = []
                        for mi, (name, dt, n, k) in enumerate(mats70):
                            g70 = torch.Generator(device="cuda").manual_seed(7_000_003 * layer + 11 * mi + 1)
                            wf = torch.randn((n, k), generator=g70, device="cuda", dtype=torch.float32) * 0.02
                            raw_d = dev.quantize_weights(dt, wf)
                            del wf
                            row.append(ctx.register_dev(raw_d, dt, n, k, repack=True, keep_raw=False))
                            del raw_d
                        w70.append(row)
                    x70 = [torch.from_numpy(np.random.default_rng(170 + i).standard_normal((1, k), dtype=np.float32)).cuda()
                           for i, (_, _, _, k) in enumerate(mats70)]
                    o70 = [torch.empty((1, w.N), device="cuda", dtype=torch.float32) for w in w70[0]]

                    def step70():
                        for row in w70:
                            for mi, w in enumerate(row):
                                dev.qmatmul(x70[mi], w, ops.Mode.ACT_Q8, out=o70[mi])

                    st = torch.cuda.Stream()
                    st.wait_stream(torch.cuda.current_stream())
                    with torch.cuda.stream(st):
                        step70()
                    torch.cuda.current_stream().wait_stream(st)
                    torch.cuda.synchronize()
                    g = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(g):
                        step70()
                    for _ in range(3):
                        g.replay()
                    torch.cuda.synchronize()
                    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    t0.record()
                    for _ in range(10):
                        g.replay()
                    t1.record()
                    torch.cuda.synchronize()
                    ms70 = t0.elapsed_time(t1) / 10
                    b70 = algorithmic_bytes(mats70, 1) * 12
                    result["stack70b"] = {"workload": WORKLOADS["llama70b"][3], "layers_timed": 12, "batch": 1,
                                          "ms_per_12_layers": ms70, "GBps": b70 / (ms70 * 1e-3) / 1e9,
                                          "frac_of_measured_hbm": b70 / (ms70 * 1e-3) / 1e9 / peak}
                    for row in w70:
                        for w in row:
                            ctx.release(w)
                    del w70, x70, o70, g
                except Exception as exc:
                    result["stack70b"] = {"error": str(exc)}

            # ---- end to end through the host-pointer C ABI
            q = ops.QuantizationOps(ctx, mode)
            xs_h = [np.random.default_rng(17 + i).standard_normal((M, k), dtype=np.float32) for i, (_, _, _, k) in enumerate(mats)]
            outs_h = [np.empty((M, n), np.float32) for (_, _, n, _) in mats]
            def e2e_step():
                i = 0
                for layer in range(L):
                    for mi, (nm, dt_, n_, k_) in enumerate(mats):
                        q.QuantizedMatMulFn(dt_, xs_h[mi], host_raw[i], outs_h[mi], M, k_, n_)
                        i += 1
            e2e_step()
            e2e_steps = max(2, args.steps // 4)
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            for _ in range(e2e_steps):
                e2e_step()
            torch.cuda.synchronize()
            el = (time.perf_counter() - t0) / e2e_steps
            result["e2e"] = {"value": step_bytes / el / 1e9, "unit": "GB/s", "ms_per_step": el * 1e3,
                             "h2d_bytes_per_step": sum(4 * M * k for _, _, _, k in mats) * L,
                             "d2h_bytes_per_step": sum(4 * M * n for _, _, n, _ in mats) * L,
                             "api": "smc_qmatmul_host: one synchronous call per matmul, host fp32 in / out"}
            # ---- prefill-sized batch on the tcgen05 tensor-core kernel (512 tokens, the Q4_K gate||up matrices)
            try:
                mp = 512
                xp = torch.from_numpy(np.random.default_rng(5).standard_normal((mp, mats[0][3]), dtype=np.float32)).cuda()
                op = torch.empty((mp, weights[0][0].N), device="cuda", dtype=torch.float32)
                dev.qmatmul(xp, weights[0][0], ops.Mode.ACT_F32, out=op)  # first call sizes the scratch
                torch.cuda.synchronize()
                t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                t0.record()
                for layer in range(L):
                    dev.qmatmul(xp, weights[layer][0], ops.Mode.ACT_F32, out=op)
                t1.record()
                torch.cuda.synchronize()
                msp = t0.elapsed_time(t1) / L
                tf = 2.0 * mp * weights[0][0].N * mats[0][3] / msp / 1e9
                tpeak = float(peaks.get("bf16_tflops", 1590.0))
                result["prefill"] = {"kernel": "prefill_q4k_kernel (tcgen05.mma kind::f16, fp16 integer weights x fp16 hi/lo activations)",
                                     "M": mp, "N": weights[0][0].N, "K": mats[0][3], "ms_per_matmul": msp, "useful_TFLOPs": tf,
                                     "tensor_TFLOPs_issued": 2 * tf, "peak_TFLOPs": tpeak, "frac_useful": tf / tpeak,
                                     "peak_source": "measured bf16 burst (MEASURED_PEAKS.json)" if "bf16_tflops" in peaks else "fallback"}
                del xp, op
            except Exception as exc:
                result["prefill"] = {"error": str(exc)}
            # ---- the other half of the metric: decode tokens/s of the Qwen3-0.6B-shaped model (configs[3])
            try:
                from sharpmind_b200 import synth
                from sharpmind_b200.profile_decode import time_decode

                rows = time_decode(ctx, dev, dict(synth.QWEN3_0_6B), [1, 32], 2048, 16)
                result["decode"] = {
                    "workload": "configs[3] Qwen3-0.6B-shaped decoder, Q8_0 weights, fp32 KV with a 2048-position seeded "
                                "random context, one greedy token per sequence per step, q8_0 activations, CUDA graph",
                    "tokens_per_s_batch1": rows[0]["tokens_per_s_graph"], "ms_per_step_batch1": rows[0]["graph_ms_per_step"],
                    "tokens_per_s_batch32": rows[1]["tokens_per_s_graph"], "ms_per_step_batch32": rows[1]["graph_ms_per_step"],
                    "GBps_batch1": rows[0]["GBps_graph"], "GBps_batch32": rows[1]["GBps_graph"]}
                from sharpmind_b200.profile_decode import time_prompt

                pr = time_prompt(ctx, dev, dict(synth.QWEN3_0_6B), 2048, 1024, "q8", 2)
                result["decode"]["prompt_pass"] = {"what": "ForwardLastLogits over a 2048-token seeded prompt in chunks of 1024, one sequence",
                                                   "ms": pr["ms"], "tokens_per_s": pr["tokens_per_s"]}
            except Exception as exc:
                result.setdefault("decode", {})["error"] = str(exc)
            # ---- the same step on a Llama-3-8B shape with K-quant weights (the formats of configs[1] in a whole decoder)
            try:
                torch.cuda.empty_cache()
                rows8 = time_decode(ctx, dev, dict(synth.LLAMA3_8B), [1, 32], 2048, 8)
                result["decode_llama8b"] = {
                    "workload": "Llama-3-8B-shaped decoder: Q4_K attention and gate||up, Q6_K down, Q8_0 tied embedding, fp32 KV, "
                                "2048-position seeded random context, q8_0 activations, CUDA graph",
                    "tokens_per_s_batch1": rows8[0]["tokens_per_s_graph"], "ms_per_step_batch1": rows8[0]["graph_ms_per_step"],
                    "tokens_per_s_batch32": rows8[1]["tokens_per_s_graph"], "ms_per_step_batch32": rows8[1]["graph_ms_per_step"],
                    "GBps_batch1": rows8[0]["GBps_graph"], "GBps_batch32": rows8[1]["GBps_graph"]}
            except Exception as exc:
                result["decode_llama8b"] = {"error": str(exc)}
            # ---- CPU baseline on the host cores
            try:
                result["cpu_baseline"], _ = cpu_port_time(args.workload, M, args.cpu_seconds)
            except Exception as exc:  # the baseline is reported, never required
                result["cpu_baseline"] = {"value": None, "unit": "GB/s", "cores": None, "kind": "port",
                                          "sample": f"failed: {exc}"}
    if rank == 0:
        print(json.dumps(result), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()
    ctx.close()


def main():
    args = parse()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
