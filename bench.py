"""Benchmark of the quantized decode GEMV hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload llama70b|llama8b] [--batch M] [--mode q8|f32] [--layers L]
                    [--only gemv:<shape>[:<M>[:q8|q8pre|f32[:ring]]] | decode[:qwen3|llama8b][:q8kv] | prompt[:llama8b] | elementwise | prefill]

Workload (default `llama70b`, BASELINE configs[4], the largest configuration that fits one GPU and the one the
multi-GPU target is stated on): the Llama-3-70B-shaped FFN GEMV stack -- per layer the fused gate||up projection
[57344 x 8192] and the down projection [8192 x 28672], both Q4_K, fp32 N(0,1) activations at batch M -- over
L = 80 layers with distinct weights (31.7 GB), so every launch streams its matrix from HBM rather than from the
126 MB L2.  `--workload llama8b` is configs[1] (gate||up [28672 x 4096] Q4_K, down [4096 x 14336] Q6_K, 32 layers).
A "step" is one pass over all layers.  Weights are N(0, 0.02) drawn on the device and quantised on the device by the
library's own TensorQuantizer kernels (bit-exact with the CPU oracle's); there is no dataset involved.

One JSON line is printed by rank 0:
  value     whole-job algorithmic GB/s (weights counted once + fp32 activations in + fp32 outputs), inputs resident
            in HBM, steps replayed from a CUDA graph, timed with CUDA events, max over ranks;
  e2e       the same metric through the host-facing call: host fp32 activations in, host fp32 outputs back, H2D / D2H
            inside the timed region.  One GPU: smc_qmatmul_host_w (the C-ABI slot a SharpMind linear layer binds);
            N GPUs: pinned host row -> device, the layer's two kernels, summed row -> pinned host, per layer;
  roofline  the kernel with the largest share of the step, timed alone over all layers against the measured HBM copy
            bandwidth in MEASURED_PEAKS.json; `kernels` carries every matrix of the workload the same way;
  parity    N > 1: before anything is timed rank 0 regenerates every rank's slices of layer 0, computes them locally and
            compares the exchanged result bit for bit;
  cpu_baseline  the reference's AVX2/FMA tier (C port, oracle/sm_cpu_fma.c) on the host cores, on a bounded sample;
  extras at N = 1: the configs[1] stack with its batch sweep, configs[0] (Q8_0 3072 x 1024 and the LM-head GEMV),
            configs[2] (the fp32 elementwise chain), the tcgen05 prefill matmul, decode tokens/s (configs[3]).
With --gpus N > 1 (launched under torchrun) the layer runs tensor-parallel with ONE exchange (`--tp ffn`, the default for
one activation row): gate||up split by rows, its output and the SiLU-gate stay on the rank, the down projection is split
along K and its partial sums are exchanged and added in rank order inside the GEMV kernel over NVLink peer memory.
`--tp rows` splits every matrix by rows and exchanges the output slices of every matmul inside the kernel;
`--gather nccl` uses a library all-gather per matmul instead.  Total work is fixed ("strong" scaling).
`--impl reference` times the CPU port alone on a bounded sample per step (rank 0 only, all host threads).
`--only ...` runs one kernel or section by itself and prints its own JSON line: the commands behind profiles/.
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

Q8_0, Q4_K, Q6_K = 8, 12, 14
BLOCK = {Q8_0: (32, 34), Q4_K: (256, 144), Q6_K: (256, 210)}
WORKLOADS = {
    # name: (hidden, ffn, default layers, down dtype, BASELINE config it stands for)
    "llama70b": (8192, 28672, 80, Q4_K, "configs[4] Llama-3-70B FFN GEMV stack: gate||up 57344x8192 Q4_K, down 8192x28672 Q4_K"),
    "llama8b": (4096, 14336, 32, Q6_K, "configs[1] Llama-3-8B-shaped FFN GEMVs: gate||up 28672x4096 Q4_K, down 4096x14336 Q6_K"),
}
# single matrices for --only gemv:<shape>: (dtype, N, K, distinct copies cycled to stay out of L2)
GEMV_SHAPES = {
    "q4k": (Q4_K, 28672, 4096, 5), "q6k": (Q6_K, 4096, 14336, 5), "q8": (Q8_0, 3072, 1024, 48),
    "lmhead": (Q8_0, 151936, 1024, 3), "q4k70": (Q4_K, 57344, 8192, 2), "q4kd70": (Q4_K, 8192, 28672, 3),
    "wo": (Q4_K, 4096, 4096, 20), "q6k70": (Q6_K, 8192, 28672, 2),
    # the Qwen3-0.6B-shaped prompt pass's matmuls (timed with M = the chunk, e.g. gemv:q8gu:1024:q8pre)
    "q8gu": (Q8_0, 6144, 1024, 8), "q8dn": (Q8_0, 1024, 3072, 8), "q8qkv": (Q8_0, 4096, 1024, 8), "q8wo": (Q8_0, 1024, 2048, 8),
}
# DRAM traffic per algorithmic byte of the one-row GEMV: ncu dram__bytes_read + dram__bytes_write of one launch of the
# largest captured shape of each format (profiles/gemv_tma_one_row_all_formats.md: reads are 0.998-1.009 of the
# algorithmic bytes, the rest are dirty lines of earlier kernels leaving the L2 during the capture); traffic grows with
# the rows a launch covers, so other shapes scale it.
NCU_TRAFFIC_PER_ALGORITHMIC_BYTE = {Q4_K: 1.022, Q6_K: 1.044, Q8_0: 1.040}


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="llama70b", choices=sorted(WORKLOADS))
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--mode", default="q8", choices=["q8", "f32"])
    ap.add_argument("--layers", type=int, default=0)
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--chunk", type=int, default=2048, help="--only prompt: tokens per ForwardLastLogits call")
    ap.add_argument("--gather", default="peer", choices=["peer", "nccl"],
                    help="N > 1: exchange inside the GEMV kernel over peer memory, or a library all-gather per matmul")
    ap.add_argument("--tp", default="ffn", choices=["ffn", "rows"],
                    help="N > 1, one row: 'ffn' = gate||up by rows, SwiGLU local, down split along K with the partial sums "
                         "exchanged and added inside the kernel (one exchange per layer); 'rows' = every matrix by rows, "
                         "one exchange per matmul")
    ap.add_argument("--tp-pairs", action="store_true",
                    help="--tp ffn: gate / up rows woven and the SiLU-gate in the first matmul's epilogue instead of the second's staging "
                         "(pays only while the rank's slice of the row is long: 14 336 elements at N = 2)")
    ap.add_argument("--no-exchange", action="store_true",
                    help="diagnosis only (the line is marked invalid): N > 1 with --tp ffn, but the partial sums are not exchanged")
    ap.add_argument("--no-extras", action="store_true", help="skip everything but the headline line (and e2e)")
    ap.add_argument("--cpu-seconds", type=float, default=12.0)
    ap.add_argument("--only", default="", help="run one kernel / section alone (see the module docstring)")
    return ap.parse_args()


def matrices(workload: str):
    """[(name, dtype, N, K)] of one layer."""
    H, F, _, down_dtype, _ = WORKLOADS[workload]
    return [("gate_up", Q4_K, 2 * F, H), ("down", down_dtype, H, F)]


def raw_bytes(dtype, n, k):
    be, bb = BLOCK[dtype]
    return n * k // be * bb


def algorithmic_bytes(mats, M):
    """Weights once + fp32 activations in + fp32 outputs, per layer."""
    return sum(raw_bytes(dt, n, k) + 4 * M * k + 4 * M * n for _, dt, n, k in mats)


def load_peaks():
    try:
        return json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except (OSError, ValueError):
        return {}


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
                "power_w_max": max(power) if power else None, "samples": len(sm), "reasons": sorted(reasons),
                "source": "sampled every 100 ms while the timed step was replayed: an untimed preload of about 1.2 s "
                          "of the very same graph, then the timed region (tens of milliseconds)"}


# ------------------------------------------------------------------------------------------ CPU arm
def _cpu_layer(workload: str, M: int):
    """One layer of the workload on the host: tiled 64-row quantised slabs (block contents do not change the CPU
    kernels' speed) and seeded activations."""
    from oracle import sm_oracle as oracle
    from sharpmind_b200 import synth

    oracle.build()
    fma = oracle.fma_lib()
    fma.smf_set_threads.restype = None
    fma.smf_set_threads.argtypes = [__import__("ctypes").c_int]
    fma.smf_set_threads(os.cpu_count() or 1)  # a launcher may have exported OMP_NUM_THREADS=1
    host = []
    for name, dt, n, k in matrices(workload):
        slab = oracle.quantize(dt, synth.normal("bench-cpu", f"{workload}.{name}", (64, k), 0.02))
        host.append((dt, n, k, np.tile(slab, n // 64), synth.normal("bench-cpu", f"{workload}.{name}.x", (M, k))))

    def one_layer():
        for dt, n, k, raw, x in host:
            oracle.qmatmul_fma(dt, x, raw, M, k, n)

    return one_layer, int(fma.smf_num_threads())


def cpu_port_time(workload: str, M: int, seconds: float):
    """Times the AVX2/FMA port on one layer of the workload, repeated for about `seconds`."""
    one_layer, threads = _cpu_layer(workload, M)
    one_layer()
    t0 = time.perf_counter()
    one_layer()
    t1 = time.perf_counter() - t0
    reps = max(1, min(200, int(seconds / max(t1, 1e-6))))
    t0 = time.perf_counter()
    for _ in range(reps):
        one_layer()
    dt_s = (time.perf_counter() - t0) / reps
    gbs = algorithmic_bytes(matrices(workload), M) / dt_s / 1e9
    return {"value": gbs, "unit": "GB/s", "cores": threads, "kind": "port",
            "sample": f"1 of the workload's layers (gate||up + down, batch {M}), {reps} repetitions, "
                      f"{dt_s * 1e3:.1f} ms per layer; C port of the reference's AVX2/FMA tier with its "
                      f"DecodeParallel chunking on {threads} threads"}


def run_reference(args):
    """The reference arm: the reference's own CPU implementation of the path (C port of its FMA tier; the C# original
    cannot be compiled on this image), all host threads, a bounded sample (one layer) per step.  Rank 0 only."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    mats = matrices(args.workload)
    M = args.batch
    step, threads = _cpu_layer(args.workload, M)
    for _ in range(max(args.warmup, 1)):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    el = time.perf_counter() - t0
    val = algorithmic_bytes(mats, M) * args.steps / el / 1e9
    base = {"value": val, "unit": "GB/s", "cores": threads, "kind": "port",
            "sample": f"each step = 1 layer of the workload (gate||up + down, batch {M}) on {threads} host threads"}
    out = {"metric": "quant GEMV HBM GB/s", "value": val, "unit": "GB/s", "impl": "reference", "n_gpus": args.gpus,
           "steps": args.steps, "warmup": args.warmup, "ms_per_step": el / args.steps * 1e3, "higher_is_better": True,
           "scaling": "strong", "vs_baseline": None, "dtype": "f32 activations x dequantised int4/int6 weights",
           "data": "synthetic", "config": {"workload": WORKLOADS[args.workload][4], "batch": M, "sample_layers_per_step": 1},
           "cpu_baseline": base,
           "e2e": {"value": val, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
           "gpu_launches": 0}
    print(json.dumps(out), flush=True)


# ------------------------------------------------------------------------------------------ timing helpers
def graph_of(torch, fn):
    """Runs `fn` once on a side stream (first calls may allocate), then captures it."""
    st = torch.cuda.Stream()
    st.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(st):
        fn()
    torch.cuda.current_stream().wait_stream(st)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        fn()
    return g


def time_graph_us(torch, fn, launches: int, reps: int = 10) -> float:
    """Average duration of one of `fn`'s `launches` launches, replayed from a CUDA graph (no host gaps), CUDA events."""
    g = graph_of(torch, fn)
    for _ in range(3):
        g.replay()
    torch.cuda.synchronize()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for _ in range(reps):
        g.replay()
    t1.record()
    torch.cuda.synchronize()
    return t0.elapsed_time(t1) * 1e3 / (reps * launches)


def device_matrix(torch, dev, ctx, dt, n, k, seed, keep_raw=False):
    g = torch.Generator(device="cuda").manual_seed(seed)
    wf = torch.randn((n, k), generator=g, device="cuda", dtype=torch.float32) * 0.02
    raw_d = dev.quantize_weights(dt, wf)
    del wf
    w = ctx.register_dev(raw_d, dt, n, k, repack=True, keep_raw=keep_raw)
    del raw_d
    return w


# ------------------------------------------------------------------------------------------ --only sections
def decoder_device_weights(torch, dev, cfg: dict, seed: int = 1234) -> dict:
    g = torch.Generator(device="cuda")
    g.manual_seed(seed)
    L, H, hd = cfg["n_layers"], cfg["hidden"], cfg["head_dim"]
    q_dim, kv_dim, F, V, dt = cfg["n_heads"] * hd, cfg["n_kv_heads"] * hd, cfg["ffn"], cfg["vocab"], cfg["dtype"]

    def mat(n, k, fmt=None):
        return dev.quantize_weights(fmt or dt, torch.randn((n, k), generator=g, device="cuda") * 0.02)

    def vec(n):
        return torch.randn(n, generator=g, device="cuda") * 0.1 + 1.0

    w = {k: [] for k in ("wq", "wk", "wv", "wo", "wgu", "wdown", "norm1", "norm2", "qnorm", "knorm")}
    for _ in range(L):
        w["wq"].append(mat(q_dim, H)), w["wk"].append(mat(kv_dim, H)), w["wv"].append(mat(kv_dim, H))
        w["wo"].append(mat(H, q_dim)), w["wgu"].append(mat(2 * F, H)), w["wdown"].append(mat(H, F, cfg.get("down_dtype")))
        w["norm1"].append(vec(H)), w["norm2"].append(vec(H)), w["qnorm"].append(vec(hd)), w["knorm"].append(vec(hd))
    w["final_norm"] = vec(H)
    w["embedding"] = mat(V, H, cfg.get("head_dtype"))
    return w


def decode_step_bytes(cfg: dict, batch: int, ctx_len: int) -> dict:
    """Bytes one step has to read: every weight block once, and the K/V rows of the context per sequence."""
    L, H, hd = cfg["n_layers"], cfg["hidden"], cfg["head_dim"]
    q_dim, kv_dim, F, V = cfg["n_heads"] * hd, cfg["n_kv_heads"] * hd, cfg["ffn"], cfg["vocab"]
    bpe = {8: 34 / 32, 12: 144 / 256, 14: 210 / 256}
    dt = cfg["dtype"]
    per_layer = (q_dim * H + 2 * kv_dim * H + H * q_dim + 2 * F * H) * bpe[dt] + H * F * bpe[cfg.get("down_dtype") or dt]
    weights = int(L * per_layer + V * H * bpe[cfg.get("head_dtype") or dt])
    kv_bpe = 34 / 32 if cfg.get("kv_dtype") == 8 else 4  # QuantizedKVCache rows are Q8_0 blocks
    kv = int(L * batch * 2 * cfg["n_kv_heads"] * (ctx_len + 1) * hd * kv_bpe)
    return {"weights": weights, "kv": kv}


def time_decode(torch, ctx, dev, cfg: dict, batches, ctx_len: int, steps: int, mode, once: bool = False) -> list:
    """Builds the model, installs a `ctx_len`-position seeded random context (the step's cost depends on the context
    length only) and times one-token steps replayed from a CUDA graph; one dict per batch size."""
    from sharpmind_b200.decoder import Decoder

    w = decoder_device_weights(torch, dev, cfg)
    dec = Decoder(ctx, cfg, w, max_batch=max(batches))
    del w
    g = torch.Generator(device="cuda")
    g.manual_seed(99)
    shape = (cfg["n_layers"], max(batches), cfg["n_kv_heads"], ctx_len, cfg["head_dim"])
    k, v = torch.randn(shape, generator=g, device="cuda"), torch.randn(shape, generator=g, device="cuda")
    dec.load_kv(k, v)
    torch.cuda.synchronize()
    del k, v
    torch.cuda.empty_cache()
    rows = []
    for B in batches:
        tok = torch.randint(0, cfg["vocab"], (B,), generator=g, device="cuda", dtype=torch.int32)
        logits = torch.empty((B, cfg["vocab"]), device="cuda")
        nxt = torch.empty(B, dtype=torch.int32, device="cuda")
        if once:
            dec.step(tok, ctx_len, mode, logits, nxt)
            torch.cuda.synchronize()
            continue
        us = time_graph_us(torch, lambda: dec.step(tok, ctx_len, mode, logits, nxt), 1, reps=steps)
        by = decode_step_bytes(cfg, B, ctx_len)
        rows.append({"batch": B, "ctx": ctx_len, "layers": cfg["n_layers"], "ms_per_step": round(us / 1e3, 4),
                     "tokens_per_s": round(B / us * 1e6, 1), "weight_MB": round(by["weights"] / 1e6, 1),
                     "kv_MB": round(by["kv"] / 1e6, 1), "GBps": round((by["weights"] + by["kv"]) / us / 1e3, 1),
                     "device_status": ctx.device_status()})
    dec.close()
    return rows


def time_prompt(torch, ctx, dev, cfg: dict, n_tokens: int, chunk: int, mode, reps: int = 3) -> dict:
    """Times ForwardLastLogits over a seeded random prompt of `n_tokens` (one sequence, chunks of `chunk` tokens)."""
    from sharpmind_b200.decoder import Decoder

    w = decoder_device_weights(torch, dev, cfg)
    dec = Decoder(ctx, cfg, w, max_batch=1)
    del w
    g = torch.Generator(device="cuda")
    g.manual_seed(7)
    tok = torch.randint(0, cfg["vocab"], (n_tokens,), generator=g, device="cuda", dtype=torch.int32)
    dec.forward_last_logits(tok, 0, 0, mode, chunk)  # grows the scratch, warms up
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        dec.forward_last_logits(tok, 0, 0, mode, chunk)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / reps
    row = {"prompt_tokens": n_tokens, "chunk": chunk, "layers": cfg["n_layers"], "ms": round(ms, 3),
           "tokens_per_s": round(n_tokens / ms * 1e3, 1), "device_status": ctx.device_status()}
    dec.close()
    return row


def time_gemv_shape(torch, ctx, dev, ops, which: str, M: int, mode: str, peak: float, once: bool = False) -> dict:
    """One matrix shape alone: `copies` distinct matrices (more than the L2 in total) cycled inside a CUDA graph."""
    dt, n, k, L = GEMV_SHAPES[which]
    ws = [device_matrix(torch, dev, ctx, dt, n, k, layer + 1) for layer in range(L)]
    x = torch.randn((M, k), device="cuda")
    act = ops.Q8Act(ctx, M, k)
    out = torch.empty((M, n), device="cuda")
    dev.quantize_q8(x, act, k)

    def body():
        for w in ws:
            if mode == "q8pre":
                dev.qmatmul_q8(act, w, out=out)
            elif mode == "q8":
                dev.qmatmul(x, w, ops.Mode.ACT_Q8, out=out)
            else:
                dev.qmatmul(x, w, ops.Mode.ACT_F32, out=out)

    if once:  # one pass over the copies, no graph: the form a counter capture wants
        body()
        torch.cuda.synchronize()
        return {"shape": which, "M": M, "mode": mode, "launches": L, "device_status": ctx.device_status()}
    us = time_graph_us(torch, body, L, reps=5)
    nbytes = raw_bytes(dt, n, k) + 4 * M * k + 4 * M * n
    for w in ws:
        ctx.release(w)
    return {"shape": which, "dtype": dt, "N": n, "K": k, "M": M, "mode": mode, "copies": L, "us_per_launch": round(us, 2),
            "algorithmic_bytes": nbytes, "GBps": round(nbytes / us / 1e3, 1), "frac_of_hbm_peak": round(nbytes / us / 1e3 / peak, 3),
            "device_status": ctx.device_status()}


def elementwise_chain(torch, ctx, dev, peak: float, rows_list=(64, 1024), reps: int = 10, once: bool = False) -> list:
    """configs[2]: RMSNorm over hidden 4096 (eps 1e-6, weight N(1, 0.1)), SiLU(gate)*up on rows x 14336, RoPE theta
    500000 on rows tokens x 32 heads x 128 (adjacent pairing), residual add of two rows x 4096 tensors, softmax over
    128256 logits (N(0, 4)), and the fused residual add + RMSNorm.  64 rows is the configuration (mostly L2-resident
    sizes: each op cycles through enough distinct input sets to exceed the 126 MB L2), 1024 rows leaves L2 by itself.
    Bytes are the algorithmic ones: every input read once, every output written once."""
    import ctypes as C

    out = []
    for R in rows_list:
        g = torch.Generator(device="cuda")
        g.manual_seed(3)

        def rnd(*shape, sigma=1.0, mean=0.0):
            return torch.randn(shape, generator=g, device="cuda") * sigma + mean

        def copies_for(bytes_per_set):
            return max(2, int(160e6 // bytes_per_set) + 1)

        cases = []
        n = copies_for(2 * R * 4096 * 4)
        xs, w = [rnd(R, 4096) for _ in range(n)], rnd(4096, sigma=0.1, mean=1.0)
        outs = [torch.empty_like(x) for x in xs]
        cases.append(("rmsnorm", 2 * R * 4096 * 4 + 4096 * 4, n, lambda i: dev.rmsnorm(xs[i], w, 1e-6, out=outs[i])))
        n2 = copies_for(3 * R * 14336 * 4)
        gs, us = [rnd(R, 14336) for _ in range(n2)], [rnd(R, 14336) for _ in range(n2)]
        so = [torch.empty_like(x) for x in gs]
        cases.append(("swiglu", 3 * R * 14336 * 4, n2, lambda i: dev.swiglu(gs[i], us[i], out=so[i])))
        n3 = copies_for(2 * R * 32 * 128 * 4)
        cos, sin = dev.rope_tables(500000.0, 128, R)
        rs = [rnd(R, 32, 128) for _ in range(n3)]
        cases.append(("rope", 2 * R * 32 * 128 * 4 + 2 * R * 64 * 4, n3, lambda i: dev.rope(rs[i], 0, cos, sin, False)))
        n4 = copies_for(3 * R * 4096 * 4)
        ax, ay = [rnd(R, 4096) for _ in range(n4)], [rnd(R, 4096) for _ in range(n4)]
        cases.append(("add", 3 * R * 4096 * 4, n4, lambda i: dev.add_(ax[i], ay[i])))
        n5 = copies_for(2 * R * 128256 * 4)
        sx = [rnd(R, 128256, sigma=2.0) for _ in range(n5)]
        sy = [torch.empty_like(x) for x in sx]
        cases.append(("softmax", 2 * R * 128256 * 4, n5, lambda i: dev.softmax(sx[i], out=sy[i])))
        fo = [torch.empty_like(x) for x in ax]

        def fused(i):
            ctx.check(ctx.lib.smc_add_rmsnorm_dev(ctx.h, ax[i].data_ptr(), ay[i].data_ptr(), w.data_ptr(), fo[i].data_ptr(), R,
                                                  4096, C.c_float(1e-6), C.c_void_p(torch.cuda.current_stream().cuda_stream)))

        cases.append(("add+rmsnorm", 4 * R * 4096 * 4 + 4096 * 4, n4, fused))
        for name, nbytes, ncopies, fn in cases:
            if once:
                fn(0)
                torch.cuda.synchronize()
                continue

            def body(fn=fn, ncopies=ncopies):
                for i in range(ncopies):
                    fn(i)

            usec = time_graph_us(torch, body, ncopies, reps=reps)
            out.append({"op": name, "rows": R, "us_per_launch": round(usec, 2), "algorithmic_MB": round(nbytes / 1e6, 3),
                        "GBps": round(nbytes / usec / 1e3, 1), "frac_of_hbm_peak": round(nbytes / usec / 1e3 / peak, 3)})
        del cases, xs, outs, gs, us, so, rs, ax, ay, sx, sy, fo
        torch.cuda.empty_cache()
    return out


def prefill_section(torch, ctx, dev, ops, peaks: dict, n: int, k: int, layers: int, mp: int = 512) -> dict:
    """`mp` tokens through the tcgen05 tensor-core kernel on `layers` distinct Q4_K matrices [n, k]."""
    ws = [device_matrix(torch, dev, ctx, Q4_K, n, k, 900 + i) for i in range(layers)]
    xp = torch.from_numpy(np.random.default_rng(5).standard_normal((mp, k), dtype=np.float32)).cuda()
    op = torch.empty((mp, n), device="cuda", dtype=torch.float32)
    dev.qmatmul(xp, ws[0], ops.Mode.ACT_F32, out=op)  # first call sizes the scratch
    torch.cuda.synchronize()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for w in ws:
        dev.qmatmul(xp, w, ops.Mode.ACT_F32, out=op)
    t1.record()
    torch.cuda.synchronize()
    msp = t0.elapsed_time(t1) / layers
    tf = 2.0 * mp * n * k / msp / 1e9
    tpeak = float(peaks.get("bf16_tflops", 1590.0))
    for w in ws:
        ctx.release(w)
    return {"kernel": "prefill_q4k_kernel (tcgen05.mma kind::f16, fp16 integer weights x fp16 hi/lo activations)",
            "M": mp, "N": n, "K": k, "ms_per_matmul": msp, "useful_TFLOPs": tf, "tensor_TFLOPs_issued": 2 * tf,
            "peak_TFLOPs": tpeak, "frac_useful": tf / tpeak,
            "peak_source": "measured bf16 burst (MEASURED_PEAKS.json)" if "bf16_tflops" in peaks else "fallback"}


def run_only(args):
    import torch

    from sharpmind_b200 import ops, synth

    torch.cuda.set_device(0)
    ctx = ops.CudaContext(0)
    dev = ops.DeviceOps(ctx)
    peaks = load_peaks()
    peak = float(peaks.get("hbm_gbs", 6650.0))
    parts = args.only.split(":")
    mode = ops.Mode.ACT_Q8 if args.mode == "q8" else ops.Mode.ACT_F32
    if parts[0] == "gemv":
        M = int(parts[2]) if len(parts) > 2 else 1
        if len(parts) > 4 and parts[4] == "ring":  # 2..32 rows: weights through the bulk-copy ring (off by default)
            ctx.set_option("small_batch_ring", 2)
        res = time_gemv_shape(torch, ctx, dev, ops, parts[1], M, parts[3] if len(parts) > 3 else "q8", peak, once=args.no_graph)
    elif parts[0] == "decode":
        cfg = dict(synth.LLAMA3_8B if len(parts) > 1 and parts[1] == "llama8b" else synth.QWEN3_0_6B)
        if parts[-1] == "q8kv":
            cfg["kv_dtype"] = 8
        if args.layers:
            cfg["n_layers"] = args.layers
        res = {"decode": time_decode(torch, ctx, dev, cfg, [args.batch], 2048, max(args.steps, 4), mode, once=args.no_graph)}
    elif parts[0] == "prompt":
        cfg = dict(synth.LLAMA3_8B if len(parts) > 1 and parts[1] == "llama8b" else synth.QWEN3_0_6B)
        if args.layers:
            cfg["n_layers"] = args.layers
        res = {"prompt": time_prompt(torch, ctx, dev, cfg, 2048, args.chunk, mode)}
    elif parts[0] == "elementwise":
        res = {"elementwise": elementwise_chain(torch, ctx, dev, peak, once=args.no_graph)}
    elif parts[0] == "prefill":
        res = {"prefill": prefill_section(torch, ctx, dev, ops, peaks, 28672, 8192, 2)}
    else:
        raise SystemExit(f"unknown --only section '{args.only}'")
    print(json.dumps(res), flush=True)
    ctx.close()


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
    from sharpmind_b200 import ops, synth
    from sharpmind_b200.sharded import KSplit, PeerGather, RowSplit

    ctx = ops.CudaContext(local)
    dev = ops.DeviceOps(ctx)
    mode = ops.Mode.ACT_Q8 if args.mode == "q8" else ops.Mode.ACT_F32
    H, F, Ldef, _, desc = WORKLOADS[args.workload]
    L = args.layers or Ldef
    mats = matrices(args.workload)
    split = RowSplit(world, rank)
    peaks = load_peaks()
    peak = float(peaks.get("hbm_gbs", 6650.0))
    peak_src = "measured (MEASURED_PEAKS.json hbm_gbs)" if "hbm_gbs" in peaks else "fallback 6650 GB/s"

    def seed_of(layer, mi, r):
        return 1_000_003 * layer + 101 * mi + 7 * r + 1

    def rows_local_of(name, n):
        parts = 2 if name == "gate_up" else 1  # gate and up are split separately
        return split.rows(n // parts) * parts

    # N > 1 with one activation row: the feed-forward dataflow with ONE exchange per layer.  gate||up is split by rows
    # along whole K-steps of the down projection (its output stays on the rank, SiLU-gate included), down along K.
    tp_ffn = world > 1 and args.gather == "peer" and args.tp == "ffn" and args.batch == 1 and mode == ops.Mode.ACT_Q8
    ksplit = KSplit(world, rank, 2048)

    def local_shapes(r):
        """[(name, dtype, rows, K)] of rank r's slices."""
        if tp_ffn:
            f0, f1 = ksplit.k_range(F, r)
            return [("gate_up", mats[0][1], 2 * (f1 - f0), H), ("down", mats[1][1], H, f1 - f0)]
        return [(name, dt, rows_local_of(name, n), k) for (name, dt, n, k) in mats]

    lmats = local_shapes(rank)

    # ---- weights: generated and quantised on the device, one slice per rank
    weights = []
    for layer in range(L):
        weights.append([device_matrix(torch, dev, ctx, dt, n, k, seed_of(layer, mi, rank)) for mi, (name, dt, n, k) in enumerate(lmats)])
    torch.cuda.synchronize()

    def make_state(M):
        xs = [torch.from_numpy(np.random.default_rng(17 + i).standard_normal((M, k), dtype=np.float32)).cuda()
              for i, (_, _, _, k) in enumerate(lmats)]
        acts = [ops.Q8Act(ctx, M, k) for (_, _, _, k) in lmats]
        outs = [torch.empty((M, w.N), device="cuda", dtype=torch.float32) for w in weights[0]]
        gathered = [torch.empty((world, M, w.N), device="cuda", dtype=torch.float32) for w in weights[0]] if world > 1 else None
        return xs, acts, outs, gathered

    comm_stream = torch.cuda.Stream() if world > 1 else None
    peer = world > 1 and args.gather == "peer"
    gathers = {}

    def gather_for(M, mi):
        # one receive buffer per (batch, matrix): the exchange runs inside the GEMV kernel over peer memory
        if (M, mi) not in gathers:
            if args.no_exchange:
                gathers[(M, mi)] = PeerGather(ctx, RowSplit(1, 0), world * M * weights[0][mi].N, None)
            else:
                gathers[(M, mi)] = PeerGather(ctx, split, world * M * weights[0][mi].N, dist)
        return gathers[(M, mi)]

    def one_matmul(state, M, layer, mi, md):
        xs, acts, outs, gathered = state
        w = weights[layer][mi]
        if peer:
            return gather_for(M, mi).matmul(xs[mi], w, md)
        if md == ops.Mode.ACT_Q8 and M > 1:
            dev.quantize_q8(xs[mi], acts[mi], w.K)
            dev.qmatmul_q8(acts[mi], w, out=outs[mi])
        else:
            # one row: the Q8_0 quantisation of the activations happens inside the GEMV kernel
            dev.qmatmul(xs[mi], w, md, out=outs[mi])
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
            return gathered[mi]
        return outs[mi]

    def ffn_layer(state, layer, md, x=None):
        """gate||up on this rank's rows, then the K-split down projection (the SiLU-gate in its staging, or with
        --tp-pairs in the first matmul's epilogue) whose tail exchanges and adds the partial sums: two launches, one
        exchange.  Returns the [1, H] sums."""
        xs, _, outs, _ = state
        fl = weights[layer][1].K
        if args.tp_pairs:  # gate||up rows woven (gate i, up i), the SiLU-gate in the first matmul's epilogue
            act = outs[0][:, :fl]
            dev.qmatmul_swiglu_pairs(xs[0] if x is None else x, weights[layer][0], out=act)
            return gather_for(1, 1).matmul_reduce(act, weights[layer][1], md)
        dev.qmatmul(xs[0] if x is None else x, weights[layer][0], md, out=outs[0])  # [gate rows | up rows]
        return gather_for(1, 1).matmul_reduce(outs[0][0, :fl], weights[layer][1], md, up=outs[0][0, fl:])

    def step(state, M, md):
        for layer in range(L):
            if tp_ffn:
                ffn_layer(state, layer, md)
                continue
            for mi in range(len(mats)):
                one_matmul(state, M, layer, mi, md)

    def launches_per_step(M, md):
        if tp_ffn:
            return 2 * L
        # a single row is quantised inside the GEMV kernel; otherwise a quantiser launch precedes it
        per = sum(2 if (md == ops.Mode.ACT_Q8 and M > 1) else 1 for _ in mats)
        if peer and not (md == ops.Mode.ACT_Q8 and M == 1):
            per += len(mats)  # the exchange is a launch of its own unless it rides in the one-row GEMV's tail
        return L * per

    def timed(M, md, steps, warmup, use_graph, preload_s=0.0):
        state = make_state(M)
        runner = lambda: step(state, M, md)  # noqa: E731
        graphed = False
        if peer:
            for mi in ([1] if tp_ffn else range(len(mats))):
                gather_for(M, mi)  # created (and peers mapped) on every rank before anything is timed or captured
        if use_graph and (world == 1 or peer):
            runner = graph_of(torch, lambda: step(state, M, md)).replay
            graphed = True
        for _ in range(max(warmup, 3)):
            runner()
        torch.cuda.synchronize()
        # The timed region of a few steps lasts tens of milliseconds, too short for the clock sampler: the same step is
        # replayed (untimed) for `preload_s` first, so that the clocks and throttle reasons that are sampled are those
        # of the GPU under this very load.  The number of replays is fixed on rank 0 and broadcast.
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
        return ms / steps, graphed

    M = args.batch

    # ---- N > 1: a correctness fact before anything is timed.  Rank 0 regenerates every rank's slice of layer 0 from
    # its seed, computes it locally with the same kernel and compares the gathered buffer bit for bit (the one-row
    # kernel's sums do not depend on how rows are divided); every rank also checks its own chunk.
    parity = {"checked": False, "note": "single GPU: results are covered by the -m gpu parity tests"}
    if world > 1 and tp_ffn and not args.no_exchange:
        # layer 0 on every rank; rank 0 then regenerates EVERY rank's two slices from their seeds, forms each rank's
        # partial sums with the same kernels and adds them in rank order: the exchanged sums must equal that bit for
        # bit, and all ranks must hold the same bits
        state = make_state(1)
        got = ffn_layer(state, 0, mode).clone()
        torch.cuda.synchronize()
        ok = True
        if rank == 0:
            want = None
            for r in range(world):
                (_, dt_g, n_g, k_g), (_, dt_d, n_d, k_d) = local_shapes(r)
                wg = weights[0][0] if r == 0 else device_matrix(torch, dev, ctx, dt_g, n_g, k_g, seed_of(0, 0, r))
                wd = weights[0][1] if r == 0 else device_matrix(torch, dev, ctx, dt_d, n_d, k_d, seed_of(0, 1, r))
                gu = dev.qmatmul(state[0][0], wg, mode)
                if args.tp_pairs:  # rows woven: gate i, up i
                    part = dev.qmatmul(dev.swiglu(gu[:, 0::2].contiguous(), gu[:, 1::2].contiguous()), wd, mode)
                else:
                    part = dev.qmatmul(dev.swiglu(gu[:, :k_d].contiguous(), gu[:, k_d:].contiguous()), wd, mode)
                want = part.clone() if want is None else want + part
                if r:
                    ctx.release(wg), ctx.release(wd)
            ok = bool(torch.equal(got, want))
        digest = got.view(torch.int32).to(torch.int64).sum()
        lo, hi = digest.clone(), digest.clone()
        dist.all_reduce(lo, op=dist.ReduceOp.MIN), dist.all_reduce(hi, op=dist.ReduceOp.MAX)
        same = bool(lo.item() == hi.item())
        flag = torch.tensor([1 if (ok and same) else 0], device="cuda")
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        parity = {"checked": True, "ok": bool(flag.item()), "what": "layer 0 of the one-exchange feed-forward block: rank 0 recomputes "
                  "every rank's partial sums from the seeds of their slices and adds them in rank order; the exchanged sums "
                  "equal that bit for bit and every rank holds the same bits", "all_ranks_identical": same}
        del state
    elif world > 1 and not args.no_exchange:
        state = make_state(M)
        ok_all, detail = True, []
        for mi, (name, dt, n, k) in enumerate(mats):
            got = one_matmul(state, M, 0, mi, mode).clone()  # [world, M, N_local]
            torch.cuda.synchronize()
            mine = dev.qmatmul(state[0][mi], weights[0][mi], mode)
            ok_local = bool(torch.equal(got[rank], mine))
            ok = ok_local
            if rank == 0:
                for r in range(1, world):
                    wr = device_matrix(torch, dev, ctx, dt, rows_local_of(name, n), k, seed_of(0, mi, r))
                    ref = dev.qmatmul(state[0][mi], wr, mode)
                    same = bool(torch.equal(got[r], ref))
                    ok = ok and same
                    ctx.release(wr)
                    del ref
            flag = torch.tensor([1 if ok else 0], device="cuda")
            dist.all_reduce(flag, op=dist.ReduceOp.MIN)
            ok_all = ok_all and bool(flag.item())
            detail.append({"matrix": name, "ok": bool(flag.item())})
        parity = {"checked": True, "ok": ok_all, "what": "layer 0, every rank's slice recomputed on rank 0 from its seed and "
                  "compared bit for bit with the gathered buffer; each rank also compares its own chunk", "matrices": detail}
        del state

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    ms_step, graphed = timed(M, mode, args.steps, args.warmup, not args.no_graph, preload_s=1.2)
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
                       f"tp{world}: gate||up by rows (whole K-steps of down: {[b // 2048 for b in ksplit.bounds(F)]}), SiLU-gate "
                       f"local, down split along K, partial sums exchanged and added in rank order inside the GEMV kernel over "
                       f"NVLink peer memory: one exchange per layer" if tp_ffn else
                       f"row-split x{world}, slices exchanged by the GEMV kernel over NVLink peer memory" if peer
                       else f"row-split x{world} + NCCL all-gather")},
        "pct_of_8TBs_nominal": value / 8000.0 * 100.0 / world,
        "frac_of_measured_hbm_per_gpu": value / peak / world,
        "gpu_launches": launches_per_step(M, mode) * args.steps,
        "clocks": clocks,
        "parity": parity,
    }
    if args.no_exchange:
        result["invalid"] = "diagnosis run: partial sums were not exchanged"

    # ---- end to end: host buffers in, host buffers out, copies inside the timed region
    xs_h = [np.random.default_rng(17 + i).standard_normal((M, k), dtype=np.float32) for i, (_, _, _, k) in enumerate(mats)]
    e2e_steps = max(2, args.steps // 4)
    if world == 1:
        q = ops.QuantizationOps(ctx, mode)
        # the caller's rows live in page-locked host memory (numpy views of pinned tensors): the call copies from and to
        # them directly
        pins = [torch.from_numpy(x).pin_memory() for x in xs_h] + [torch.empty((M, n), dtype=torch.float32).pin_memory() for (_, _, n, _) in mats]
        xs_h = [t.numpy() for t in pins[:len(mats)]]
        outs_h = [t.numpy() for t in pins[len(mats):]]

        def e2e_step():
            for layer in range(L):
                for mi, (_, _, n_, k_) in enumerate(mats):
                    q.QuantizedMatMulHandle(xs_h[mi], weights[layer][mi], outs_h[mi], M, k_, n_)

        api = "smc_qmatmul_host_w: one synchronous C-ABI call per matmul, page-locked host fp32 rows in / out"
    elif tp_ffn:
        pin_x = torch.from_numpy(xs_h[0]).pin_memory()
        dev_x0 = torch.empty((1, H), device="cuda")
        pin_y = torch.empty((1, H), dtype=torch.float32).pin_memory()
        st_e = make_state(1)
        gather_for(1, 1)

        def e2e_step():
            for layer in range(L):
                dev_x0.copy_(pin_x, non_blocking=True)
                pin_y.copy_(ffn_layer(st_e, layer, mode, dev_x0), non_blocking=True)
                torch.cuda.current_stream().synchronize()  # the caller reads the block's output before its next call

        api = ("per layer: pinned host row -> device, gate||up on the rank's rows, smc_qmatmul_reduce_dev (SiLU-gate in the "
               "staging, K-split down, partial sums exchanged and added in the kernel), summed row -> pinned host, stream "
               "synchronised")
    else:
        pin_x = [torch.from_numpy(x).pin_memory() for x in xs_h]
        dev_x = [torch.empty((M, k), device="cuda") for (_, _, _, k) in mats]
        pin_o = [torch.empty((world, M, w.N), dtype=torch.float32).pin_memory() for w in weights[0]]
        for mi in range(len(mats)):
            if peer:
                gather_for(M, mi)
        st_e = make_state(M)

        def e2e_step():
            for layer in range(L):
                for mi in range(len(mats)):
                    dev_x[mi].copy_(pin_x[mi], non_blocking=True)
                    if peer:
                        got = gather_for(M, mi).matmul(dev_x[mi], weights[layer][mi], mode)
                    else:
                        st_e[0][mi].copy_(dev_x[mi])
                        got = one_matmul(st_e, M, layer, mi, mode)
                    pin_o[mi].copy_(got, non_blocking=True)
                    torch.cuda.current_stream().synchronize()  # the caller reads the result before its next call

        api = ("per matmul: pinned host row -> device, smc_qmatmul_gather_dev (row-split + in-kernel exchange), gathered "
               "row -> pinned host, stream synchronised")
    e2e_step()
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        e2e_step()
    torch.cuda.synchronize()
    el = (time.perf_counter() - t0) / e2e_steps
    if dist is not None:
        t = torch.tensor([el], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        el = float(t.item())
    result["e2e"] = {"value": step_bytes / el / 1e9, "unit": "GB/s", "ms_per_step": el * 1e3,
                     "h2d_bytes_per_step": (4 * H if tp_ffn else sum(4 * M * k for _, _, _, k in mats)) * L,
                     "d2h_bytes_per_step": (4 * H if tp_ffn else sum(4 * M * n for _, _, n, _ in mats)) * L, "api": api}

    if rank == 0 and not args.no_extras:
        # ---- every matrix of the workload alone over all layers; the roofline names the one with the largest share
        state = make_state(M)
        kern = {}
        for mi, (name, dt, n, k) in enumerate(lmats):
            if mode == ops.Mode.ACT_Q8 and M > 1:
                dev.quantize_q8(state[0][mi], state[1][mi], k)

            def alone(mi=mi):
                for layer in range(L):
                    if mode == ops.Mode.ACT_Q8 and M > 1:
                        dev.qmatmul_q8(state[1][mi], weights[layer][mi], out=state[2][mi])
                    else:
                        dev.qmatmul(state[0][mi], weights[layer][mi], mode, out=state[2][mi])

            us = time_graph_us(torch, alone, L)
            n_local = weights[0][mi].N
            kbytes = raw_bytes(dt, n_local, k) + 4 * M * k + 4 * M * n_local
            kern[name] = {"kernel": f"gemv_tma_kernel<{ {Q4_K: 'MathQ4K', Q6_K: 'MathQ6K', Q8_0: 'MathQ8_0'}[dt] }> ({name}, "
                                    f"{n_local}x{k})" if M == 1 and mode == ops.Mode.ACT_Q8 else f"{name} {n_local}x{k}",
                          "us": us, "algorithmic_bytes_per_launch": kbytes, "GBps": kbytes / us / 1e3,
                          "frac": kbytes / us / 1e3 / peak, "traffic": NCU_TRAFFIC_PER_ALGORITHMIC_BYTE.get(dt, 0) * kbytes or None}
        total_us = sum(v["us"] for v in kern.values())
        for v in kern.values():
            v["share_of_step"] = v["us"] / total_us
        dom = max(kern.values(), key=lambda v: v["us"])
        result["roofline"] = {"bound": "hbm", "kernel": dom["kernel"], "achieved": dom["GBps"], "peak": peak, "unit": "GB/s",
                              "frac": dom["frac"], "peak_source": peak_src, "us_per_launch": dom["us"],
                              "share_of_step": dom["share_of_step"],
                              "algorithmic_bytes_per_launch": dom["algorithmic_bytes_per_launch"], "traffic": dom["traffic"],
                              "traffic_source": "ncu dram__bytes_read + write of one launch of this kernel per algorithmic byte "
                                                "(summaries under profiles/), scaled to this launch's bytes"}
        result["kernels"] = kern
        del state

    if rank == 0 and world == 1 and not args.no_extras:
        for row in weights:
            for w in row:
                ctx.release(w)
        weights.clear()
        torch.cuda.empty_cache()
        extras = {}

        def guarded(name, fn):
            try:
                extras[name] = fn()
            except Exception as exc:  # an extra never takes the headline line down
                extras[name] = {"error": f"{type(exc).__name__}: {exc}"}
            torch.cuda.empty_cache()

        # ---- the other FFN stack (configs[1] when the headline is configs[4] and the other way round), with its
        # batch sweep in both fast modes
        other = "llama8b" if args.workload == "llama70b" else "llama70b"

        def other_stack():
            omats = matrices(other)
            oL = WORKLOADS[other][2] if other == "llama8b" else 12
            ow = [[device_matrix(torch, dev, ctx, dt, n, k, 7_000_003 * layer + 11 * mi + 1) for mi, (_, dt, n, k) in enumerate(omats)]
                  for layer in range(oL)]
            res = {"workload": WORKLOADS[other][4], "layers_timed": oL}
            sweep, kerns = {}, {}
            for m2 in (1, 8, 32):
                for md, label in ((ops.Mode.ACT_Q8, "q8"), (ops.Mode.ACT_F32, "f32")):
                    if md == ops.Mode.ACT_F32 and m2 > 8:
                        continue  # CUDA-core bound by construction; not a bandwidth number
                    xs = [torch.from_numpy(np.random.default_rng(170 + i).standard_normal((m2, k), dtype=np.float32)).cuda()
                          for i, (_, _, _, k) in enumerate(omats)]
                    os_ = [torch.empty((m2, n), device="cuda") for (_, _, n, _) in omats]

                    def st():
                        for row in ow:
                            for mi, w in enumerate(row):
                                dev.qmatmul(xs[mi], w, md, out=os_[mi])

                    us = time_graph_us(torch, st, 1, reps=max(2, args.steps // 2))
                    sweep[f"{label}_b{m2}"] = algorithmic_bytes(omats, m2) * oL / us / 1e3
                    if m2 == 1 and md == ops.Mode.ACT_Q8:
                        res["ms_per_step"] = us / 1e3
                        for mi, (name, dt, n, k) in enumerate(omats):
                            def alone(mi=mi):
                                for row in ow:
                                    dev.qmatmul(xs[mi], row[mi], md, out=os_[mi])
                            u1 = time_graph_us(torch, alone, oL)
                            b1 = raw_bytes(dt, n, k) + 4 * k + 4 * n
                            kerns[name] = {"us": u1, "GBps": b1 / u1 / 1e3, "frac": b1 / u1 / 1e3 / peak}
            res["GBps"] = sweep["q8_b1"]
            res["frac_of_measured_hbm"] = sweep["q8_b1"] / peak
            res["sweep_GBps"] = sweep
            res["kernels"] = kerns
            for row in ow:
                for w in row:
                    ctx.release(w)
            return res

        guarded("stack_" + other, other_stack)

        # ---- configs[0]: Q8_0 3072x1024 (latency-bound: 3.36 MB per launch) and the LM-head GEMV as the Q8_0 bandwidth witness
        def config0():
            r = {}
            for which in ("q8", "lmhead"):
                t = time_gemv_shape(torch, ctx, dev, ops, which, 1, "q8", peak)
                r[which] = {k: t[k] for k in ("N", "K", "copies", "us_per_launch", "algorithmic_bytes", "GBps", "frac_of_hbm_peak")}
            r["note"] = ("q8 = configs[0] Q8_0 3072x1024, 48 distinct copies (160 MB) cycled in a CUDA graph so that no launch "
                         "finds its matrix in L2; lmhead = 151936x1024 Q8_0, the largest Q8_0 GEMV of configs[3]")
            return r

        guarded("config0_q8_0", config0)
        # ---- configs[2]: the fp32 elementwise / reduction chain
        guarded("config2_elementwise", lambda: elementwise_chain(torch, ctx, dev, peak))
        # ---- prefill-sized batch on the tcgen05 tensor-core kernel (512 tokens, Llama-3-70B gate/up shape)
        guarded("prefill", lambda: prefill_section(torch, ctx, dev, ops, peaks, 28672, 8192, 4))

        # ---- the other half of the metric: decode tokens/s of the Qwen3-0.6B-shaped model (configs[3])
        def decode():
            rows = time_decode(torch, ctx, dev, dict(synth.QWEN3_0_6B), [1, 32], 2048, 16, ops.Mode.ACT_Q8)
            d = {"workload": "configs[3] Qwen3-0.6B-shaped decoder, Q8_0 weights, fp32 KV with a 2048-position seeded random "
                             "context, one greedy token per sequence per step, q8_0 activations, CUDA graph",
                 "tokens_per_s_batch1": rows[0]["tokens_per_s"], "ms_per_step_batch1": rows[0]["ms_per_step"],
                 "tokens_per_s_batch32": rows[1]["tokens_per_s"], "ms_per_step_batch32": rows[1]["ms_per_step"],
                 "GBps_batch1": rows[0]["GBps"], "GBps_batch32": rows[1]["GBps"]}
            q8kv = time_decode(torch, ctx, dev, dict(synth.QWEN3_0_6B, kv_dtype=8), [1, 32], 2048, 16, ops.Mode.ACT_Q8)
            prq8 = time_prompt(torch, ctx, dev, dict(synth.QWEN3_0_6B, kv_dtype=8), 2048, 2048, ops.Mode.ACT_Q8, 2)
            d["q8_0_kv"] = {"prompt_pass_tokens_per_s": prq8["tokens_per_s"],
                            "what": "the same steps over a Q8_0 KV cache (QuantizedKVCache rows)",
                            "tokens_per_s_batch1": q8kv[0]["tokens_per_s"], "tokens_per_s_batch32": q8kv[1]["tokens_per_s"],
                            "kv_MB_batch32": q8kv[1]["kv_MB"], "GBps_batch32": q8kv[1]["GBps"]}
            pr = time_prompt(torch, ctx, dev, dict(synth.QWEN3_0_6B), 2048, 2048, ops.Mode.ACT_Q8, 2)
            pr1k = time_prompt(torch, ctx, dev, dict(synth.QWEN3_0_6B), 2048, 1024, ops.Mode.ACT_Q8, 2)
            d["prompt_pass"] = {"what": "ForwardLastLogits over a 2048-token seeded prompt in one call (as the reference runs it), one sequence",
                                "ms": pr["ms"], "tokens_per_s": pr["tokens_per_s"],
                                "in_chunks_of_1024": {"ms": pr1k["ms"], "tokens_per_s": pr1k["tokens_per_s"]}}
            return d

        guarded("decode", decode)

        def decode8b():
            rows8 = time_decode(torch, ctx, dev, dict(synth.LLAMA3_8B), [1, 32], 2048, 8, ops.Mode.ACT_Q8)
            pr8 = time_prompt(torch, ctx, dev, dict(synth.LLAMA3_8B), 2048, 2048, ops.Mode.ACT_Q8, 2)
            return {"prompt_pass": {"what": "ForwardLastLogits over a 2048-token seeded prompt in one call (Q4_K matmuls on tcgen05 over "
                                            "the Q8_0 activation rows, Q6_K down on int8 mma.sync)",
                                    "ms": pr8["ms"], "tokens_per_s": pr8["tokens_per_s"]},
                    "workload": "Llama-3-8B-shaped decoder: Q4_K attention and gate||up, Q6_K down, Q8_0 tied embedding, fp32 KV, "
                                "2048-position seeded random context, q8_0 activations, CUDA graph",
                    "tokens_per_s_batch1": rows8[0]["tokens_per_s"], "ms_per_step_batch1": rows8[0]["ms_per_step"],
                    "tokens_per_s_batch32": rows8[1]["tokens_per_s"], "ms_per_step_batch32": rows8[1]["ms_per_step"],
                    "GBps_batch1": rows8[0]["GBps"], "GBps_batch32": rows8[1]["GBps"]}

        guarded("decode_llama8b", decode8b)
        result.update(extras)
        # ---- CPU baseline on the host cores
        try:
            result["cpu_baseline"] = cpu_port_time(args.workload, M, args.cpu_seconds)
        except Exception as exc:  # the baseline is reported, never required
            result["cpu_baseline"] = {"value": None, "unit": "GB/s", "cores": None, "kind": "port", "sample": f"failed: {exc}"}
    if rank == 0:
        print(json.dumps(result), flush=True)
    for g in gathers.values():
        g.close()
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()
    ctx.close()


def main():
    args = parse()
    if args.impl == "reference":
        run_reference(args)
    elif args.only:
        run_only(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
