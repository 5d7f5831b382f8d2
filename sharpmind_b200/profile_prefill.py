"""Times the tensor-core (tcgen05) Q4_K matmul on the Llama-3-70B FFN shapes at prefill batch sizes.

    python -m sharpmind_b200.profile_prefill [--m 512] [--shape up|down|8b] [--copies 3] [--reps 10] [--once]

Weights are seeded normal(0, 0.02) values quantised on the device; `copies` distinct matrices are cycled so
that the weights of a launch are not in L2 from the previous one.  Prints useful TFLOP/s = 2 M N K / time
(the hi/lo activation split doubles the tensor-core work; that factor is not counted).
"""
from __future__ import annotations

import argparse
import json

from . import ops

SHAPES = {"up": (28672, 8192), "down": (8192, 28672), "8b": (28672, 4096)}


def main():
    import torch

    ap = argparse.ArgumentParser()
    ap.add_argument("--m", type=int, default=512)
    ap.add_argument("--shape", default="up", choices=sorted(SHAPES))
    ap.add_argument("--copies", type=int, default=3)
    ap.add_argument("--reps", type=int, default=10)
    ap.add_argument("--once", action="store_true")
    a = ap.parse_args()
    n, k = SHAPES[a.shape]
    ctx = ops.CudaContext(0)
    dev = ops.DeviceOps(ctx)
    g = torch.Generator(device="cuda")
    g.manual_seed(5)
    ws = []
    for _ in range(a.copies):
        raw = dev.quantize_weights(12, torch.randn((n, k), generator=g, device="cuda") * 0.02)
        ws.append(ctx.register_dev(raw, 12, n, k))
        del raw
    x = torch.randn((a.m, k), generator=g, device="cuda")
    out = torch.empty((a.m, n), device="cuda")
    dev.qmatmul_tc(x, ws[0], out=out)  # allocates the scratch
    torch.cuda.synchronize()
    if a.once:
        dev.qmatmul_tc(x, ws[-1], out=out)
        torch.cuda.synchronize()
        ctx.close()
        return
    for w in ws:
        dev.qmatmul_tc(x, w, out=out)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(a.reps):
        for w in ws:
            dev.qmatmul_tc(x, w, out=out)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / (a.reps * len(ws))
    flops = 2.0 * a.m * n * k
    print(json.dumps({"shape": [n, k], "M": a.m, "ms_per_matmul": round(ms, 4),
                      "useful_TFLOPs": round(flops / ms / 1e9, 1),
                      "weight_GBps": round(n * k / 256 * 144 / ms / 1e6, 1), "device_status": ctx.device_status()}), flush=True)
    ctx.close()


if __name__ == "__main__":
    main()
