"""Times the fp32 elementwise / reduction ops of the decoder at the sizes of the fused-chain configuration.

    python -m sharpmind_b200.profile_elementwise [--rows-scale 1] [--reps 20] [--once]

RMSNorm over hidden 4096 for 64 rows (eps 1e-6, weight N(1, 0.1)), SiLU(gate)*up on 64 x 14336, RoPE theta
500000 on 64 tokens x 32 heads x 128 (adjacent pairing, positions 0..63), residual add of two 64 x 4096 tensors,
softmax over 128256 logits for 64 rows (N(0, 4)), and the fused residual add + RMSNorm.  At these sizes most
tensors fit the 126 MB L2, so each op cycles through `copies` distinct input sets sized to exceed it, and
`--rows-scale 16` runs 16x the rows.  Bytes are the algorithmic ones: every input read once, every output written
once.  Timing: CUDA graph of one pass over all copies, replayed `reps` times, CUDA events.
"""
from __future__ import annotations

import argparse
import json

from . import ops


def main():
    import torch

    ap = argparse.ArgumentParser()
    ap.add_argument("--rows-scale", type=int, default=1)
    ap.add_argument("--reps", type=int, default=20)
    ap.add_argument("--once", action="store_true")
    a = ap.parse_args()
    R = 64 * a.rows_scale
    ctx = ops.CudaContext(0)
    dev = ops.DeviceOps(ctx)
    g = torch.Generator(device="cuda")
    g.manual_seed(3)

    def rnd(*shape, sigma=1.0, mean=0.0):
        return torch.randn(shape, generator=g, device="cuda") * sigma + mean

    def copies_for(bytes_per_set):
        return max(2, int(160e6 // bytes_per_set) + 1)

    cases = []
    # RMSNorm
    n = copies_for(2 * R * 4096 * 4)
    xs, w = [rnd(R, 4096) for _ in range(n)], rnd(4096, sigma=0.1, mean=1.0)
    outs = [torch.empty_like(x) for x in xs]
    cases.append(("rmsnorm 64x4096", 2 * R * 4096 * 4 + 4096 * 4, n, lambda i: dev.rmsnorm(xs[i], w, 1e-6, out=outs[i])))
    # SwiGLU
    n2 = copies_for(3 * R * 14336 * 4)
    gs, us = [rnd(R, 14336) for _ in range(n2)], [rnd(R, 14336) for _ in range(n2)]
    so = [torch.empty_like(x) for x in gs]
    cases.append(("swiglu 64x14336", 3 * R * 14336 * 4, n2, lambda i: dev.swiglu(gs[i], us[i], out=so[i])))
    # RoPE (in place)
    n3 = copies_for(2 * R * 32 * 128 * 4)
    cos, sin = dev.rope_tables(500000.0, 128, R)
    rs = [rnd(R, 32, 128) for _ in range(n3)]
    cases.append(("rope 64x32x128", 2 * R * 32 * 128 * 4 + 2 * R * 64 * 4, n3, lambda i: dev.rope(rs[i], 0, cos, sin, False)))
    # residual add (in place)
    n4 = copies_for(3 * R * 4096 * 4)
    ax, ay = [rnd(R, 4096) for _ in range(n4)], [rnd(R, 4096) for _ in range(n4)]
    cases.append(("add 64x4096", 3 * R * 4096 * 4, n4, lambda i: dev.add_(ax[i], ay[i])))
    # softmax
    n5 = copies_for(2 * R * 128256 * 4)
    sx = [rnd(R, 128256, sigma=2.0) for _ in range(n5)]
    sy = [torch.empty_like(x) for x in sx]
    cases.append(("softmax 64x128256", 2 * R * 128256 * 4, n5, lambda i: dev.softmax(sx[i], out=sy[i])))
    # fused residual add + RMSNorm (x read and written, y read, out written)
    import ctypes as C

    fo = [torch.empty_like(x) for x in ax]

    def fused(i):
        ctx.check(ctx.lib.smc_add_rmsnorm_dev(ctx.h, ax[i].data_ptr(), ay[i].data_ptr(), w.data_ptr(), fo[i].data_ptr(), R, 4096,
                                              C.c_float(1e-6), C.c_void_p(torch.cuda.current_stream().cuda_stream)))

    cases.append(("add+rmsnorm 64x4096", 4 * R * 4096 * 4 + 4096 * 4, n4, fused))

    for name, nbytes, ncopies, fn in cases:
        if a.once:
            fn(0)
            torch.cuda.synchronize()
            continue
        side = torch.cuda.Stream()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            for i in range(ncopies):
                fn(i)
            side.synchronize()
            with torch.cuda.graph(graph, stream=side):
                for i in range(ncopies):
                    fn(i)
        torch.cuda.synchronize()
        graph.replay()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(a.reps):
            graph.replay()
        e1.record()
        torch.cuda.synchronize()
        usec = e0.elapsed_time(e1) * 1e3 / (a.reps * ncopies)
        print(json.dumps({"op": name.replace("64x", f"{R}x"), "us_per_launch": round(usec, 2), "algorithmic_MB": round(nbytes / 1e6, 3),
                          "GBps": round(nbytes / usec / 1e3, 1), "copies": ncopies}), flush=True)
    ctx.close()


if __name__ == "__main__":
    main()
