"""Small driver for timing / profiling one decode GEMV shape over a few distinct weight matrices.

    python -m sharpmind_b200.profile_gemv {q4k|q6k|q8|lmhead|q4k70|wo|q6k70|wo70} [M] [q8|q8f|f32]

q4k = Llama-3-8B gate||up 28672x4096 Q4_K, q6k = down 4096x14336 Q6_K, q8 = Qwen3-0.6B gate||up 6144x1024 Q8_0,
lmhead = 151936x1024 Q8_0, q4k70 = Llama-3-70B gate||up 57344x8192 Q4_K, wo = 8B attention output 4096x4096 Q4_K,
q6k70 = 70B down 8192x28672 Q6_K, wo70 = 70B attention output 8192x8192 Q4_K.  Modes: q8 = activations quantised by a
separate launch, q8f = smc_qmatmul_dev(SMC_ACT_Q8) as callers use it (one row is quantised inside the kernel),
f32 = fp32 activations.  The matrices (more than the 126 MB L2 in total) are cycled inside a CUDA graph and
timed with CUDA events; under `ncu -k regex:gemv_` the same launches are what gets captured.
"""
import sys

import torch

from sharpmind_b200 import ops

SHAPES = {"q4k": (12, 28672, 4096, 5), "q6k": (14, 4096, 14336, 5), "q8": (8, 6144, 1024, 40),
          "lmhead": (8, 151936, 1024, 3), "q4k70": (12, 57344, 8192, 3), "wo": (12, 4096, 4096, 20),
          "q6k70": (14, 8192, 28672, 2), "wo70": (12, 8192, 8192, 5)}
BLOCK = {8: (32, 34), 12: (256, 144), 14: (256, 210)}


def main():
    which = sys.argv[1] if len(sys.argv) > 1 else "q4k"
    M = int(sys.argv[2]) if len(sys.argv) > 2 else 1
    mode = sys.argv[3] if len(sys.argv) > 3 else "q8f"
    ctx = ops.CudaContext(0)
    dev = ops.DeviceOps(ctx)
    dt, n, k, L = SHAPES[which]
    ws = []
    for layer in range(L):
        g = torch.Generator(device="cuda").manual_seed(layer + 1)
        wf = torch.randn((n, k), generator=g, device="cuda") * 0.02
        ws.append(ctx.register_dev(dev.quantize_weights(dt, wf), dt, n, k))
        del wf
    x = torch.randn((M, k), device="cuda")
    act = ops.Q8Act(ctx, M, k)
    out = torch.empty((M, n), device="cuda")
    dev.quantize_q8(x, act, k)

    def body():
        for w in ws:
            if mode == "q8":
                dev.qmatmul_q8(act, w, out=out)
            elif mode == "q8f":
                dev.qmatmul(x, w, ops.Mode.ACT_Q8, out=out)
            else:
                dev.qmatmul(x, w, ops.Mode.ACT_F32, out=out)

    body()
    torch.cuda.synchronize()
    st = torch.cuda.Stream()
    st.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(st):
        body()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        body()
    for _ in range(3):
        g.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    reps = 5
    e0.record()
    for _ in range(reps):
        g.replay()
    e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / (L * reps)
    be, bb = BLOCK[dt]
    nbytes = n * k // be * bb + 4 * M * k + 4 * M * n
    print(f"{which} M={M} {mode}: {us:.2f} us/launch, {nbytes / us / 1e3:.0f} GB/s "
          f"({nbytes / us / 1e3 / 6520.5 * 100:.1f}% of the measured 6520.5 GB/s)")
    assert ctx.device_status() == 0
    ctx.close()


if __name__ == "__main__":
    main()
