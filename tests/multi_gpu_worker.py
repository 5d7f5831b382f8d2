"""Worker of the multi-GPU parity test: run under torch.distributed.run, one process per GPU.

Every rank quantises the same seeded matrix on its own GPU, keeps its row slice, and checks that the row-split
matmul with the in-kernel peer exchange reproduces the unsplit matmul of the same library bit for bit (each
output row is computed by the same kernel arithmetic whichever rank owns it), for the fused one-row path, the
several-row path, repeated exchanges, two objects in alternation, and a replayed CUDA graph.

Then the one-exchange feed-forward block: gate||up split by rows, SwiGLU local, down split along K with the partial
sums exchanged and added in rank order inside the producing kernel.  Every rank can form every rank's partial on its
own GPU with the same kernel (a row's bits do not depend on the grid), so the sum is checked bit for bit against the
rank-ordered sum of those, and within the parity bound against the unsplit block (summation order is all that differs).
"""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from sharpmind_b200 import ops, synth  # noqa: E402
from sharpmind_b200.sharded import KSplit, PeerGather, RowSplit, ShardedLinear  # noqa: E402


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    ctx = ops.CudaContext(local)
    dev = ops.DeviceOps(ctx)
    split = RowSplit(world, rank)
    failures = []
    for dtype, n, k in ((12, 4096, 4096), (14, 2048, 4096), (8, 3072, 1024), (12, 1024, 16384)):
        wf = torch.from_numpy(synth.normal("multi", f"w{dtype}_{k}", (n, k), 0.02)).cuda()
        raw = dev.quantize_weights(dtype, wf)
        full = ctx.register_dev(raw, dtype, n, k)
        part = ctx.register_dev(split.slice_raw(raw, dtype, n, k).contiguous(), dtype, n // world, k)
        lin = ShardedLinear(split, n, None, dist)
        ga = PeerGather(ctx, split, 8 * n, dist)
        gb = PeerGather(ctx, split, 8 * n, dist)
        for m in (1, 4, 8):
            for it in range(6):
                x = torch.from_numpy(synth.normal("multi", f"x{dtype}_{m}_{it}", (m, k))).cuda()
                want = dev.qmatmul(x, full, ops.Mode.ACT_Q8)
                g = ga if it % 2 == 0 else gb
                got = lin.assemble(g.matmul(x, part, ops.Mode.ACT_Q8))
                if not torch.equal(got, want):
                    failures.append(f"dtype {dtype} M {m} iteration {it}: max diff {(got - want).abs().max().item()}")
        # a slice of a megabyte or more goes as bulk stores + one flag instead of packets
        if dtype == 12 and k == 4096:
            m = 128 * world
            big = PeerGather(ctx, split, world * m * (n // world), dist)
            for it in range(3):
                x = torch.from_numpy(synth.normal("multi", f"xb{it}", (m, k))).cuda()
                want = dev.qmatmul(x, full, ops.Mode.ACT_Q8)
                got = lin.assemble(big.matmul(x, part, ops.Mode.ACT_Q8))
                if not torch.equal(got, want):
                    failures.append(f"bulk exchange iteration {it}: max diff {(got - want).abs().max().item()}")
                # alternate with a small (packet) exchange on the same object
                x1 = torch.from_numpy(synth.normal("multi", f"xs{it}", (1, k))).cuda()
                if not torch.equal(lin.assemble(big.matmul(x1, part, ops.Mode.ACT_Q8)), dev.qmatmul(x1, full, ops.Mode.ACT_Q8)):
                    failures.append(f"packet exchange after bulk, iteration {it}")
            dist.barrier()
            big.close()
        # replayed graph: the exchange counter lives in device memory, so replays stay in step
        x = torch.from_numpy(synth.normal("multi", f"xg{dtype}", (1, k))).cuda()
        want = dev.qmatmul(x, full, ops.Mode.ACT_Q8)
        side = torch.cuda.Stream()
        with torch.cuda.stream(side):
            ga.matmul(x, part, ops.Mode.ACT_Q8)
            side.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                for _ in range(3):
                    view = ga.matmul(x, part, ops.Mode.ACT_Q8)
        torch.cuda.synchronize()
        dist.barrier()
        for _ in range(5):
            graph.replay()
        torch.cuda.synchronize()
        if not torch.equal(lin.assemble(view), want):
            failures.append(f"dtype {dtype}: graph replay differs")
        dist.barrier()
        ga.close(), gb.close()
    # ---- feed-forward block with one exchange (K-split down projection)
    for down_dt, H, F in ((12, 2048, 16384), (14, 1024, 16384)):
        ks = KSplit(world, rank)
        wgu = dev.quantize_weights(12, torch.from_numpy(synth.normal("multi", f"ffn_gu{H}", (2 * F, H), 0.03)).cuda())
        wdn = dev.quantize_weights(down_dt, torch.from_numpy(synth.normal("multi", f"ffn_dn{H}", (H, F), 0.03)).cuda())
        full_gu, full_dn = ctx.register_dev(wgu, 12, 2 * F, H), ctx.register_dev(wdn, down_dt, H, F)
        gu_parts, dn_parts = [], []
        for r in range(world):
            f0, f1 = ks.k_range(F, r)
            gu_parts.append(ctx.register_dev(ks.slice_fused_rows_raw(wgu, 12, F, H, r).contiguous(), 12, 2 * (f1 - f0), H))
            if r == rank:  # the same rows woven (gate i, up i) for the matmul with the SiLU-gate in its epilogue
                gu_woven = ctx.register_dev(ks.slice_fused_rows_raw(wgu, 12, F, H, r, interleave=True).contiguous(), 12, 2 * (f1 - f0), H)
            dn_parts.append(ctx.register_dev(ks.slice_columns_raw(wdn, down_dt, H, F, r), down_dt, H, f1 - f0))
        red = PeerGather(ctx, split, world * 4 * H, dist)
        for m in (1, 1, 1, 4):
            x = torch.from_numpy(synth.normal("multi", f"ffn_x{H}_{m}", (m, H))).cuda()
            # what every rank's partial is, formed locally, and their sum in rank order
            want = None
            for r in range(world):
                fl = dn_parts[r].K
                gu = dev.qmatmul(x, gu_parts[r], ops.Mode.ACT_Q8)
                act = dev.swiglu(gu[:, :fl].contiguous(), gu[:, fl:].contiguous())
                p = dev.qmatmul(act, dn_parts[r], ops.Mode.ACT_Q8)
                want = p.clone() if want is None else want + p
            fl = dn_parts[rank].K
            gu = dev.qmatmul(x, gu_parts[rank], ops.Mode.ACT_Q8)
            if m == 1:  # the SiLU-gate rides in the staging of the K-split matmul: one kernel per projection
                got = red.matmul_reduce(gu[0, :fl], dn_parts[rank], ops.Mode.ACT_Q8, up=gu[0, fl:]).clone()
            else:
                act = dev.swiglu(gu[:, :fl].contiguous(), gu[:, fl:].contiguous())
                got = red.matmul_reduce(act, dn_parts[rank], ops.Mode.ACT_Q8).clone()
            if not torch.equal(got, want):
                failures.append(f"ffn H {H} M {m}: differs from the rank-ordered sum by {(got - want).abs().max().item()}")
            if m == 1 and H % 2048 == 0:  # the other one-row form (rows of whole 2048-element steps): SiLU-gate in the first matmul's epilogue, a plain row into the K-split matmul
                act = dev.qmatmul_swiglu_pairs(x, gu_woven)
                got2 = red.matmul_reduce(act, dn_parts[rank], ops.Mode.ACT_Q8).clone()
                if not torch.equal(got2, want):
                    failures.append(f"ffn H {H}: woven gate/up form differs by {(got2 - want).abs().max().item()}")
            gu_f = dev.qmatmul(x, full_gu, ops.Mode.ACT_Q8)
            unsplit = dev.qmatmul(dev.swiglu(gu_f[:, :F].contiguous(), gu_f[:, F:].contiguous()), full_dn, ops.Mode.ACT_Q8)
            # each rank quantises its slice of the activation row with per-block scales, as the unsplit row does: the
            # integer sums are the same, only the fp32 additions are grouped per rank
            if (got - unsplit).abs().max().item() > 1e-5 * unsplit.abs().max().item():
                failures.append(f"ffn H {H} M {m}: {((got - unsplit).abs().max() / unsplit.abs().max()).item():.2e} from the unsplit block")
            # every rank must hold the same bits
            mine = got.view(torch.int32).sum(dtype=torch.int64)
            lo, hi = mine.clone(), mine.clone()
            dist.all_reduce(lo, op=dist.ReduceOp.MIN), dist.all_reduce(hi, op=dist.ReduceOp.MAX)
            if lo.item() != hi.item():
                failures.append(f"ffn H {H} M {m}: ranks hold different sums")
        dist.barrier()
        red.close()
    status = ctx.device_status()
    if status:
        failures.append(f"device status {status}")
    flag = torch.tensor([len(failures)], device="cuda")
    dist.all_reduce(flag)
    if failures:
        print(f"rank {rank}: " + "; ".join(failures[:5]), flush=True)
    dist.barrier()
    dist.destroy_process_group()
    ctx.close()
    sys.exit(1 if flag.item() else 0)


if __name__ == "__main__":
    main()
