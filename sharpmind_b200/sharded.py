"""Row-split quantized matmul across the GPUs of one node.

Output rows are independent (out[:, c] depends only on weight row c), so each rank keeps rows
[rank*N/G, (rank+1)*N/G) of every matrix, uploaded once, computes its output slice with the same
single-GPU kernels and one all-gather (NCCL over NVLink) reassembles [M, N].  Activations are
replicated.  A split point must fall on a block boundary of the flat tensor: (N/G)*K must be a
multiple of the format's block size, otherwise the slice would start inside a block.

The fused gate||up matrix is split per half (each rank holds its gate rows followed by its up rows)
so that SwiGLU can run on local data; `gather_fused` restores the [gate | up] column order.

The reference has no multi-device path (single process, single accelerator); this is the exchange
step the row-split adds, and the only collective on the path.
"""
from __future__ import annotations

from dataclasses import dataclass

BLOCK_ELEMS = {8: 32, 12: 256, 14: 256}


@dataclass(frozen=True)
class RowSplit:
    world: int
    rank: int

    def rows(self, n: int) -> int:
        if n % self.world:
            raise ValueError(f"{n} rows do not split evenly over {self.world} ranks")
        return n // self.world

    def row_range(self, n: int) -> tuple[int, int]:
        r = self.rows(n)
        return self.rank * r, (self.rank + 1) * r

    def check_block_aligned(self, dtype: int, n: int, k: int) -> None:
        be = BLOCK_ELEMS[int(dtype)]
        if int(dtype) == 8:
            if k % be:
                raise ValueError("Q8_0 rows must be whole blocks to be split")
        elif (self.rows(n) * k) % be:
            raise ValueError(f"a slice of {self.rows(n)} rows x K={k} does not end on a {be}-element block boundary")

    def slice_raw(self, raw, dtype: int, n: int, k: int):
        """The bytes of this rank's rows out of a whole GGUF-layout tensor (numpy or torch uint8)."""
        self.check_block_aligned(dtype, n, k)
        per_row = raw.shape[0] // n
        if per_row * n != raw.shape[0]:
            raise ValueError("tensor bytes are not a whole number of rows")
        r0, r1 = self.row_range(n)
        return raw[r0 * per_row:r1 * per_row]

    def slice_fused_raw(self, raw, dtype: int, n_half: int, k: int):
        """gate||up [2*n_half, k]: this rank's gate rows followed by its up rows."""
        self.check_block_aligned(dtype, n_half, k)
        per_row = raw.shape[0] // (2 * n_half)
        r0, r1 = self.row_range(n_half)
        gate = raw[r0 * per_row:r1 * per_row]
        up = raw[(n_half + r0) * per_row:(n_half + r1) * per_row]
        import numpy as np

        if isinstance(raw, np.ndarray):
            return np.concatenate([gate, up])
        import torch

        return torch.cat([gate, up])


class ShardedLinear:
    """One row-split matmul: local compute + all-gather.

    `compute(x) -> [M, N_local]` is the local matmul (the CUDA kernels in the product; the CPU
    tests of the exchange logic inject their own).  `dist` is torch.distributed with an initialised
    process group (nccl on GPUs, gloo on CPU).
    """

    def __init__(self, split: RowSplit, n: int, compute, dist=None, fused_halves: int = 1):
        self.split, self.n, self.compute, self.dist, self.halves = split, n, compute, dist, fused_halves
        self.n_local = split.rows(n // fused_halves) * fused_halves

    def forward(self, x, out=None):
        import torch

        local = self.compute(x)  # [M, n_local]
        m = local.shape[0]
        if self.split.world == 1:
            return local
        gathered = torch.empty((self.split.world, m, self.n_local), dtype=local.dtype, device=local.device)
        # the flat [G*M, n_local] view is the shape every backend accepts
        self.dist.all_gather_into_tensor(gathered.view(self.split.world * m, self.n_local), local.contiguous())
        return self.assemble(gathered, out)

    def assemble(self, gathered, out=None):
        """[G, M, n_local] -> [M, N] in the unsplit column order."""
        import torch

        g, m, nl = gathered.shape
        if self.halves == 1:
            res = gathered.permute(1, 0, 2).reshape(m, g * nl)
        else:
            h = nl // self.halves
            # per rank: [half0 rows | half1 rows]; wanted: all half0 columns, then all half1 columns
            res = gathered.reshape(g, m, self.halves, h).permute(1, 2, 0, 3).reshape(m, self.halves * g * h)
        if out is not None:
            out.copy_(res)
            return out
        return res.contiguous() if not res.is_contiguous() else res


class PeerGather:
    """Row-split matmul whose exchange runs inside the producing kernel over peer memory (no collective).

    Wraps the library's gather object: allocates this rank's receive buffer, swaps the CUDA IPC handles with
    one `all_gather_object` on `dist` (any backend: only 64 bytes per rank travel) and maps the peers.
    `matmul(x, w_local)` returns a [world, M, N_local] view of the receive buffer, valid until the next
    exchange on this object; `ShardedLinear.assemble` puts it into the unsplit column order.
    """

    def __init__(self, ctx, split: RowSplit, capacity_floats: int, dist=None):
        import ctypes as C

        import torch

        self.ctx, self.split, self.torch, self.C, self.dist = ctx, split, torch, C, dist
        self.capacity = int(capacity_floats)
        h = C.c_void_p()
        ctx.check(ctx.lib.smc_gather_create(ctx.h, split.rank, split.world, self.capacity, C.byref(h)))
        self.h = h
        if split.world > 1:
            mine = (C.c_ubyte * 64)()
            ctx.check(ctx.lib.smc_gather_export(ctx.h, self.h, mine))
            handles = [None] * split.world
            dist.all_gather_object(handles, bytes(mine))
            blob = (C.c_ubyte * (64 * split.world)).from_buffer_copy(b"".join(handles))
            ctx.check(ctx.lib.smc_gather_connect(ctx.h, self.h, blob))
            dist.barrier()  # nobody starts an exchange before every rank has mapped its peers
        p = C.c_void_p()
        ctx.check(ctx.lib.smc_gather_buffer(ctx.h, self.h, C.byref(p)))
        self._ptr = p.value
        self._view = None

    def buffer(self):
        """The whole receive buffer as a flat fp32 CUDA tensor (no copy; owned by the library)."""
        if self._view is None:
            t = self.torch

            class _Holder:  # minimal __cuda_array_interface__ provider
                pass

            hld = _Holder()
            hld.__cuda_array_interface__ = {"shape": (self.capacity,), "typestr": "<f4", "data": (self._ptr, False),
                                            "version": 2}
            self._view = t.as_tensor(hld, device=f"cuda:{self.ctx.device}")
        return self._view

    def _stream(self):
        return self.C.c_void_p(self.torch.cuda.current_stream().cuda_stream)

    def matmul(self, x, w_local, mode: int):
        m = x.shape[0] if x.dim() > 1 else 1
        self.ctx.check(self.ctx.lib.smc_qmatmul_gather_dev(self.ctx.h, self.h, x.data_ptr(), w_local.handle, m,
                                                           int(mode), self._stream()))
        return self.buffer()[: self.split.world * m * w_local.N].view(self.split.world, m, w_local.N)

    def exchange(self, count: int):
        self.ctx.check(self.ctx.lib.smc_gather_exchange_dev(self.ctx.h, self.h, int(count), self._stream()))

    def close(self):
        """Every rank must call this (it is collective when `dist` was given): a peer's kernel may still be storing
        packets or ready flags into this rank's buffer, so each rank first finishes its own device work and then all
        ranks meet before any of them unmaps or frees anything."""
        if self.h:
            self.torch.cuda.synchronize()
            if self.dist is not None and self.split.world > 1:
                self.dist.barrier()
            self.ctx.lib.smc_gather_destroy(self.ctx.h, self.h)
            self.h = None
