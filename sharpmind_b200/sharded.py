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
