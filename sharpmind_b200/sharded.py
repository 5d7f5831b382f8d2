"""Row-split quantized matmul across the GPUs of one node.

Output rows are independent (out[:, c] depends only on weight row c), so each rank keeps rows
[rank*N/G, (rank+1)*N/G) of every matrix, uploaded once, computes its output slice with the same
single-GPU kernels and one all-gather (NCCL over NVLink) reassembles [M, N].  Activations are
replicated.  A split point must fall on a block boundary of the flat tensor: (N/G)*K must be a
multiple of the format's block size, otherwise the slice would start inside a block.

The fused gate||up matrix is split per half (each rank holds its gate rows followed by its up rows)
so that SwiGLU can run on local data; `gather_fused` restores the [gate | up] column order.

A feed-forward block needs only ONE exchange when its second matrix is split along K instead (`KSplit`):
gate||up by rows with a split that follows whole K-steps of the down projection, SwiGLU on local data, then
rank g multiplies its slice of the activation row by columns [k0_g, k1_g) of every row of `down` and the
partial sums of all ranks are added in rank order (`PeerGather.matmul_reduce`, inside the producing kernel).

The reference has no multi-device path (single process, single accelerator); these are the exchange
steps the split adds, and the only collectives on the path.
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


# elements one step of the one-row kernel covers: K-slices are whole steps so that every rank's slice runs on it
KSTEP_ELEMS = {8: 1024, 12: 2048, 14: 2048}


@dataclass(frozen=True)
class KSplit:
    """Split of an inner dimension of `k` elements into whole steps of `step` elements, as even as whole steps allow:
    with s = k / step steps over G ranks the first s % G ranks take one step more.  (28672 columns of a Q4_K / Q6_K
    matrix are 14 steps: 7 + 7 over two ranks, 4 + 4 + 3 + 3 over four, 2 x 6 + 1 x 2 over eight.)"""
    world: int
    rank: int
    step: int = 2048

    def bounds(self, k: int) -> list[int]:
        if k % self.step:
            raise ValueError(f"K = {k} is not a whole number of {self.step}-element steps")
        steps = k // self.step
        if steps < self.world:
            raise ValueError(f"{steps} steps cannot be split over {self.world} ranks")
        base, extra = divmod(steps, self.world)
        b = [0]
        for r in range(self.world):
            b.append(b[-1] + (base + (1 if r < extra else 0)) * self.step)
        return b

    def k_range(self, k: int, rank: int | None = None) -> tuple[int, int]:
        b = self.bounds(k)
        r = self.rank if rank is None else rank
        return b[r], b[r + 1]

    def slice_columns_raw(self, raw, dtype: int, n: int, k: int, rank: int | None = None):
        """Columns [k0, k1) of every row of a GGUF-layout [n, k] tensor as a contiguous [n, k1 - k0] tensor."""
        be = BLOCK_ELEMS[int(dtype)]
        k0, k1 = self.k_range(k, rank)
        per_row = raw.shape[0] // n
        bb = per_row * be // k  # bytes per block
        if per_row * n != raw.shape[0] or bb * (k // be) != per_row:
            raise ValueError("tensor bytes are not whole rows of whole blocks")
        rows = raw.reshape(n, per_row)[:, k0 // be * bb:k1 // be * bb]
        import numpy as np

        if isinstance(raw, np.ndarray):
            return np.ascontiguousarray(rows).reshape(-1)
        return rows.contiguous().reshape(-1)

    def slice_fused_rows_raw(self, raw, dtype: int, n_half: int, k: int, rank: int | None = None, interleave: bool = False):
        """gate||up [2 * n_half, k] split by ROWS the way this split cuts the `n_half` inner elements of the down
        projection: this rank's gate rows followed by its up rows, or (`interleave`) woven gate 0, up 0, gate 1, ...
        for the matmul that applies the SiLU-gate in its epilogue."""
        f0, f1 = self.k_range(n_half, rank)
        per_row = raw.shape[0] // (2 * n_half)
        gate = raw[f0 * per_row:f1 * per_row]
        up = raw[(n_half + f0) * per_row:(n_half + f1) * per_row]
        import numpy as np

        if interleave:
            if isinstance(raw, np.ndarray):
                return np.stack([gate.reshape(f1 - f0, per_row), up.reshape(f1 - f0, per_row)], axis=1).reshape(-1)
            import torch

            return torch.stack([gate.reshape(f1 - f0, per_row), up.reshape(f1 - f0, per_row)], dim=1).reshape(-1)

        if isinstance(raw, np.ndarray):
            return np.concatenate([gate, up])
        import torch

        return torch.cat([gate, up])


class ShardedFfn:
    """One gated feed-forward block over G ranks with a single exchange: y = down(SiLU(gate(x)) * up(x)).

    `gate_up(x) -> [M, 2 * F_local]` and `down_partial(act) -> [M, H]` are the local matmuls on this rank's slices
    (injected, as for ShardedLinear); `dist.all_reduce` stands in for the in-kernel exchange on backends without peer
    memory (gloo on CPU).  The product path is PeerGather.matmul_reduce."""

    def __init__(self, split: KSplit, gate_up, down_partial, dist=None):
        self.split, self.gate_up, self.down_partial, self.dist = split, gate_up, down_partial, dist

    def forward(self, x):
        import torch

        gu = self.gate_up(x)
        f = gu.shape[-1] // 2
        g, u = gu[..., :f], gu[..., f:]
        act = g / (1.0 + torch.exp(-g)) * u
        part = self.down_partial(act)
        if self.split.world == 1:
            return part
        # rank-ordered sum: gather the partials and add them 0, 1, ..., G - 1 (what the kernel's tail does)
        parts = [torch.empty_like(part) for _ in range(self.split.world)]
        self.dist.all_gather(parts, part.contiguous())
        out = parts[0].clone()
        for p in parts[1:]:
            out += p
        return out


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
            dist.all_gather_object(handles, (self.capacity, bytes(mine)))
            if any(cap != self.capacity for cap, _ in handles):
                # a peer's packet areas are addressed through this rank's own capacity: all buffers must be laid out alike
                ctx.lib.smc_gather_destroy(ctx.h, self.h)
                self.h = None
                raise ValueError(f"PeerGather: ranks asked for different capacities {[cap for cap, _ in handles]}")
            blob = (C.c_ubyte * (64 * split.world)).from_buffer_copy(b"".join(h_ for _, h_ in handles))
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

    def matmul_reduce(self, x, w_local, mode: int, up=None):
        """K-split matmul: `w_local` holds this rank's columns of every row, `x` the matching slice of the activation
        row(s) (or, with `up`, the local gate slice: the activation is SiLU(x) * up).  Returns a [M, N] view of the
        receive buffer holding the sum of all ranks' partial products in rank order, identical on every rank."""
        m = x.shape[0] if x.dim() > 1 else 1
        self.ctx.check(self.ctx.lib.smc_qmatmul_reduce_dev(self.ctx.h, self.h, x.data_ptr(), None if up is None else up.data_ptr(),
                                                           w_local.handle, m, int(mode), self._stream()))
        return self.buffer()[: m * w_local.N].view(m, w_local.N)

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
