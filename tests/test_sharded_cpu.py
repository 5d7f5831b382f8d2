"""Row-split exchange logic on CPU: two gloo ranks, the local matmul injected (the oracle stands in for
the CUDA kernels, which is the only place a test may do that).  Checks that slicing the GGUF bytes per
rank, computing slices and all-gathering reproduces the unsplit result bit for bit, for a plain matrix
and for the fused gate||up matrix, and that bad splits are refused."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
Q8_0, Q4_K, Q6_K = 8, 12, 14


def _worker(rank, world, port, results):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import sm_oracle as oracle
        from sharpmind_b200 import synth
        from sharpmind_b200.sharded import RowSplit, ShardedLinear

        split = RowSplit(world, rank)
        out = {}
        for dtype, n, k, m in ((Q8_0, 64, 128, 3), (Q4_K, 32, 512, 2), (Q6_K, 16, 256, 1)):
            w = synth.normal("shard", f"w{dtype}", (n, k), 0.02)
            raw = oracle.quantize(dtype, w)
            x = synth.normal("shard", f"x{dtype}", (m, k))
            full = oracle.qmatmul(dtype, x, raw, m, k, n)
            local_raw = np.ascontiguousarray(split.slice_raw(raw, dtype, n, k))
            nl = split.rows(n)

            def compute(xt, local_raw=local_raw, dtype=dtype, k=k, nl=nl):
                xx = xt.numpy()
                return torch.from_numpy(oracle.qmatmul(dtype, xx, local_raw, xx.shape[0], k, nl))

            lin = ShardedLinear(split, n, compute, dist)
            got = lin.forward(torch.from_numpy(x)).numpy()
            out[f"plain{dtype}"] = bool(np.array_equal(got.view(np.uint32), full.view(np.uint32)))
        # fused gate||up: each rank holds its gate rows followed by its up rows
        F, k, m = 32, 512, 2
        w = synth.normal("shard", "wgu", (2 * F, k), 0.02)
        raw = oracle.quantize(Q4_K, w)
        x = synth.normal("shard", "xgu", (m, k))
        full = oracle.qmatmul(Q4_K, x, raw, m, k, 2 * F)
        local_raw = np.ascontiguousarray(split.slice_fused_raw(raw, Q4_K, F, k))
        nl = 2 * split.rows(F)
        lin = ShardedLinear(split, 2 * F,
                            lambda xt: torch.from_numpy(oracle.qmatmul(Q4_K, xt.numpy(), local_raw, m, k, nl)), dist,
                            fused_halves=2)
        got = lin.forward(torch.from_numpy(x)).numpy()
        out["fused"] = bool(np.array_equal(got.view(np.uint32), full.view(np.uint32)))
        # one exchange per feed-forward block: gate||up by rows, down split along K, partial sums added in rank order
        from sharpmind_b200.sharded import KSplit, ShardedFfn

        H, F, m = 256, 1024, 2
        ks = KSplit(world, rank, step=256)
        raw_gu = oracle.quantize(Q4_K, synth.normal("shard", "ffn_gu", (2 * F, H), 0.05))
        raw_dn = oracle.quantize(Q6_K, synth.normal("shard", "ffn_dn", (H, F), 0.05))
        x = synth.normal("shard", "ffn_x", (m, H))

        def ffn_parts(r):
            f0, f1 = ks.k_range(F, r)
            gu_l = ks.slice_fused_rows_raw(raw_gu, Q4_K, F, H, r)
            dn_l = ks.slice_columns_raw(raw_dn, Q6_K, H, F, r)
            gu = oracle.qmatmul(Q4_K, x, gu_l, m, H, 2 * (f1 - f0))
            act = oracle.swiglu(np.ascontiguousarray(gu[:, :f1 - f0]), np.ascontiguousarray(gu[:, f1 - f0:]))
            return oracle.qmatmul(Q6_K, act, dn_l, m, f1 - f0, H)

        f0, f1 = ks.k_range(F)
        gu_local = ks.slice_fused_rows_raw(raw_gu, Q4_K, F, H)
        dn_local = ks.slice_columns_raw(raw_dn, Q6_K, H, F)
        ffn = ShardedFfn(ks,
                         lambda xt: torch.from_numpy(oracle.qmatmul(Q4_K, xt.numpy(), gu_local, m, H, 2 * (f1 - f0))),
                         lambda at: torch.from_numpy(oracle.qmatmul(Q6_K, np.ascontiguousarray(at.numpy()), dn_local, m, f1 - f0, H)),
                         dist)
        got = ffn.forward(torch.from_numpy(x)).numpy()
        want_sum = ffn_parts(0)
        for r in range(1, world):
            want_sum = want_sum + ffn_parts(r)
        gu = oracle.qmatmul(Q4_K, x, raw_gu, m, H, 2 * F)
        full = oracle.qmatmul(Q6_K, oracle.swiglu(np.ascontiguousarray(gu[:, :F]), np.ascontiguousarray(gu[:, F:])), raw_dn, m, F, H)
        # torch's SiLU-gate differs from the oracle's in the last place, so the sum is held to the parity bound, and
        # the K-split differs from the unsplit product by summation order only
        out["ffn_rank_order"] = bool(np.max(np.abs(got - want_sum)) <= 1e-5 * np.max(np.abs(full)))
        out["ffn_vs_unsplit"] = bool(np.max(np.abs(got - full)) <= 1e-5 * np.max(np.abs(full)))
        results[rank] = out
    finally:
        dist.destroy_process_group()


def test_row_split_two_ranks_gloo():
    world = 2
    mgr = mp.Manager()
    results = mgr.dict()
    port = 29500 + (os.getpid() % 2000)
    mp.spawn(_worker, args=(world, port, results), nprocs=world, join=True)
    assert len(results) == world
    for rank in range(world):
        assert all(results[rank].values()), results[rank]


def test_split_refuses_unaligned_slices():
    from sharpmind_b200.sharded import RowSplit

    s = RowSplit(2, 0)
    with pytest.raises(ValueError):
        s.rows(7)
    with pytest.raises(ValueError):  # 3 rows x 96 = 288 elements: not a whole number of 256-element blocks
        s.check_block_aligned(Q4_K, 6, 96)
    s.check_block_aligned(Q4_K, 4, 128)  # 2 rows x 128 = one block
    with pytest.raises(ValueError):
        s.check_block_aligned(Q8_0, 4, 48)
    assert RowSplit(4, 3).row_range(16) == (12, 16)


def test_k_split_follows_whole_steps():
    from sharpmind_b200.sharded import KSplit

    assert KSplit(2, 0).bounds(28672) == [0, 14336, 28672]
    assert KSplit(4, 0).bounds(28672) == [0, 8192, 16384, 22528, 28672]                   # 4 + 4 + 3 + 3 steps
    assert [b // 2048 for b in KSplit(8, 0).bounds(28672)] == [0, 2, 4, 6, 8, 10, 12, 13, 14]
    assert KSplit(8, 7).k_range(28672) == (26624, 28672)
    with pytest.raises(ValueError):
        KSplit(2, 0).bounds(3000)          # not whole steps
    with pytest.raises(ValueError):
        KSplit(8, 0).bounds(4 * 2048)      # fewer steps than ranks
    # column slices of a GGUF tensor: rows keep their order, blocks [k0/256, k1/256) of each row
    raw = np.arange(4 * 16 * 144, dtype=np.uint32).astype(np.uint8)  # 4 rows x 16 Q4_K blocks
    ks = KSplit(2, 1, step=2048)
    sl = ks.slice_columns_raw(raw, Q4_K, 4, 4096)
    assert sl.shape[0] == 4 * 8 * 144
    assert np.array_equal(sl.reshape(4, 8 * 144), raw.reshape(4, 16 * 144)[:, 8 * 144:])


def test_assemble_single_rank_is_identity():
    from sharpmind_b200.sharded import RowSplit, ShardedLinear

    lin = ShardedLinear(RowSplit(1, 0), 8, lambda x: x * 2.0)
    x = torch.arange(16, dtype=torch.float32).reshape(2, 8)
    assert torch.equal(lin.forward(x), x * 2.0)
