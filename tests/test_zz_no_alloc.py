"""smc_qmatmul_q8_noalloc: the quantised-activation matmul for hosts that may not allocate device memory
while they run (memory fully budgeted at start-up, or no tolerance for cudaMalloc's device-wide
synchronisation).  Its intermediate buffer is a fixed array inside the library, so the test checks that it
gives the same bits as the allocating entry point, twice in a row with different inputs (the array keeps the
first call's contents), and that shapes beyond the array are refused.  Collected last on purpose."""
import numpy as np
import pytest

from sharpmind_b200 import synth

pytestmark = pytest.mark.gpu
Q8_0, Q4_K, Q6_K = 8, 12, 14


def test_noalloc_matches_allocating_entry_point_twice(oracle, cuda, dev):
    import torch

    from sharpmind_b200 import ops

    for dtype, n, k in ((Q4_K, 256, 4096), (Q6_K, 64, 2048), (Q8_0, 192, 1024)):
        raw = oracle.quantize(dtype, synth.normal("noalloc", f"w{dtype}", (n, k), 0.02))
        w = cuda.register(raw, dtype, n, k)
        for call, m in enumerate((4, 7)):  # two calls in a row, different rows and row counts
            x = torch.from_numpy(synth.normal("noalloc", f"x{dtype}_{call}", (m, k))).cuda()
            want = dev.qmatmul(x, w, ops.Mode.ACT_Q8).cpu().numpy()
            got = dev.qmatmul_q8_noalloc(x, w).cpu().numpy()
            assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), (dtype, call)
            # and against the oracle fed the dequantised activations, at the suite's tolerance
            xq = oracle.quantize_rows_q8_0(x.cpu().numpy(), m, k)
            xhat = np.stack([oracle.dequantize(Q8_0, xq[r], k) for r in range(m)])
            ref = oracle.qmatmul(dtype, xhat, raw, m, k, n)
            wn = np.linalg.norm(oracle.dequantize(dtype, raw, n * k).reshape(n, k).astype(np.float64), axis=1)
            bound = 1e-5 * np.linalg.norm(xhat.astype(np.float64), axis=1)[:, None] * wn[None, :]
            assert np.all(np.abs(got - ref) <= bound)
        cuda.release(w)
    assert cuda.device_status() == 0


def test_noalloc_at_its_limit_and_refusal_beyond(oracle, cuda, dev):
    """M * K exactly at the limit with seeded random rows, for every format (Q4_K reads the block sums, Q6_K the
    half-block sums, so every region of the fixed array is exercised at full size); a smaller shape straight
    after shows that what the large call left behind does no harm; one row more is refused."""
    import torch

    from sharpmind_b200 import ops

    k, n = 16384, 32  # 32 * 16384 = SMC_NOALLOC_MAX_ELEMS exactly
    for dtype in (Q8_0, Q4_K, Q6_K):
        raw = oracle.quantize(dtype, synth.normal("noalloc", f"wbig{dtype}", (n, k), 0.02))
        w = cuda.register(raw, dtype, n, k)
        full = torch.from_numpy(synth.normal("noalloc", f"xbig{dtype}", (32, k))).cuda()
        want = dev.qmatmul(full, w, ops.Mode.ACT_Q8).cpu().numpy()
        got = dev.qmatmul_q8_noalloc(full, w).cpu().numpy()
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), dtype
        small = torch.from_numpy(synth.normal("noalloc", f"xsmall{dtype}", (3, k))).cuda()
        want = dev.qmatmul(small, w, ops.Mode.ACT_Q8).cpu().numpy()
        got = dev.qmatmul_q8_noalloc(small, w).cpu().numpy()
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), dtype
        one = small[1:2].contiguous()  # a single row takes the bulk-copy kernel on the rows quantised into the array
        want = dev.qmatmul(one, w, ops.Mode.ACT_Q8).cpu().numpy()
        got = dev.qmatmul_q8_noalloc(one, w).cpu().numpy()
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), dtype
        too_big = torch.zeros((33, k), device="cuda")
        with pytest.raises(ops.ArgumentOutOfRangeException):
            dev.qmatmul_q8_noalloc(too_big, w)
        cuda.release(w)
    assert cuda.device_status() == 0
