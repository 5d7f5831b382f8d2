"""Parity of the CUDA quantized matmul (through the C ABI) with the CPU oracle.

Bars: SMC_REF_ORDER is bit-exact with the scalar tier; SMC_ACT_F32 is within 1e-5*||w||*||x|| per
output; SMC_ACT_Q8 has bit-exact activation quants, fp16 scales and per-block int32 sums, and fp32
outputs within 1e-5*||w||*||x_hat|| of the oracle fed the dequantised activations.
"""
import os

import numpy as np
import pytest

from sharpmind_b200 import synth
from tests.gpu_util import Q4_K, Q6_K, Q8_0, bits, row_norm_bound, to_dev
from tests.test_oracle_pins import _random_raw

pytestmark = pytest.mark.gpu

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "vecdot_golden.npz")


def make_weight(oracle, dtype, n, k, name):
    w = synth.normal("gpu", name, (n, k), 0.02)
    return oracle.quantize(dtype, w)


SHAPES = [
    (Q8_0, 3072, 1024),   # Qwen3-0.6B FFN-up: the reference's own CPU-runnable case
    (Q8_0, 96, 3072), (Q8_0, 40, 64), (Q8_0, 17, 32),
    (Q4_K, 256, 4096), (Q4_K, 33, 256), (Q4_K, 64, 1024),
    (Q6_K, 64, 14336), (Q6_K, 33, 256), (Q6_K, 128, 1024),
]


@pytest.mark.parametrize("dtype,n,k", SHAPES)
@pytest.mark.parametrize("m", [1, 2, 3, 8, 32])
def test_qmatmul_modes_against_oracle(oracle, cuda, dev, dtype, n, k, m):
    from sharpmind_b200.ops import Mode, Q8Act

    if m > 3 and n * k > 2_000_000:
        pytest.skip("oracle time: large shapes are checked at small M")
    raw = make_weight(oracle, dtype, n, k, f"w{dtype}_{n}_{k}")
    x = synth.normal("gpu", f"x{dtype}_{n}_{k}_{m}", (m, k))
    w = cuda.register(raw, dtype, n, k)
    try:
        want = oracle.qmatmul(dtype, x, raw, m, k, n)
        xd = to_dev(x)
        # reference order: bit exact
        got = dev.qmatmul(xd, w, Mode.REF_ORDER).cpu().numpy()
        assert np.array_equal(bits(got), bits(want))
        # fp32 activations
        got = dev.qmatmul(xd, w, Mode.ACT_F32).cpu().numpy()
        bound = row_norm_bound(oracle, dtype, raw, n, k, x)
        assert np.all(np.abs(got.astype(np.float64) - want) <= bound), np.max(np.abs(got - want) / bound)
        # quantised activations
        act = Q8Act(cuda, max(m, 1), k)
        dev.quantize_q8(xd, act, k)
        q, dbits = act.read()
        xq = oracle.quantize_rows_q8_0(x, m, k)
        oq, od = oracle.split_q8_rows(xq)
        assert np.array_equal(q, oq) and np.array_equal(dbits, od)
        sums = dev.block_isums(act, m - 1, w, 0, min(n, 8)).cpu().numpy()
        for c in range(min(n, 8)):
            assert np.array_equal(sums[c], oracle.block_isums(dtype, raw, xq[m - 1], c, k))
        xhat = np.stack([oracle.dequantize(Q8_0, xq[r], k) for r in range(m)])
        want_q = oracle.qmatmul(dtype, xhat, raw, m, k, n)
        got_q = dev.qmatmul_q8(act, w).cpu().numpy()
        bound_q = row_norm_bound(oracle, dtype, raw, n, k, xhat)
        assert np.all(np.abs(got_q.astype(np.float64) - want_q) <= bound_q), np.max(np.abs(got_q - want_q) / bound_q)
        # the one-call form (quantise + matmul on the context's scratch) gives the same bits
        got_q2 = dev.qmatmul(xd, w, Mode.ACT_Q8).cpu().numpy()
        assert np.array_equal(bits(got_q2), bits(got_q))
        act.close()
    finally:
        cuda.release(w)


def test_results_do_not_depend_on_batch_size(oracle, cuda, dev):
    """Row r of an M-row call has the same bits for every M >= 2, whatever the other rows hold (both fast modes,
    all formats); the one-row kernels use a different summation tree and agree within the parity bound."""
    from sharpmind_b200.ops import Mode

    for dtype, n, k in ((Q8_0, 512, 1024), (Q4_K, 256, 4096), (Q6_K, 64, 14336)):
        raw = make_weight(oracle, dtype, n, k, f"bs{dtype}")
        w = cuda.register(raw, dtype, n, k)
        xh = synth.normal("gpu", f"bsx{dtype}", (32, k))
        x = to_dev(xh)
        bound = row_norm_bound(oracle, dtype, raw, n, k, xh)
        for mode in (Mode.ACT_F32, Mode.ACT_Q8):
            full = dev.qmatmul(x, w, mode).cpu().numpy()
            for m in (2, 5, 8, 9, 16, 17):
                part = dev.qmatmul(x[:m].contiguous(), w, mode).cpu().numpy()
                assert np.array_equal(bits(part), bits(full[:m])), (dtype, mode, m)
            pair = dev.qmatmul(x[[31, 7]].contiguous(), w, mode).cpu().numpy()  # other neighbours, other slot
            assert np.array_equal(bits(pair[0]), bits(full[31])) and np.array_equal(bits(pair[1]), bits(full[7]))
            for r in (0, 7, 31):
                one = dev.qmatmul(x[r:r + 1].contiguous(), w, mode).cpu().numpy()
                assert np.all(np.abs(one[0].astype(np.float64) - full[r]) <= 2 * bound[r]), (dtype, mode, r)
        cuda.release(w)


@pytest.mark.parametrize("n,k", [(100, 1024), (96, 3072), (40, 640), (64, 2048)])
def test_q8_0_prompt_sized_batches_keep_the_small_batch_bits(oracle, cuda, dev, n, k):
    """Q8_0 at 256 rows and more runs a kernel in which a warp owns a whole output tile (no K split across warps): it
    must give each row the bits the 32-row kernel gives it (ragged last tiles, rows past N, group counts that do not fill
    the eight classes), and sampled rows must meet the oracle."""
    from sharpmind_b200.ops import Mode

    raw = make_weight(oracle, Q8_0, n, k, f"pq{n}_{k}")
    w = cuda.register(raw, Q8_0, n, k)
    for m in (256, 300, 577):
        xh = synth.normal("gpu", f"pqx{k}_{m}", (m, k))
        x = to_dev(xh)
        full = dev.qmatmul(x, w, Mode.ACT_Q8).cpu().numpy()
        for lo in (0, 32, m - 32):  # the same rows as batches of 32: the K-split kernel
            part = dev.qmatmul(x[lo:lo + 32].contiguous(), w, Mode.ACT_Q8).cpu().numpy()
            assert np.array_equal(bits(part), bits(full[lo:lo + 32])), (m, lo)
        mid = dev.qmatmul(x[:128].contiguous(), w, Mode.ACT_Q8).cpu().numpy()  # 64-token passes of the K-split kernel
        assert np.array_equal(bits(mid), bits(full[:128]))
        rows = [0, m // 2, m - 1]
        xq = oracle.quantize_rows_q8_0(xh[rows], len(rows), k)
        xhat = np.stack([oracle.dequantize(Q8_0, xq[r], k) for r in range(len(rows))])
        want = oracle.qmatmul(Q8_0, xhat, raw, len(rows), k, n)
        bound = row_norm_bound(oracle, Q8_0, raw, n, k, xhat)
        assert np.all(np.abs(full[rows].astype(np.float64) - want) <= bound)
    cuda.release(w)


@pytest.mark.parametrize("dtype,n,k", [(Q6_K, 64, 2048), (Q8_0, 96, 1024), (Q4_K, 96, 4096), (Q6_K, 40, 14336)])
@pytest.mark.parametrize("m", [2, 7, 64, 100])
def test_fp32_activations_as_int8_digit_planes(oracle, cuda, dev, dtype, n, k, m):
    """SMC_ACT_F32 with two rows and more, where no tcgen05 kernel takes the format or shape: the fp32 rows go through the
    int8 tensor-core kernels as three digit planes.  Same per-output bound against the oracle as the CUDA-core kernel it
    replaces, and agreement with that kernel (option off) inside twice the bound; rows with a zero block, a huge value
    and tiny values included."""
    from sharpmind_b200.ops import Mode

    raw = make_weight(oracle, dtype, n, k, f"dg{dtype}_{n}_{k}")
    w = cuda.register(raw, dtype, n, k)
    x = synth.normal("gpu", f"dgx{dtype}_{k}_{m}", (m, k))
    x[1, :32] = 0.0
    x[0, 5] = 3.0e4
    x[m - 1] *= 1.0e-6
    xd = to_dev(x)
    got = dev.qmatmul(xd, w, Mode.ACT_F32).cpu().numpy()
    want = oracle.qmatmul(dtype, x, raw, m, k, n)
    bound = row_norm_bound(oracle, dtype, raw, n, k, x)
    assert np.all(np.abs(got.astype(np.float64) - want) <= bound), float(np.max(np.abs(got - want) / bound))
    cuda.set_option("f32_prefill_int8_digits", 0)
    try:
        old = dev.qmatmul(xd, w, Mode.ACT_F32).cpu().numpy()
    finally:
        cuda.set_option("f32_prefill_int8_digits", 1)
    assert np.all(np.abs(old.astype(np.float64) - got) <= 2 * bound)
    assert not np.array_equal(bits(old), bits(got))  # the option really switches kernels
    cuda.release(w)
    assert cuda.device_status() == 0


def test_fp32_digit_scratch_is_stable_across_shapes_under_capture(oracle, cuda, dev):
    """The digit planes live in one scratch allocation sized by the largest call so far: alternating between matrices of
    different K after a warm-up must not allocate again, or a stream capture of the same calls would be invalidated."""
    import torch

    from sharpmind_b200.ops import Mode

    ws, xs = [], []
    for n, k in ((64, 14336), (96, 4096), (32, 2048)):
        ws.append(cuda.register(make_weight(oracle, Q6_K, n, k, f"cap{n}_{k}"), Q6_K, n, k))
        xs.append(to_dev(synth.normal("gpu", f"capx{k}", (3, k))))
    outs = [torch.empty((3, w.N), device="cuda") for w in ws]
    want = [dev.qmatmul(x, w, Mode.ACT_F32).clone() for x, w in zip(xs, ws)]  # warm-up: the scratch reaches its size

    def body():
        for i in (0, 1, 2, 0, 1):
            dev.qmatmul(xs[i], ws[i], Mode.ACT_F32, out=outs[i])

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        body()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        body()
    for o in outs:
        o.zero_()
    g.replay()
    torch.cuda.synchronize()
    for o, w_ in zip(outs, want):
        assert torch.equal(o, w_)
    for w in ws:
        cuda.release(w)
    assert cuda.device_status() == 0


RING_SHAPES = [
    (Q4_K, 304, 4096), (Q4_K, 48, 14336), (Q4_K, 16, 2048), (Q6_K, 64, 14336), (Q6_K, 160, 4096), (Q6_K, 2384, 2048),
    (Q8_0, 272, 5120), (Q8_0, 64, 1024), (Q8_0, 4752, 1024),
]


@pytest.mark.parametrize("dtype,n,k", RING_SHAPES)
def test_small_batch_ring_kernel(oracle, cuda, dev, dtype, n, k):
    """2..32 rows with the weights streamed through the bulk-copy ring: every output within the SMC_ACT_Q8 bound of the
    oracle fed the dequantised activations; the same bits whatever the grid (1, 5, 37 CTAs, one per SM), whatever the
    batch size a row travels in, and with dependent launch off; within the bound of the kernel that fetches its
    fragments from global memory (the two add a row's blocks in different orders)."""
    from sharpmind_b200.ops import Mode

    raw = make_weight(oracle, dtype, n, k, f"ring{dtype}_{n}_{k}")
    w = cuda.register(raw, dtype, n, k)
    xh = synth.normal("gpu", f"ringx{dtype}_{n}_{k}", (32, k))
    x = to_dev(xh)
    cuda.set_option("small_batch_ring", 2)  # every format through the ring (off by default)
    try:
        full = dev.qmatmul(x, w, Mode.ACT_Q8).cpu().numpy()
        xq = oracle.quantize_rows_q8_0(xh, 32, k)
        xhat = np.stack([oracle.dequantize(Q8_0, xq[r], k) for r in range(32)])
        cols = sorted({c for c in (0, 15, 16, n // 2, n - 17, n - 1) if 0 <= c < n})
        bound = row_norm_bound(oracle, dtype, raw, n, k, xhat)
        for c in cols:
            want = oracle.qmatmul(dtype, xhat, raw, 32, k, n, cols=(c, c + 1))[:, c]
            assert np.all(np.abs(full[:, c].astype(np.float64) - want) <= bound[:, c]), (c, float(np.max(np.abs(full[:, c] - want) / bound[:, c])))
        for m in (2, 7, 8, 9, 16, 17, 31):
            part = dev.qmatmul(x[:m].contiguous(), w, Mode.ACT_Q8).cpu().numpy()
            assert np.array_equal(bits(part), bits(full[:m])), m
        for opts in ({"gemv_ctas": 1}, {"gemv_ctas": 5, "pdl": 0}, {"gemv_ctas": 37}):
            for name, v in opts.items():
                cuda.set_option(name, v)
            try:
                got = dev.qmatmul(x[:9].contiguous(), w, Mode.ACT_Q8).cpu().numpy()
            finally:
                for name in opts:
                    cuda.set_option(name, {"pdl": 1}.get(name, 0))
            assert np.array_equal(bits(got), bits(full[:9])), opts
        cuda.set_option("small_batch_ring", 0)
        other = dev.qmatmul(x, w, Mode.ACT_Q8).cpu().numpy()
        assert np.all(np.abs(other.astype(np.float64) - full) <= 2 * bound), float(np.max(np.abs(other - full) / bound))
    finally:
        cuda.set_option("small_batch_ring", 0)
        cuda.release(w)
    assert cuda.device_status() == 0


# One row against few long rows: row counts near the number of resident warps (some warps take one row, some two),
# rows of many steps, and row counts that the warps do not divide.
LONG_ROW_SHAPES = [
    (Q4_K, 4096, 4096),    # attention output of an 8B decoder
    (Q6_K, 4096, 14336),   # FFN down of an 8B decoder
    (Q4_K, 400, 16384), (Q8_0, 400, 8192),
    (Q8_0, 1500, 2048), (Q6_K, 1001, 6144),
]


@pytest.mark.parametrize("dtype,n,k", LONG_ROW_SHAPES)
def test_one_row_long_rows_against_oracle(oracle, cuda, dev, dtype, n, k):
    from sharpmind_b200.ops import Mode

    raw = make_weight(oracle, dtype, n, k, f"team{dtype}_{n}_{k}")
    x = synth.normal("gpu", f"teamx{dtype}_{n}_{k}", (1, k))
    w = cuda.register(raw, dtype, n, k)
    try:
        xq = oracle.quantize_rows_q8_0(x, 1, k)
        xhat = oracle.dequantize(Q8_0, xq[0], k)[None, :]
        want = oracle.qmatmul(dtype, xhat, raw, 1, k, n)
        bound = row_norm_bound(oracle, dtype, raw, n, k, xhat)
        got = dev.qmatmul(to_dev(x), w, Mode.ACT_Q8).cpu().numpy()
        assert np.all(np.abs(got.astype(np.float64) - want) <= bound), np.max(np.abs(got - want) / bound)
        # the same row inside a two-row call runs the tensor-core kernel: equal to rounding, not to the bit
        two = dev.qmatmul(to_dev(np.concatenate([x, x])), w, Mode.ACT_Q8).cpu().numpy()
        assert np.all(np.abs(two[0].astype(np.float64) - got[0]) <= 2 * bound[0])
        # repeatable
        again = dev.qmatmul(to_dev(x), w, Mode.ACT_Q8).cpu().numpy()
        assert np.array_equal(bits(again), bits(got))
    finally:
        cuda.release(w)
    assert cuda.device_status() == 0


# The one-row kernel cuts a CTA's rows into equal pieces per warp without regard to row boundaries and continues a
# row from the lane sums its previous warp left: an output's bits must not depend on how the rows were divided.
# The options change the grid, the stage length and with them every piece boundary.
PARTITION_SHAPES = [
    (Q4_K, 28672, 4096),   # the Llama-3-8B gate||up launch of the benchmark
    (Q4_K, 8192, 28672),   # Llama-3-70B down: the row takes two rounds of activation loads
    (Q6_K, 4096, 14336), (Q6_K, 3, 14336), (Q6_K, 37, 6144), (Q4_K, 4096, 4096), (Q4_K, 1, 8192), (Q4_K, 445, 2048),
    (Q8_0, 1500, 2048), (Q8_0, 7, 5120), (Q8_0, 3072, 1024), (Q8_0, 300, 8192),
]


@pytest.mark.parametrize("dtype,n,k", PARTITION_SHAPES)
def test_one_row_bits_do_not_depend_on_the_partition(oracle, cuda, dev, dtype, n, k):
    import torch

    from sharpmind_b200.ops import Mode

    g = torch.Generator(device="cuda").manual_seed(n * 31 + k)
    raw_d = dev.quantize_weights(dtype, torch.randn((n, k), generator=g, device="cuda") * 0.02)
    w = cuda.register_dev(raw_d, dtype, n, k, keep_raw=True)
    x = to_dev(synth.normal("gpu", f"partx{dtype}_{n}_{k}", (1, k)))
    try:
        base = dev.qmatmul(x, w, Mode.ACT_Q8).cpu().numpy()
        # the exact integer block sums and fp32 scaling of the reference-order-free generic kernel bound it
        rows = sorted({0, n // 2, n - 1})
        raw = raw_d.cpu().numpy()
        xq = oracle.quantize_rows_q8_0(x.cpu().numpy(), 1, k)
        xhat = oracle.dequantize(Q8_0, xq[0], k)[None, :]
        per_row = len(raw) // n
        for r in rows:
            want = oracle.qmatmul(dtype, xhat, raw, 1, k, n, cols=(r, r + 1))[0, r]
            wrow = oracle.dequantize(dtype, raw[r * per_row:(r + 1) * per_row], k)
            assert abs(float(base[0, r]) - float(want)) <= 1e-5 * np.linalg.norm(wrow) * np.linalg.norm(xhat)
        for opts in ({"gemv_ctas": 37}, {"gemv_ctas": 296, "gemv_steps_per_stage": 1, "gemv_prefetch_first": 0},
                     {"gemv_steps_per_stage": 4, "gemv_slots": 3}, {"gemv_ctas": 1, "gemv_slots": 4, "pdl": 0},
                     {"gemv_pair_staging": 0}, {"gemv_pair_staging": 0, "gemv_ctas": 74}, {"gemv_ctas": 74}):
            # (gemv_pair_staging: rows of 8192 elements and more are quantised half each by the two SMs of a pair)
            for name, v in opts.items():
                cuda.set_option(name, v)
            try:
                got = dev.qmatmul(x, w, Mode.ACT_Q8).cpu().numpy()
            finally:
                for name in opts:
                    cuda.set_option(name, {"pdl": 1, "gemv_prefetch_first": 1, "gemv_pair_staging": 1}.get(name, 0))
            assert np.array_equal(bits(got), bits(base)), opts
    finally:
        cuda.release(w)
    assert cuda.device_status() == 0


@pytest.mark.parametrize("k", [8, 15, 20, 32, 33, 40, 63, 64, 96, 137, 896])
def test_q8_0_block_tails_with_poisoned_padding(oracle, cuda, dev, k):
    # Q8BlockTailTests.cs:25-97: partial last blocks; anything read past K would pick up 1e6
    from sharpmind_b200.ops import Mode

    n = 3
    raw = _random_raw(Q8_0, oracle.raw_bytes(Q8_0, n, k), f"tail{k}")
    x = np.full((2, k + 64), 1e6, np.float32)
    x[:, :k] = synth.uniform("gpu", f"tailx{k}", (2, k))
    xin = np.ascontiguousarray(x[:, :k])
    w = cuda.register(raw, Q8_0, n, k)
    want = oracle.qmatmul(Q8_0, xin, raw, 2, k, n)
    for mode in (Mode.REF_ORDER, Mode.ACT_F32):
        got = dev.qmatmul(to_dev(xin), w, mode).cpu().numpy()
        if mode == Mode.REF_ORDER or k % 32:
            assert np.array_equal(bits(got), bits(want))
        else:
            assert np.all(np.abs(got - want) <= 1e-4 * np.maximum(1.0, np.abs(want)))
    cuda.release(w)


@pytest.mark.parametrize("dtype", [Q4_K, Q6_K])
@pytest.mark.parametrize("n,k", [(8, 96), (8, 160), (4, 320), (6, 1024)])
def test_kquant_rows_that_start_inside_a_block(oracle, cuda, dev, dtype, n, k):
    """Flat-tensor addressing (startBlock / colBlockStart): rows need not start on a block boundary."""
    from sharpmind_b200.ops import Mode

    nbytes = oracle.raw_bytes(dtype, n, k)
    raw = _random_raw(dtype, nbytes + 256, f"rag{dtype}_{n}_{k}")[:nbytes].copy()
    # The reference's Q6_K loop reads up to 96 floats past a row that ends inside a 128-element half
    # (into the next input row, or past the tensor).  The CUDA kernel reproduces reads inside the
    # tensor and returns 0 past its end, so the oracle is given a zero-padded backing buffer.
    backing = np.zeros(2 * k + 128, np.float32)
    backing[:2 * k] = synth.uniform("gpu", f"ragx{dtype}_{n}_{k}", (2 * k,))
    x = backing[:2 * k].reshape(2, k)
    w = cuda.register(raw, dtype, n, k)
    want = oracle.qmatmul(dtype, x, raw, 2, k, n)
    for mode in (Mode.REF_ORDER, Mode.ACT_F32):
        got = dev.qmatmul(to_dev(x), w, mode).cpu().numpy()
        if k % 256:
            assert np.array_equal(bits(got), bits(want)), mode
        else:
            assert np.allclose(got, want, rtol=0, atol=1e-3 * np.abs(want).max())
    cuda.release(w)


def test_golden_vectors_through_the_c_abi(oracle, cuda):
    """Outputs recorded from the reference's own compiled C, reproduced bit for bit by the CUDA path."""
    from sharpmind_b200.ops import QuantizationOps

    q = QuantizationOps(cuda)
    gold = np.load(GOLDEN)
    for key in gold.files:
        if not key.startswith("out_"):
            continue
        _, dtype, n, k = key.split("_")
        dtype, n, k = int(dtype), int(n), int(k)
        nbytes = oracle.raw_bytes(dtype, n, k)
        raw = _random_raw(dtype, nbytes + 256, f"gold{dtype}_{n}_{k}")[:nbytes].copy()
        x = synth.uniform("pins", f"goldx{dtype}_{n}_{k}", (k,))
        w = cuda.register(raw, dtype, n, k)
        fn = {Q8_0: q.VecDotQ8_0, Q4_K: q.VecDotQ4K, Q6_K: q.VecDotQ6K}[dtype]
        got = np.array([fn(x, raw, c, k) for c in range(n)], np.float32)
        assert np.array_equal(bits(got), bits(gold[key])), key
        cuda.release(w)


def test_known_answer_blocks_through_the_c_abi(cuda):
    # VecDotTests.cs:87-172
    from sharpmind_b200.ops import QuantizationOps

    q = QuantizationOps(cuda)
    b8 = np.zeros(34, np.uint8); b8[1], b8[2] = 0x40, 0x03
    b4 = np.zeros(144, np.uint8); b4[1], b4[4], b4[16] = 0x3C, 0x11, 0x01
    b6 = np.zeros(210, np.uint8); b6[209] = 0x3C
    for raw, dtype, fn, want in ((b8, Q8_0, q.VecDotQ8_0, 6.0), (b4, Q4_K, q.VecDotQ4K, 17.0), (b6, Q6_K, q.VecDotQ6K, 0.0)):
        w = cuda.register(raw, dtype, 1, 1)
        assert fn(np.array([1.0], np.float32), raw, 0, 1) == want
        cuda.release(w)


def test_host_slot_equals_device_path_and_guards(oracle, cuda, dev):
    from sharpmind_b200 import ops

    n, k, m = 192, 1024, 3
    raw = make_weight(oracle, Q8_0, n, k, "slot")
    x = synth.normal("gpu", "slotx", (m, k))
    w = cuda.register(raw, Q8_0, n, k)
    for mode in (ops.Mode.ACT_F32, ops.Mode.ACT_Q8, ops.Mode.REF_ORDER):
        q = ops.QuantizationOps(cuda, mode)
        out = np.zeros((m, n), np.float32)
        q.QuantizedMatMulQ8_0(x, raw, out, m, k, n)
        ref = dev.qmatmul(to_dev(x), w, mode).cpu().numpy()
        assert np.array_equal(bits(out), bits(ref))
    # page-locked caller buffers are copied from / to directly, pageable ones through the bounce buffer: same bits
    import torch

    q = ops.QuantizationOps(cuda, ops.Mode.ACT_Q8)
    ref = dev.qmatmul(to_dev(x), w, ops.Mode.ACT_Q8).cpu().numpy()
    for pin_in in (False, True):
        for pin_out in (False, True):
            xi = torch.from_numpy(x).pin_memory().numpy() if pin_in else x.copy()
            oo = torch.zeros((m, n), dtype=torch.float32).pin_memory().numpy() if pin_out else np.zeros((m, n), np.float32)
            q.QuantizedMatMulQ8_0(xi, raw, oo, m, k, n)
            assert np.array_equal(bits(oo), bits(ref)), (pin_in, pin_out)
    # an ordinary array page-locked in place through the library (what a host without the CUDA runtime does)
    xi, oo = x.copy(), np.zeros((m, n), np.float32)
    q.QuantizedMatMulQ8_0(xi, raw, oo, m, k, n)   # seen as pageable first: the remembered answer must not stick
    cuda.host_register(xi), cuda.host_register(oo)
    oo[:] = 0
    q.QuantizedMatMulQ8_0(xi, raw, oo, m, k, n)
    assert np.array_equal(bits(oo), bits(ref))
    cuda.host_unregister(xi), cuda.host_unregister(oo)
    oo[:] = 0
    q.QuantizedMatMulQ8_0(xi, raw, oo, m, k, n)
    assert np.array_equal(bits(oo), bits(ref))
    q = ops.QuantizationOps(cuda)
    out = np.zeros((m, n), np.float32)
    with pytest.raises(ops.InvalidOperationException):  # shape does not match the registration
        q.QuantizedMatMulQ8_0(x, raw, np.zeros((m, n - 32), np.float32), m, k, n - 32)
    with pytest.raises(ops.InvalidOperationException):  # never registered
        q.QuantizedMatMulQ8_0(x, raw.copy(), out, m, k, n)
    with pytest.raises(ops.InvalidOperationException):  # byte count guard on arrival
        cuda.register(raw[:-34], Q8_0, n, k)
    with pytest.raises(ops.ArgumentOutOfRangeException):
        q.VecDotQ8_0(x[0], raw, n, k)
    cuda.release(w)
    w2 = cuda.register(raw, Q8_0, n, k, repack=False)
    with pytest.raises(ops.NotSupportedException):
        dev.qmatmul(to_dev(x), w2, ops.Mode.ACT_Q8)
    cuda.release(w2)
    # M = 0 is a no-op
    w3 = cuda.register(raw, Q8_0, n, k)
    assert dev.qmatmul(to_dev(np.zeros((0, k), np.float32)), w3).shape == (0, n)
    cuda.release(w3)


def test_repeated_launches_are_bit_identical(oracle, cuda, dev):
    """Race check: the same launch repeated gives the same bits."""
    from sharpmind_b200.ops import Mode

    raw = make_weight(oracle, Q4_K, 512, 4096, "race")
    w = cuda.register(raw, Q4_K, 512, 4096)
    x = to_dev(synth.normal("gpu", "racex", (4, 4096)))
    for mode in (Mode.ACT_F32, Mode.ACT_Q8):
        first = dev.qmatmul(x, w, mode).cpu().numpy()
        for _ in range(5):
            assert np.array_equal(bits(dev.qmatmul(x, w, mode).cpu().numpy()), bits(first))
    cuda.release(w)


def test_llama8b_ffn_shapes_sampled_rows_and_linearity(oracle, cuda, dev):
    """Full-size Llama-3-8B FFN matrices: weights quantised on device, sampled rows against the
    oracle, and linearity (W(a*x + y) = a*Wx + Wy) as the size-independent property."""
    import torch

    from sharpmind_b200.ops import Mode

    for dtype, n, k in ((Q4_K, 14336, 4096), (Q6_K, 4096, 14336)):
        g = torch.Generator(device="cuda").manual_seed(1234 + dtype)
        wf = torch.randn((n, k), generator=g, device="cuda", dtype=torch.float32) * 0.02
        raw_d = dev.quantize_weights(dtype, wf)
        raw = raw_d.cpu().numpy()
        del wf
        w = cuda.register(raw, dtype, n, k, keep_raw=False)
        x = synth.normal("gpu", f"full{dtype}", (2, k))
        rows = [0, 1, n // 2, n - 1]
        for mode in (Mode.ACT_F32,):
            got = dev.qmatmul(to_dev(x), w, mode).cpu().numpy()
            for r in rows:
                want = oracle.qmatmul(dtype, x, raw, 2, k, n, cols=(r, r + 1))[:, r]
                wrow = oracle.dequantize(dtype, raw[r * (len(raw) // n):(r + 1) * (len(raw) // n)], k)
                tol = 1e-5 * np.linalg.norm(wrow) * np.linalg.norm(x, axis=1)
                assert np.all(np.abs(got[:, r] - want) <= tol)
        # one row over a matrix this large also goes through the digit planes; the fp32 one-row kernel is the option-off form
        one = dev.qmatmul(to_dev(x[:1]), w, Mode.ACT_F32).cpu().numpy()
        cuda.set_option("f32_one_row_digits_min_mb", 0)
        try:
            plain = dev.qmatmul(to_dev(x[:1]), w, Mode.ACT_F32).cpu().numpy()
        finally:
            cuda.set_option("f32_one_row_digits_min_mb", 32)
        assert np.array_equal(bits(one), bits(plain)) == (len(raw) < (32 << 20))  # the 33.0 MB Q4_K matrix is just below the limit
        for r in rows:
            want = oracle.qmatmul(dtype, x[:1], raw, 1, k, n, cols=(r, r + 1))[0, r]
            wrow = oracle.dequantize(dtype, raw[r * (len(raw) // n):(r + 1) * (len(raw) // n)], k)
            tol = 1e-5 * np.linalg.norm(wrow) * np.linalg.norm(x[0])
            assert abs(one[0, r] - want) <= tol and abs(plain[0, r] - want) <= tol
        a = np.float32(0.5)
        xs = to_dev(np.stack([x[0], x[1], a * x[0] + x[1]]))
        y = dev.qmatmul(xs, w, Mode.ACT_F32).cpu().numpy().astype(np.float64)
        scale = np.abs(y).max()
        assert np.max(np.abs(a * y[0] + y[1] - y[2])) <= 2e-5 * scale
        cuda.release(w)
