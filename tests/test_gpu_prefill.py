"""Prefill-sized Q4_K matmul on the tensor cores against the oracle's scalar vec-dot (fp32 activations).

Bound: 1e-5 * ||w_row|| * ||x_row|| per output, the same as the fp32-activation GEMV: the tensor-core path
multiplies exact integer weight parts with an fp16 (hi, lo) split of the activations.
"""
import numpy as np
import pytest

from sharpmind_b200 import ops, synth
from tests.gpu_util import Q4_K, row_norm_bound, to_dev

pytestmark = pytest.mark.gpu


def _case(oracle, cuda, dev, n, k, m, sigma_x=1.0, tag=""):
    wf = synth.normal("prefill", f"w{n}x{k}{tag}", (n, k), 0.02)
    raw = oracle.quantize(Q4_K, wf)
    x = synth.normal("prefill", f"x{m}x{k}{tag}", (m, k), sigma_x)
    w = cuda.register(raw, Q4_K, n, k)
    got = dev.qmatmul_tc(to_dev(x), w).cpu().numpy()
    assert cuda.device_status() == 0
    return raw, x, got, w


@pytest.mark.parametrize("n,k,m", [
    (128, 256, 128),     # one tile, one block
    (128, 1024, 128),    # several blocks: both accumulator buffers, stage reuse
    (256, 2048, 200),    # two row tiles, ragged token tile
    (384, 512, 1),       # a single token
    (128, 4096, 300),    # three token tiles
])
def test_tc_matmul_matches_oracle(oracle, cuda, dev, n, k, m):
    raw, x, got, w = _case(oracle, cuda, dev, n, k, m)
    want = oracle.qmatmul(Q4_K, x, raw, m, k, n)
    bound = row_norm_bound(oracle, Q4_K, raw, n, k, x)
    err = np.abs(got - want)
    assert np.all(err <= bound), float(np.max(err / bound))
    cuda.release(w)


@pytest.mark.parametrize("n,k", [(28672, 8192), (8192, 28672)])
def test_tc_matmul_llama70b_shapes_sampled_rows(oracle, cuda, dev, n, k):
    """The benchmarked prefill shapes (Llama-3-70B FFN, 512 tokens): weights drawn and quantised on the device, sampled
    weight rows (first, last, both sides of a 128-row tile edge, 16 random ones) against the oracle's scalar vec-dot
    on every token, at the same per-output bound as the small shapes (the bound scales with ||w|| ||x||, hence with K)."""
    import torch

    m = 512
    g = torch.Generator(device="cuda").manual_seed(n + 7 * k)
    raw_d = dev.quantize_weights(Q4_K, torch.randn((n, k), generator=g, device="cuda") * 0.02)
    w = cuda.register_dev(raw_d, Q4_K, n, k)
    x = synth.normal("prefill", f"x70b_{k}", (m, k))
    got = dev.qmatmul_tc(to_dev(x), w).cpu().numpy()
    assert cuda.device_status() == 0
    rs = np.random.default_rng(n)
    rows = sorted({0, n - 1, 127, 128, n // 2 - 1, n // 2} | set(int(r) for r in rs.integers(0, n, 16)))
    per_row = k // 256 * 144
    xn = np.linalg.norm(x.astype(np.float64), axis=1)
    worst = 0.0
    for r in rows:
        raw_row = raw_d[r * per_row:(r + 1) * per_row].cpu().numpy()
        want = oracle.qmatmul(Q4_K, x, raw_row, m, k, 1)[:, 0]
        wn = np.linalg.norm(oracle.dequantize(Q4_K, raw_row, k).astype(np.float64))
        bound = 1e-5 * wn * xn
        err = np.abs(got[:, r].astype(np.float64) - want)
        worst = max(worst, float(np.max(err / bound)))
        assert np.all(err <= bound), (r, worst)
    print(f"tcgen05 matmul {n}x{k}, 512 tokens: worst error {worst:.3f} of the bound over {len(rows)} sampled rows")
    cuda.release(w)


def test_tc_matmul_scaling_and_zero_rows(oracle, cuda, dev):
    """Rows of very different magnitude (per-token power-of-two scale) and an all-zero row."""
    n, k, m = 128, 512, 16
    wf = synth.normal("prefill", "wz", (n, k), 0.02)
    raw = oracle.quantize(Q4_K, wf)
    x = synth.normal("prefill", "xz", (m, k))
    x[1] *= 1e-6
    x[2] *= 3e5
    x[3] = 0.0
    w = cuda.register(raw, Q4_K, n, k)
    got = dev.qmatmul_tc(to_dev(x), w).cpu().numpy()
    want = oracle.qmatmul(Q4_K, x, raw, m, k, n)
    bound = row_norm_bound(oracle, Q4_K, raw, n, k, x)
    assert np.all(np.abs(got - want) <= bound + 1e-30)
    assert np.all(got[3] == 0.0)
    cuda.release(w)


def test_tc_matmul_agrees_with_gemv_path(oracle, cuda, dev):
    n, k, m = 256, 1024, 64
    raw, x, got, w = _case(oracle, cuda, dev, n, k, m, tag="g")
    ref = dev.qmatmul(to_dev(x), w, ops.Mode.ACT_F32).cpu().numpy()
    bound = 2 * row_norm_bound(oracle, Q4_K, raw, n, k, x)
    assert np.all(np.abs(got - ref) <= bound)
    cuda.release(w)


def test_tc_matmul_rejects_other_shapes(oracle, cuda, dev):
    raw = oracle.quantize(Q4_K, synth.normal("prefill", "wr", (64, 256), 0.02))
    w = cuda.register(raw, Q4_K, 64, 256)
    with pytest.raises(ops.NotSupportedException):
        dev.qmatmul_tc(to_dev(synth.normal("prefill", "xr", (4, 256))), w)
    cuda.release(w)


@pytest.mark.parametrize("n,k,m", [(256, 2048, 64), (128, 4096, 300), (384, 1024, 129)])
def test_quantised_activations_at_prefill_sizes_run_on_the_tensor_cores(oracle, cuda, dev, n, k, m):
    """SMC_ACT_Q8 over Q4_K at 64 rows and more: the Q8_0 activation rows go through the tcgen05 kernel (d * q is exact in
    its fp16 pairs).  Against the oracle on the dequantised rows at the mode's bound; against the int8 kernels of the same
    library (option off) to a few ulps of the row scale; and the two entry points (fp32 rows in, Q8 rows in) bit for bit."""
    raw = oracle.quantize(Q4_K, synth.normal("prefill", f"wq{n}x{k}", (n, k), 0.02))
    x = synth.normal("prefill", f"xq{m}x{k}", (m, k))
    w = cuda.register(raw, Q4_K, n, k)
    xd = to_dev(x)
    got = dev.qmatmul(xd, w, ops.Mode.ACT_Q8).cpu().numpy()
    xq = oracle.quantize_rows_q8_0(x, m, k)
    from tests.gpu_util import Q8_0
    xhat = np.stack([oracle.dequantize(Q8_0, xq[r], k) for r in range(m)])
    want = oracle.qmatmul(Q4_K, xhat, raw, m, k, n)
    bound = row_norm_bound(oracle, Q4_K, raw, n, k, xhat)
    assert np.all(np.abs(got - want) <= bound), float(np.max(np.abs(got - want) / bound))
    act = ops.Q8Act(cuda, m, k)
    dev.quantize_q8(xd, act, k)
    assert np.array_equal(dev.qmatmul_q8(act, w).cpu().numpy().view(np.uint32), got.view(np.uint32))
    cuda.set_option("q8_prefill_tensor_cores", 0)
    try:
        ints = dev.qmatmul_q8(act, w).cpu().numpy()
    finally:
        cuda.set_option("q8_prefill_tensor_cores", 1)
    assert np.all(np.abs(ints - got) <= bound)
    act.close()
    cuda.release(w)
    assert cuda.device_status() == 0
