"""Parity of the fp32 ops around the matmuls with the CPU oracle, through the C ABI.

Bars: norms / softmax / SiLU-gate within 1e-5 relative; RoPE, residual add, argmax, embedding gather
and the weight quantisers bit-exact (same operations, same roundings).
"""
import numpy as np
import pytest

from sharpmind_b200 import synth
from tests.gpu_util import Q4_K, Q6_K, Q8_0, bits, to_dev

pytestmark = pytest.mark.gpu


def rel_ok(got, want, tol=1e-5, floor=1e-30):
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    return np.all(np.abs(got - want) <= tol * np.maximum(np.abs(want), floor) + 1e-37)


# ---------------------------------------------------------------- weight quantisers (bit exact)
@pytest.mark.parametrize("dtype", [Q8_0, Q4_K, Q6_K])
def test_weight_quantisers_match_oracle_bytes(oracle, dev, dtype):
    w = synth.normal("gpuq", f"w{dtype}", (64, 1024), 0.02)
    w[3, :256] = 0.0            # an all-zero block
    w[5, 256:288] = 0.0123      # a flat 32-element sub-block (Q4_K leaves its codes at zero)
    w[7, 512:528] = 0.0         # an all-zero 16-group inside a live block (Q6_K code 32)
    w[9, :] = synth.uniform("gpuq", f"u{dtype}", (1024,))
    got = dev.quantize_weights(dtype, to_dev(w)).cpu().numpy()
    want = oracle.quantize(dtype, w)
    assert got.size == want.size
    assert np.array_equal(got, want), np.flatnonzero(got != want)[:10]


def test_weight_quantiser_rejects_ragged_length(dev):
    import torch

    from sharpmind_b200 import ops

    with pytest.raises(ops.InvalidOperationException):
        dev.quantize_weights(Q4_K, torch.zeros(300, device="cuda"))
    with pytest.raises(ops.InvalidOperationException):
        dev.quantize_weights(Q8_0, torch.zeros(40, device="cuda"))


# ---------------------------------------------------------------- RMSNorm
@pytest.mark.parametrize("rows,n", [(64, 4096), (1, 1024), (24, 128), (5, 100), (3, 2), (2, 5000), (1, 14336)])
def test_rmsnorm(oracle, dev, rows, n):
    x = synth.normal("gpue", f"rx{rows}_{n}", (rows, n))
    w = synth.normal("gpue", f"rw{n}", (n,), 0.1, 1.0)
    want = oracle.rmsnorm(x, w, 1e-6)
    got = dev.rmsnorm(to_dev(x), to_dev(w), 1e-6).cpu().numpy()
    assert rel_ok(got, want)
    xd = to_dev(x)  # in place, as the final norm runs
    dev.rmsnorm(xd, to_dev(w), 1e-6, out=xd)
    assert np.array_equal(bits(xd.cpu().numpy()), bits(got))


def test_rmsnorm_reference_unit_cases(dev):
    # ActivationTests.cs: RMSNorm_UnitWeights_NormalisesInput / RMSNorm_WeightScales
    r = dev.rmsnorm(to_dev(np.array([[3, 4]], np.float32)), to_dev(np.ones(2, np.float32)), 0.0).cpu().numpy()
    assert abs(np.sqrt(np.mean(r * r)) - 1) < 1e-4
    r = dev.rmsnorm(to_dev(np.ones((1, 4), np.float32)), to_dev(np.full(4, 2, np.float32)), 0.0).cpu().numpy()
    assert np.allclose(r, 2, atol=1e-4)


def test_rmsnorm_row_slot(oracle, cuda):
    from sharpmind_b200.ops import ActivationOps

    a = ActivationOps(cuda)
    src = synth.normal("gpue", "rrs", (333,))
    w = synth.normal("gpue", "rrw", (333,), 0.1, 1.0)
    inv = oracle.rmsnorm_param(src, 1e-6)
    dst = np.zeros(333, np.float32)
    a.ApplyRMSNormRow(src, w, dst, inv)
    assert np.array_equal(bits(dst), bits(oracle.rmsnorm_row(src, w, inv)))


# ---------------------------------------------------------------- SwiGLU / SiLU
@pytest.mark.parametrize("rows,F", [(64, 14336), (1, 3072), (3, 37)])
def test_swiglu(oracle, dev, rows, F):
    gu = synth.normal("gpue", f"gu{rows}_{F}", (rows, 2 * F))
    want = oracle.swiglu(np.ascontiguousarray(gu[:, :F]), np.ascontiguousarray(gu[:, F:]))
    got = dev.swiglu_fused(to_dev(gu), F).cpu().numpy()
    assert rel_ok(got, want, floor=1e-6)
    got2 = dev.swiglu(to_dev(np.ascontiguousarray(gu[:, :F])), to_dev(np.ascontiguousarray(gu[:, F:]))).cpu().numpy()
    assert np.array_equal(bits(got2), bits(got))


def test_silu_and_slots(oracle, cuda, dev):
    from sharpmind_b200.ops import ActivationOps

    x = synth.normal("gpue", "silu", (1000,), 3.0)
    want = oracle.silu(x)
    assert rel_ok(dev.silu(to_dev(x)).cpu().numpy(), want, floor=1e-6)
    a = ActivationOps(cuda)
    dst = np.zeros(1000, np.float32)
    a.ApplyPointwise(x, dst)
    assert rel_ok(dst, want, floor=1e-6)
    assert dev.silu(to_dev(np.zeros(4, np.float32))).cpu().numpy().tolist() == [0, 0, 0, 0]
    u = synth.normal("gpue", "silu_u", (1000,))
    a.ApplyGate(x, u, dst)
    assert rel_ok(dst, oracle.swiglu(x, u), floor=1e-6)


# ---------------------------------------------------------------- softmax
@pytest.mark.parametrize("rows,n", [(64, 128256), (3, 1000), (2, 7), (1, 151936), (4, 4096)])
def test_softmax(oracle, dev, rows, n):
    x = synth.normal("gpue", f"sm{rows}_{n}", (rows, n), 2.0)
    got = dev.softmax(to_dev(x)).cpu().numpy()
    if rows * n > 2_000_000:
        check = [0, rows // 2, rows - 1]
    else:
        check = range(rows)
    # The scalar reference adds n exponentials one after another in fp32, so its own normaliser
    # carries about sqrt(n) * 2^-24 of rounding noise (1.2e-5 at n = 128256).  The CUDA kernel is
    # held to 1e-5 against the exact (fp64) softmax, and to 1e-5 plus that noise against the oracle.
    noise = np.sqrt(n) * 2.0 ** -24
    for r in check:
        want = oracle.softmax_rows(x[r])
        assert rel_ok(got[r], want, tol=1e-5 + noise, floor=1e-12), r
        z = x[r].astype(np.float64)
        e = np.exp(z - z.max())
        assert rel_ok(got[r], e / e.sum(), tol=1e-5, floor=1e-12), r
    assert np.allclose(got.sum(axis=1, dtype=np.float64), 1.0, atol=1e-5)


def test_softmax_reference_properties(cuda, dev):
    from sharpmind_b200.ops import ActivationOps

    r = dev.softmax(to_dev(np.array([[1000, 1001, 1002]], np.float32))).cpu().numpy()
    assert abs(r.sum() - 1) < 1e-4 and not np.isnan(r).any()
    r = dev.softmax(to_dev(np.array([[1, 2, 3, 4]], np.float32))).cpu().numpy()[0]
    assert abs(r.sum() - 1) < 1e-5 and np.all(np.diff(r) > 0)
    a = ActivationOps(cuda)
    out = a.Softmax(np.array([[1, 2, 3], [4, 5, 6]], np.float32))
    assert np.allclose(out.sum(axis=1), 1, atol=1e-5)


# ---------------------------------------------------------------- RoPE (bit exact: same tables, same ops)
@pytest.mark.parametrize("neox", [False, True])
def test_rope_llama3_shape(oracle, dev, neox):
    seq, heads, hd, theta = 64, 32, 128, 500000.0
    x = synth.normal("gpue", f"rope{neox}", (seq, heads, hd))
    cos, sin = oracle.rope_tables(theta, hd, 128)
    dcos, dsin = dev.rope_tables(theta, hd, 128)
    assert np.array_equal(bits(dcos.cpu().numpy()), bits(cos)) and np.array_equal(bits(dsin.cpu().numpy()), bits(sin))
    for off in (0, 17):
        want = oracle.rope_apply(x, off, cos, sin, neox)
        got = dev.rope(to_dev(x), off, dcos, dsin, neox).cpu().numpy()
        assert np.array_equal(bits(got), bits(want))


def test_rope_reference_unit_cases(dev):
    # RoPETests.cs:44-79, RoPEConventionTests.cs:34-67
    from sharpmind_b200 import ops

    cos, sin = dev.rope_tables(10000.0, 4, 8)
    x = dev.rope(to_dev(np.array([[[1, 2, 3, 4]]], np.float32)), 1, cos, sin, False).cpu().numpy()[0, 0]
    th2 = float(np.float32(10000.0) ** np.float32(-0.5))
    want = [np.cos(1.0) - 2 * np.sin(1.0), 2 * np.cos(1.0) + np.sin(1.0),
            3 * np.cos(th2) - 4 * np.sin(th2), 4 * np.cos(th2) + 3 * np.sin(th2)]
    assert np.allclose(x, want, atol=5e-6)
    x = dev.rope(to_dev(np.array([[[1, 2, 3, 4]]], np.float32)), 1, cos, sin, True).cpu().numpy()[0, 0]
    c0, s0, c1, s1 = np.cos(1.0), np.sin(1.0), np.cos(th2), np.sin(th2)
    assert np.allclose(x, [c0 - 3 * s0, 2 * c1 - 4 * s1, 3 * c0 + s0, 4 * c1 + 2 * s1], atol=5e-5)
    x = dev.rope(to_dev(np.array([[[1, 2, 3, 4]]], np.float32)), 0, cos, sin, True).cpu().numpy()[0, 0]
    assert x.tolist() == [1, 2, 3, 4]
    with pytest.raises(ops.ArgumentOutOfRangeException):  # Apply_ExceedsMaxSeqLen_Throws
        dev.rope(to_dev(np.ones((5, 1, 4), np.float32)), 4, cos, sin, False)


# ---------------------------------------------------------------- add / argmax / embedding
def test_residual_add(oracle, dev):
    for n in (64 * 4096, 1024, 7):
        a = synth.normal("gpue", f"adda{n}", (n,))
        b = synth.normal("gpue", f"addb{n}", (n,))
        got = dev.add_(to_dev(a), to_dev(b)).cpu().numpy()
        assert np.array_equal(bits(got), bits(oracle.add(a, b)))


def test_argmax_first_maximum_wins(oracle, dev):
    x = synth.normal("gpue", "am", (5, 151936))
    x[1, 77] = x[1, 150000] = 99.0     # tie: the lower index must win
    x[2, 0] = 50.0
    x[3, 151935] = 50.0
    got = dev.argmax(to_dev(x)).cpu().numpy()
    assert got.tolist() == [oracle.argmax(x[r]) for r in range(5)]
    assert got[1] == 77
    assert dev.argmax(to_dev(np.array([[1, 5, 5, 2]], np.float32))).cpu().numpy().tolist() == [1]


def test_embedding_gather_is_the_dequantised_row(oracle, cuda, dev):
    vocab, H = 1000, 1024
    raw = oracle.quantize(Q8_0, synth.normal("gpue", "emb", (vocab, H), 0.02))
    table = oracle.dequantize(Q8_0, raw, vocab * H).reshape(vocab, H)
    tok = np.array([0, 999, 17, 17, 512], np.int32)
    for repack in (True, False):
        w = cuda.register(raw, Q8_0, vocab, H, repack=repack)
        got = dev.embed(w, to_dev(tok)).cpu().numpy()
        assert np.array_equal(bits(got), bits(table[tok]))
        cuda.release(w)


def test_empty_inputs_are_no_ops(dev):
    import torch

    e = torch.zeros((0, 128), device="cuda")
    w = torch.ones(128, device="cuda")
    assert dev.rmsnorm(e, w, 1e-6).shape == (0, 128)
    assert dev.softmax(e).shape == (0, 128)
    assert dev.silu(e).shape == (0, 128)


@pytest.mark.parametrize("rows,n", [(1, 1024), (3, 4096), (5, 1000), (2, 128), (4, 1026)])
def test_add_rmsnorm_equals_separate_launches(dev, rows, n):
    """The fused residual add + RMSNorm gives the bits of smc_add_dev followed by smc_rmsnorm_dev."""
    import ctypes as C

    import torch

    x = to_dev(synth.normal("gpue", f"arx{rows}_{n}", (rows, n)))
    y = to_dev(synth.normal("gpue", f"ary{rows}_{n}", (rows, n)))
    w = to_dev(synth.normal("gpue", f"arw{n}", (n,), 0.1, 1.0))
    x1 = x.clone()
    dev.add_(x1, y)
    want = dev.rmsnorm(x1, w, 1e-6)
    x2, out = x.clone(), torch.empty_like(x)
    ctx = dev.ctx
    ctx.check(ctx.lib.smc_add_rmsnorm_dev(ctx.h, x2.data_ptr(), y.data_ptr(), w.data_ptr(), out.data_ptr(), rows, n,
                                          C.c_float(1e-6), C.c_void_p(torch.cuda.current_stream().cuda_stream)))
    assert torch.equal(x1, x2)
    assert torch.equal(out, want)


@pytest.mark.parametrize("rows,n,with_add", [(1, 1024, True), (7, 4096, True), (33, 2560, True), (5, 1024, False), (300, 8192, True)])
def test_add_rmsnorm_q8_equals_separate_launches(dev, rows, n, with_add):
    """Residual add + RMSNorm + Q8_0 row quantiser in one pass: the quants and fp16 scales are those of the separate
    kernels, and so are the per-block sums the Q4_K / Q6_K matmuls read (checked through a matmul of each format)."""
    import ctypes as C

    import torch

    from sharpmind_b200 import ops

    ctx = dev.ctx
    x = to_dev(synth.normal("gpue", f"aqx{rows}_{n}", (rows, n)))
    y = to_dev(synth.normal("gpue", f"aqy{rows}_{n}", (rows, n))) if with_add else None
    w = to_dev(synth.normal("gpue", f"aqw{n}", (n,), 0.1, 1.0))
    x1 = x.clone()
    if with_add:
        dev.add_(x1, y)
    normed = dev.rmsnorm(x1, w, 1e-6)
    want = ops.Q8Act(ctx, rows, n)
    dev.quantize_q8(normed, want, n)
    x2, out = x.clone(), torch.empty_like(x)
    got = dev.add_rmsnorm_q8(x2, y, w, 1e-6, ops.Q8Act(ctx, rows, n), out=out)
    assert torch.equal(x1, x2) and torch.equal(out, normed)
    (wq, wd), (gq, gd) = want.read(), got.read()
    assert np.array_equal(wq, gq) and np.array_equal(wd, gd)
    got2 = dev.add_rmsnorm_q8(x.clone(), y, w, 1e-6, ops.Q8Act(ctx, rows, n))  # without the fp32 copy
    assert np.array_equal(got2.read()[0], wq)
    for dtype in (8, 12, 14):
        mat = ctx.register_dev(dev.quantize_weights(dtype, to_dev(synth.normal("gpue", f"aqm{dtype}_{n}", (64, n), 0.05))), dtype, 64, n)
        assert torch.equal(dev.qmatmul_q8(got2, mat), dev.qmatmul_q8(want, mat)), dtype
        ctx.release(mat)
    with pytest.raises(Exception):  # rows that are not whole 32-element blocks keep to the separate kernels
        dev.add_rmsnorm_q8(to_dev(np.zeros((2, 1000), np.float32)), None, to_dev(np.ones(1000, np.float32)), 1e-6, ops.Q8Act(ctx, 2, 1024))


@pytest.mark.parametrize("rows,F", [(1, 3072), (5, 1024), (33, 14336), (300, 3072), (2, 32)])
def test_swiglu_quantize_q8_equals_separate_launches(dev, rows, F):
    """SiLU(gate) * up and the Q8_0 row quantiser in one pass (16-byte accesses for batches, one lane per value for a
    block or two): quants and scales of the separate kernels, and their block sums through a matmul of each format."""
    import torch

    from sharpmind_b200 import ops

    ctx = dev.ctx
    gu = to_dev(synth.normal("gpue", f"sq{rows}_{F}", (rows, 2 * F), 1.5))
    want = ops.Q8Act(ctx, rows, F)
    dev.quantize_q8(dev.swiglu_fused(gu, F), want, F)
    got = dev.swiglu_quantize_q8(gu, F, ops.Q8Act(ctx, rows, F))
    (wq, wd), (gq, gd) = want.read(), got.read()
    assert np.array_equal(wq, gq) and np.array_equal(wd, gd)
    if F % 256 == 0:
        for dtype in (8, 12, 14):
            mat = ctx.register_dev(dev.quantize_weights(dtype, to_dev(synth.normal("gpue", f"sqm{dtype}_{F}", (32, F), 0.05))), dtype, 32, F)
            assert torch.equal(dev.qmatmul_q8(got, mat), dev.qmatmul_q8(want, mat)), dtype
            ctx.release(mat)


def test_argmax_first_maximum_over_chunks(dev):
    import torch

    logits = to_dev(synth.normal("gpue", "amx", (5, 151936)))
    logits[1, 70000] = 50.0
    logits[1, 150000] = 50.0   # a later tie: the first one wins
    logits[2, 0] = 60.0
    logits[3, 151935] = 60.0
    logits[4, :] = -3.0        # all equal: index 0
    got = dev.argmax(logits).cpu().numpy()
    want = logits.cpu().numpy().argmax(axis=1)
    assert got.tolist() == want.tolist()
    assert got[1] == 70000 and got[4] == 0
    small = to_dev(synth.normal("gpue", "ams", (7, 100)))
    assert dev.argmax(small).cpu().numpy().tolist() == small.cpu().numpy().argmax(axis=1).tolist()


@pytest.mark.parametrize("dtype,n,k", [(Q8_0, 1024, 2048), (Q8_0, 256, 3072), (Q4_K, 512, 2048), (Q6_K, 600, 8192), (Q4_K, 300, 14336), (Q8_0, 200, 9216)])
def test_fused_one_row_matmuls(oracle, cuda, dev, dtype, n, k):
    """SiLU-gate and residual add + RMSNorm folded into the staging of a one-row matmul, against the separate kernels."""
    import ctypes as C

    import torch

    from sharpmind_b200.ops import Mode

    raw = oracle.quantize(dtype, synth.normal("gpue", f"fw{dtype}_{n}_{k}", (n, k), 0.02))
    w = cuda.register(raw, dtype, n, k)
    st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    lib, h = cuda.lib, cuda.h
    # SwiGLU prologue: same bits as swiglu followed by the quantised-activation matmul
    gu = to_dev(synth.normal("gpue", f"fgu{k}", (1, 2 * k)))
    act = dev.swiglu_fused(gu, k)
    want = dev.qmatmul(act, w, Mode.ACT_Q8)
    got = torch.empty_like(want)
    cuda.check(lib.smc_qmatmul_swiglu_dev(h, gu.data_ptr(), gu.data_ptr() + 4 * k, w.handle, got.data_ptr(), st))
    assert torch.equal(got, want)
    if k > 9216:  # the norm prologue keeps a thread's chunks in registers: rows up to 9216
        cuda.release(w)
        return
    # add + norm prologue: the stream sum has the bits of the add kernel; the matmul agrees to rounding
    x = to_dev(synth.normal("gpue", f"fx{k}", (1, k)))
    y = to_dev(synth.normal("gpue", f"fy{k}", (1, k)))
    nw = to_dev(synth.normal("gpue", f"fn{k}", (k,), 0.1, 1.0))
    xs = x.clone()
    dev.add_(xs, y)
    want = dev.qmatmul(dev.rmsnorm(xs, nw, 1e-6), w, Mode.ACT_Q8)
    got, summ = torch.empty_like(want), torch.empty_like(x)
    cuda.check(lib.smc_qmatmul_addnorm_dev(h, x.data_ptr(), y.data_ptr(), nw.data_ptr(), C.c_float(1e-6), summ.data_ptr(),
                                           w.handle, got.data_ptr(), st))
    assert torch.equal(summ, xs)
    scale = want.abs().max().item()
    assert (got - want).abs().max().item() <= 2e-2 * scale
    # without an addend it is the plain norm
    want = dev.qmatmul(dev.rmsnorm(x, nw, 1e-6), w, Mode.ACT_Q8)
    cuda.check(lib.smc_qmatmul_addnorm_dev(h, x.data_ptr(), None, nw.data_ptr(), C.c_float(1e-6), None, w.handle,
                                           got.data_ptr(), st))
    assert (got - want).abs().max().item() <= 2e-2 * want.abs().max().item()
    cuda.release(w)


# ------------------------------------------------------------------------------------------ sampler
@pytest.mark.parametrize("n", [1000, 151936])
@pytest.mark.parametrize("cfg", [
    dict(temperature=1.0, top_k=0, top_p=1.0, min_p=0.0),
    dict(temperature=0.7, top_k=40, top_p=1.0, min_p=0.0),
    dict(temperature=0.8, top_k=0, top_p=0.9, min_p=0.0),
    dict(temperature=1.3, top_k=50, top_p=0.95, min_p=0.05),
    dict(temperature=0.0, top_k=40, top_p=0.9, min_p=0.0),     # greedy shortcut
    dict(temperature=1.0, top_k=1, top_p=1.0, min_p=0.0),      # top-1 = argmax whatever the draw
])
def test_sampler_matches_reference_given_the_same_uniform(oracle, cuda, dev, n, cfg):
    """Sampler.Sample: with the host's uniform number r handed in, the device picks the token whose interval of the
    cumulative distribution contains r.  The reference finds it with a sequential fp32 running sum, whose value after
    i terms is off the exact sum by up to about i * 2^-24 relative (1e-5 at 152k tokens, several tokens wide where each
    holds 1e-5 of the mass); the device's fixed summation tree rounds differently.  So the contract is stated on the
    reference's own probabilities, summed exactly: cum(i - 1) - tol <= r <= cum(i) + tol with tol = 3e-5 (the fp32
    uncertainty of either side), the picked token must have kept its mass, and the reference's own pick satisfies the
    same inequality.  For short rows, and whenever top-k leaves few candidates, this means the same token."""
    rows = 24
    logits = synth.normal("sampler", f"l{n}", (rows, n), 2.0)
    r = synth.uniform("sampler", f"r{n}", (rows,), 0.0, 1.0).astype(np.float32)
    got = dev.sample(to_dev(logits), uniform=to_dev(r), **cfg).cpu().numpy()
    args = (cfg["temperature"], cfg["top_k"], cfg["top_p"], cfg["min_p"])
    same = 0
    for i in range(rows):
        if cfg["temperature"] <= 0:
            assert int(got[i]) == oracle.sample(logits[i], *args, float(r[i]))
            same += 1
            continue
        want, probs = oracle.sample_probs(logits[i], *args, float(r[i]))
        cum = np.cumsum(probs.astype(np.float64))
        tol = 3e-5
        for tok in (int(got[i]), want):
            assert probs[tok] > 0
            lo = cum[tok - 1] if tok > 0 else 0.0
            assert lo - tol <= float(r[i]) <= cum[tok] + tol, (i, tok, lo, float(r[i]), cum[tok])
        same += int(got[i]) == want
    if n <= 1000 or 0 < cfg["top_k"] <= 50:
        assert same == rows, f"{same}/{rows} rows picked the reference's token"


def test_sampler_guards_and_repetition_penalty(oracle, cuda, dev):
    n = 4096
    logits = synth.normal("sampler", "guard", (3, n), 2.0)
    logits[1, 77] = np.inf          # the softmax guard: a point mass on token 0
    logits[2, 5] = np.nan
    r = np.array([0.3, 0.9, 0.1], np.float32)
    got = dev.sample(to_dev(logits), 1.0, uniform=to_dev(r)).cpu().numpy()
    assert got[1] == 0 and got[2] == 0
    assert got[0] == oracle.sample(logits[0], 1.0, 0, 1.0, 0.0, 0.3)
    # repetition penalty: distinct ids scale once, out-of-range ids and padding are skipped
    ids = np.array([[5, 9, 5, 4095, -1, 7000, 9], [1, 1, 1, 2, -1, -1, -1], [0, 3, 3, 3, 3, 3, 3]], np.int32)
    base = synth.normal("sampler", "rep", (3, n), 2.0)
    x = to_dev(base.copy())
    dev.repetition_penalty_(x, to_dev(ids), 1.3)
    out = x.cpu().numpy()
    for i in range(3):
        want = oracle.repetition_penalty(base[i], ids[i], 1.3)
        assert np.array_equal(out[i].view(np.uint32), want.view(np.uint32))


@pytest.mark.parametrize("dtype,ffn,k", [(Q4_K, 1184, 2048), (Q4_K, 7168, 4096), (Q6_K, 333, 2048), (Q8_0, 1536, 1024), (Q8_0, 5, 3072)])
def test_gate_up_interleaved_with_the_activation_in_the_epilogue(oracle, cuda, dev, dtype, ffn, k):
    """gate and up woven row by row, one launch gives SiLU(gate . x) * (up . x): the bits of the two matmuls followed by
    the SwiGLU kernel, whatever the grid; the woven matrix itself is rows 2i = gate i, 2i + 1 = up i of every layout."""
    import torch

    from sharpmind_b200.ops import Mode

    g_raw = oracle.quantize(dtype, synth.normal("gpue", f"pg{dtype}_{ffn}_{k}", (ffn, k), 0.02))
    u_raw = oracle.quantize(dtype, synth.normal("gpue", f"pu{dtype}_{ffn}_{k}", (ffn, k), 0.02))
    wg, wu = cuda.register(g_raw, dtype, ffn, k, keep_raw=True), cuda.register(u_raw, dtype, ffn, k, keep_raw=True)
    woven = dev.interleave_rows(wg, wu)
    x = to_dev(synth.normal("gpue", f"px{k}", (1, k)))
    want = dev.swiglu(dev.qmatmul(x, wg, Mode.ACT_Q8), dev.qmatmul(x, wu, Mode.ACT_Q8))
    got = dev.qmatmul_swiglu_pairs(x, woven)
    assert torch.equal(got, want)
    for ctas in (1 if ffn <= 2048 else 5, 7, 148):  # (one CTA parks all row sums in shared memory: small matrices only)
        cuda.set_option("gemv_ctas", ctas)
        try:
            again = dev.qmatmul_swiglu_pairs(x, woven)
        finally:
            cuda.set_option("gemv_ctas", 0)
        assert torch.equal(again, want), ctas
    # the woven matrix as a plain matmul (reference order reads its GGUF copy): outputs alternate gate, up
    both = dev.qmatmul(x, woven, Mode.REF_ORDER)
    assert torch.equal(both[0, 0::2], dev.qmatmul(x, wg, Mode.REF_ORDER)[0]) and torch.equal(both[0, 1::2], dev.qmatmul(x, wu, Mode.REF_ORDER)[0])
    # against the oracle: matmuls on the dequantised activation row, then the scalar SwiGLU
    xq = oracle.quantize_rows_q8_0(x.cpu().numpy(), 1, k)
    xhat = oracle.dequantize(Q8_0, xq[0], k)[None, :]
    ref = oracle.swiglu(oracle.qmatmul(dtype, xhat, g_raw, 1, k, ffn), oracle.qmatmul(dtype, xhat, u_raw, 1, k, ffn))
    assert np.max(np.abs(got.cpu().numpy() - ref)) <= 2e-5 * max(1.0, float(np.max(np.abs(ref))))
    for w_ in (wg, wu, woven):
        cuda.release(w_)
    assert cuda.device_status() == 0
