"""Pins the CPU oracle before anything is compared against it.

Sources of truth, in order of strength:
  1. the reference's own C oracle (tools/ReferenceDataGenerator/vecdot_ref.c) compiled from the
     reference tree into oracle/_ref -- called directly when present;
  2. golden vectors produced with it (tests/golden/vecdot_golden.npz, made by
     tests/golden/make_golden.py) -- checked everywhere;
  3. the literal known-answer values in the reference's unit tests (cited per test).
"""
import os

import numpy as np
import pytest

from sharpmind_b200 import synth

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "vecdot_golden.npz")
Q8_0, Q4_K, Q6_K = 8, 12, 14


# ---- SharpMind.Tests/Quantization/VecDotTests.cs:87-172: single-block known answers --------
def test_known_answer_q8_0(oracle):
    block = np.zeros(34, np.uint8)
    block[0], block[1], block[2] = 0x00, 0x40, 0x03  # d = 2.0, q0 = 3
    assert oracle.vecdot(Q8_0, [1.0], block, 0, 1) == 6.0
    assert oracle.vecdot_fma(Q8_0, [1.0], block, 0, 1) == 6.0


def test_known_answer_q4_k(oracle):
    block = np.zeros(144, np.uint8)
    block[0], block[1] = 0x00, 0x3C  # d = 1.0
    block[4] = 0x11  # scale 17, min 0
    block[16] = 0x01  # first nibble = 1
    assert oracle.vecdot(Q4_K, [1.0], block, 0, 1) == 17.0
    assert oracle.vecdot_fma(Q4_K, [1.0], block, 0, 1) == 17.0


def test_known_answer_q6_k(oracle):
    block = np.zeros(210, np.uint8)
    block[208], block[209] = 0x00, 0x3C
    assert oracle.vecdot(Q6_K, [1.0], block, 0, 1) == 0.0
    assert oracle.vecdot_fma(Q6_K, [1.0], block, 0, 1) == 0.0


# ---- SharpMind.Tests/Quantization/HalfToFloatTests.cs:11-28 --------------------------------
@pytest.mark.parametrize("half,bits", [
    (0x0000, 0x00000000), (0x8000, 0x80000000), (0x3C00, 0x3F800000), (0xBC00, 0xBF800000),
    (0x3800, 0x3F000000), (0x4000, 0x40000000), (0x7BFF, 0x477FE000), (0x0400, 0x38800000),
    (0x0001, 0x33800000), (0x03FF, 0x387FC000), (0x1955, 0x3B2AA000), (0x67FF, 0x44FFE000),
])
def test_half_to_float_bit_patterns(oracle, half, bits):
    assert oracle.half_bits_to_float_bits(half) == bits


# ---- SharpMind.Tests/Quantization/HalfWideningTests.cs:17-51: all 65 536 patterns ----------
def test_half_to_float_all_patterns(oracle):
    halves = np.arange(65536, dtype=np.uint16)
    want = halves.view(np.float16).astype(np.float32).view(np.uint32)
    got = np.array([oracle.half_bits_to_float_bits(int(h)) for h in halves], dtype=np.uint32)
    nan = np.isnan(halves.view(np.float16))
    assert np.array_equal(got[~nan], want[~nan])
    assert np.all(np.isnan(got[nan].view(np.float32)))


def test_float_to_half_is_round_to_nearest_even(oracle):
    g = synth.rng("pins", "f2h")
    vals = np.concatenate([
        g.standard_normal(20000).astype(np.float32) * np.float32(0.02),
        g.standard_normal(20000).astype(np.float32) * np.float32(300.0),
        (g.standard_normal(5000) * 1e-6).astype(np.float32),
        np.array([0.0, -0.0, 65504.0, 65519.9, 65520.0, 1e9, -1e9, 5.9604645e-8, 2.9802322e-8,
                  2.98023e-8, 6.1035156e-5, 6.0975552e-5, 1.0009766, 1.00048828125], np.float32),
        # exact ties between neighbouring halves
        (np.arange(1024, 1124, dtype=np.float32) + np.float32(0.5)) / np.float32(1024.0),
    ])
    with np.errstate(over="ignore"):
        want = vals.astype(np.float16).view(np.uint16)
    got = np.array([oracle.float_to_half(float(v)) for v in vals], dtype=np.uint16)
    assert np.array_equal(got, want)
    # the reference's scalar narrowing truncates and therefore differs somewhere
    trunc = np.array([oracle.float_to_half_trunc(float(v)) for v in vals[:2000]], dtype=np.uint16)
    assert np.any(trunc != want[:2000])


def test_scale_min_k4_roundtrip(oracle):
    # PackScaleMinK4 (TensorQuantizer.KQuant.cs:451-459) then GetScaleMinK4_* must return the inputs
    g = synth.rng("pins", "k4")
    for _ in range(200):
        sc = g.integers(0, 64, 8)
        mn = g.integers(0, 64, 8)
        packed = np.zeros(12, np.uint8)
        for j in range(4):
            packed[j] = (sc[j] & 0x3F) | ((sc[4 + j] >> 4) << 6)
            packed[4 + j] = (mn[j] & 0x3F) | ((mn[4 + j] >> 4) << 6)
            packed[8 + j] = (sc[4 + j] & 0x0F) | ((mn[4 + j] & 0x0F) << 4)
        s, m = oracle.scale_min_k4(packed)
        assert list(s) == list(sc) and list(m) == list(mn)


# ---- restatement == the reference's own compiled C, bit for bit ----------------------------
def _random_raw(dtype, n_bytes, name):
    """Random bytes with every fp16 scale pinned to something tame (as the reference's
    agreement tests do, QuantizationAgreementTests.cs / Q8BlockTailTests.cs:46-55)."""
    g = synth.rng("pins", name)
    raw = g.integers(0, 256, n_bytes, dtype=np.uint8)
    bb = {Q8_0: 34, Q4_K: 144, Q6_K: 210}[dtype]
    blocks = raw[: n_bytes // bb * bb].reshape(-1, bb)
    if dtype == Q8_0:
        blocks[:, 0], blocks[:, 1] = 0x00, 0x38
    elif dtype == Q4_K:
        blocks[:, 0], blocks[:, 1] = 0x00, 0x2C
        blocks[:, 2], blocks[:, 3] = 0x00, 0x28
    else:
        blocks[:, 208], blocks[:, 209] = 0x00, 0x24
    return raw


CASES = [
    (Q8_0, 5, 8), (Q8_0, 5, 15), (Q8_0, 5, 32), (Q8_0, 5, 33), (Q8_0, 5, 137), (Q8_0, 7, 896),
    (Q8_0, 4, 1024),
    (Q4_K, 6, 256), (Q4_K, 6, 1024), (Q4_K, 8, 96), (Q4_K, 8, 160), (Q4_K, 4, 320),
    (Q6_K, 6, 256), (Q6_K, 6, 1024), (Q6_K, 8, 96), (Q6_K, 8, 160), (Q6_K, 4, 320),
]


@pytest.mark.parametrize("dtype,n,k", CASES)
def test_restatement_matches_reference_c(oracle, dtype, n, k):
    if oracle.ref_lib() is None:
        pytest.skip("oracle/_ref not built (reference tree absent)")
    raw = _random_raw(dtype, oracle.raw_bytes(dtype, n, k) + 256, f"raw{dtype}_{n}_{k}")
    x = synth.uniform("pins", f"x{dtype}_{n}_{k}", (k,))
    for col in range(n):
        want = np.float32(oracle.vecdot_ref(dtype, x, raw, col, k))
        got = np.float32(oracle.vecdot(dtype, x, raw, col, k))
        assert got.view(np.uint32) == want.view(np.uint32), (dtype, col, k, got, want)


def test_golden_vectors(oracle):
    """Outputs recorded from the reference's compiled C on seeded inputs."""
    gold = np.load(GOLDEN)
    for key in gold.files:
        if not key.startswith("out_"):
            continue
        _, dtype, n, k = key.split("_")
        dtype, n, k = int(dtype), int(n), int(k)
        raw = _random_raw(dtype, oracle.raw_bytes(dtype, n, k) + 256, f"gold{dtype}_{n}_{k}")
        x = synth.uniform("pins", f"goldx{dtype}_{n}_{k}", (k,))
        got = np.array([oracle.vecdot(dtype, x, raw, c, k) for c in range(n)], np.float32)
        assert np.array_equal(got.view(np.uint32), gold[key].view(np.uint32)), key
        # quantised weights made by the oracle quantiser, dotted by the reference's C
        wkey = f"qout_{dtype}_{n}_{k}"
        if wkey in gold.files:
            w = synth.normal("pins", f"goldw{dtype}_{n}_{k}", (n, k), 0.02)
            rawq = oracle.quantize(dtype, w)
            got = np.array([oracle.vecdot(dtype, x, rawq, c, k) for c in range(n)], np.float32)
            assert np.array_equal(got.view(np.uint32), gold[wkey].view(np.uint32)), wkey


# ---- SharpMind.Tests/Quantization/Q8BlockTailTests.cs:25-97 --------------------------------
@pytest.mark.parametrize("k", [8, 15, 20, 32, 33, 40, 63, 64, 96, 137, 896])
def test_q8_tail_vector_tier_agrees_with_scalar(oracle, k):
    n_cols = 3
    raw = _random_raw(Q8_0, oracle.raw_bytes(Q8_0, n_cols, k), f"tail{k}")
    x = np.full(k + 64, 1e6, np.float32)  # loud padding: any over-read blows the tolerance
    x[:k] = synth.uniform("pins", f"tailx{k}", (k,))
    for c in range(n_cols):
        want = oracle.vecdot(Q8_0, x, raw, c, k)
        got = oracle.vecdot_fma(Q8_0, x, raw, c, k)
        assert abs(want - got) <= 1e-4 * max(1.0, abs(want))


# ---- QuantizationAgreementTests.cs:133-250: vector tier vs scalar, abs<1 or rel<1e-3 -------
@pytest.mark.parametrize("dtype", [Q8_0, Q4_K, Q6_K])
def test_fma_port_agrees_with_scalar(oracle, dtype):
    be = 32 if dtype == Q8_0 else 256
    k, n, m = 8 * be, 4 * be // 8, 3
    w = synth.normal("pins", f"agree_w{dtype}", (n, k), 0.02)
    raw = oracle.quantize(dtype, w)
    x = synth.normal("pins", f"agree_x{dtype}", (m, k))
    a = oracle.qmatmul(dtype, x, raw, m, k, n)
    b = oracle.qmatmul_fma(dtype, x, raw, m, k, n)
    scale = np.linalg.norm(w, axis=1)[None, :] * np.linalg.norm(x, axis=1)[:, None]
    assert np.all(np.abs(a - b) <= 1e-5 * scale)


# ---- SharpMind.Tests/Quantization/KQuantEncoderTests.cs:37-103 -----------------------------
@pytest.mark.parametrize("dtype,bound", [(Q4_K, 0.120), (Q6_K, 0.040)])
def test_kquant_roundtrip_fidelity(oracle, dtype, bound):
    n_cols, in_f = 3, 4 * 256
    w = synth.uniform("pins", f"rt{dtype}", (n_cols, in_f))
    raw = oracle.quantize(dtype, w)
    assert raw.size == oracle.raw_bytes(dtype, n_cols, in_f)
    back = oracle.dequantize(dtype, raw, n_cols * in_f).reshape(n_cols, in_f)
    for c in range(n_cols):
        rel = np.sqrt(np.sum((w[c] - back[c]) ** 2, dtype=np.float64) / np.sum(w[c] ** 2, dtype=np.float64))
        assert rel < bound


def test_q8_0_roundtrip_fidelity(oracle):
    w = synth.normal("pins", "rt8", (4, 1024), 0.02)
    back = oracle.dequantize(Q8_0, oracle.quantize(Q8_0, w), w.size).reshape(w.shape)
    assert np.max(np.abs(w - back)) <= np.max(np.abs(w)) / 127.0


@pytest.mark.parametrize("dtype", [Q8_0, Q4_K, Q6_K])
def test_zero_block_encodes_to_zero(oracle, dtype):
    raw = oracle.quantize(dtype, np.zeros(256, np.float32))
    assert not raw.any()
    assert not oracle.dequantize(dtype, raw, 256).any()


def test_quantizers_reject_ragged_lengths(oracle):
    with pytest.raises(ValueError):
        oracle.quantize(Q4_K, np.arange(300, dtype=np.float32))
    with pytest.raises(ValueError):
        oracle.quantize(Q6_K, np.arange(300, dtype=np.float32))
    with pytest.raises(ValueError):
        oracle.quantize(Q8_0, np.arange(40, dtype=np.float32))


def test_raw_byte_counts(oracle):
    # QuantizationOps.GetRawTensorByteCount (QuantizationOps.cs:15-72) at the headline shapes
    assert oracle.raw_bytes(Q8_0, 3072, 1024) == 3_342_336
    assert oracle.raw_bytes(Q4_K, 14336, 4096) == 33_030_144
    assert oracle.raw_bytes(Q6_K, 4096, 14336) == 48_168_960
    assert oracle.raw_bytes(Q4_K, 28672, 8192) == 132_120_576
    assert oracle.raw_bytes(Q8_0, 3, 33) == 3 * 2 * 34


# ---- activation quantiser (QuantizedKVCache.QuantizeRowQ8_0) ------------------------------
def test_activation_quantiser_rules(oracle):
    x = np.zeros((1, 40), np.float32)
    x[0, :4] = [0.5, 1.5, 2.5, 127.0]  # d == 1 -> ties go to even
    q, d = oracle.split_q8_rows(oracle.quantize_rows_q8_0(x, 1, 40))
    assert list(q[0, :4]) == [0, 2, 2, 127]
    assert d[0, 0] == 0x3C00
    assert d[0, 1] == 0x3C00 and not q[0, 32:].any()  # all-zero block stores d = 1, padded zeros
    x = synth.normal("pins", "actq", (3, 96))
    q, d = oracle.split_q8_rows(oracle.quantize_rows_q8_0(x, 3, 96))
    amax = np.abs(x.reshape(3, 3, 32)).max(axis=2)
    assert np.array_equal(d, (amax / np.float32(127.0)).astype(np.float16).view(np.uint16))
    assert np.abs(q).max() == 127


def test_block_isums_match_dequantised_dot(oracle):
    for dtype, k in ((Q8_0, 128), (Q4_K, 512), (Q6_K, 512)):
        w = synth.normal("pins", f"isw{dtype}", (3, k), 0.02)
        raw = oracle.quantize(dtype, w)
        x = synth.normal("pins", f"isx{dtype}", (1, k))
        xq = oracle.quantize_rows_q8_0(x, 1, k)
        qx, _ = oracle.split_q8_rows(xq)
        sums = oracle.block_isums(dtype, raw, xq[0], 1, k)
        assert sums.dtype == np.int32 and sums.size == k // 32
        if dtype == Q8_0:
            qw = raw.reshape(3, k // 32, 34)[1, :, 2:].view(np.int8).astype(np.int64)
            want = (qw * qx[0].reshape(-1, 32).astype(np.int64)).sum(axis=1)
            assert np.array_equal(sums, want)


# ---- RoPE: SharpMind.Tests/Core/RoPETests.cs:44-79, RoPEConventionTests.cs:34-135 ----------
def test_rope_adjacent_headdim4(oracle):
    cos, sin = oracle.rope_tables(10000.0, 4, 8)
    x = oracle.rope_apply(np.array([[[1, 2, 3, 4]]], np.float32), 1, cos, sin, neox=False)[0, 0]
    th1, th2 = 1.0, float(np.float32(10000.0) ** np.float32(-0.5))
    want = [np.cos(th1) - 2 * np.sin(th1), 2 * np.cos(th1) + np.sin(th1),
            3 * np.cos(th2) - 4 * np.sin(th2), 4 * np.cos(th2) + 3 * np.sin(th2)]
    assert np.allclose(x, want, atol=5e-6)


def test_rope_adjacent_headdim8(oracle):
    cos, sin = oracle.rope_tables(10000.0, 8, 8)
    x = oracle.rope_apply(np.arange(1, 9, dtype=np.float32).reshape(1, 1, 8), 1, cos, sin, neox=False)[0, 0]
    for i in range(4):
        th = float(np.float32(10000.0) ** np.float32(-2.0 * i / 8.0))
        assert abs(x[2 * i] - ((2 * i + 1) * np.cos(th) - (2 * i + 2) * np.sin(th))) < 5e-5
        assert abs(x[2 * i + 1] - ((2 * i + 2) * np.cos(th) + (2 * i + 1) * np.sin(th))) < 5e-5


def test_rope_neox_pairs_d_with_d_plus_half(oracle):
    cos, sin = oracle.rope_tables(10000.0, 4, 8)
    x = oracle.rope_apply(np.array([[[1, 2, 3, 4]]], np.float32), 1, cos, sin, neox=True)[0, 0]
    f1 = 1.0 / float(np.float32(10000.0) ** np.float32(0.5))
    c0, s0, c1, s1 = np.cos(1.0), np.sin(1.0), np.cos(f1), np.sin(f1)
    assert np.allclose(x, [c0 - 3 * s0, 2 * c1 - 4 * s1, 3 * c0 + s0, 4 * c1 + 2 * s1], atol=5e-5)
    adj = oracle.rope_apply(np.array([[[1, 2, 3, 4]]], np.float32), 1, cos, sin, neox=False)[0, 0]
    assert abs(adj[0] - x[0]) > 1e-3


def test_rope_position0_is_identity_and_theta_matters(oracle):
    for neox in (False, True):
        cos, sin = oracle.rope_tables(10000.0, 4, 8)
        x = oracle.rope_apply(np.array([[[1, 2, 3, 4]]], np.float32), 0, cos, sin, neox=neox)[0, 0]
        assert np.array_equal(x, [1, 2, 3, 4])
    a = oracle.rope_apply(np.array([[[1, 2, 3, 4]]], np.float32), 1, *oracle.rope_tables(1e4, 4, 8), neox=False)
    b = oracle.rope_apply(np.array([[[1, 2, 3, 4]]], np.float32), 1, *oracle.rope_tables(5e5, 4, 8), neox=False)
    assert abs(a[0, 0, 2] - b[0, 0, 2]) > 1e-4 and a[0, 0, 0] == b[0, 0, 0]


# ---- activations: SharpMind.Tests/Core/ActivationTests.cs:23-82,150-231 --------------------
def test_softmax_properties(oracle):
    r = oracle.softmax_rows(np.array([1, 2, 3, 4], np.float32))
    assert abs(r.sum() - 1) < 1e-5 and np.all(np.diff(r) > 0)
    r = oracle.softmax_rows(np.array([1000, 1001, 1002], np.float32))
    assert abs(r.sum() - 1) < 1e-4 and not np.isnan(r).any()
    r = oracle.softmax_rows(np.array([[1, 2, 3], [4, 5, 6]], np.float32))
    assert np.allclose(r.sum(axis=1), 1, atol=1e-5)


def test_rmsnorm_properties(oracle):
    r = oracle.rmsnorm(np.array([3, 4], np.float32), np.ones(2, np.float32), 0.0)
    assert abs(np.sqrt(np.mean(r * r)) - 1) < 1e-4
    r = oracle.rmsnorm(np.ones(4, np.float32), np.full(4, 2, np.float32), 0.0)
    assert np.allclose(r, 2, atol=1e-4)


def test_silu_swiglu_properties_and_vector_parity(oracle):
    assert oracle.silu(np.zeros(4, np.float32)).tolist() == [0, 0, 0, 0]
    assert abs(oracle.silu(np.array([10.0], np.float32))[0] - 10.0) < 1e-3
    g = synth.normal("pins", "swg", (1000,))
    u = synth.normal("pins", "swu", (1000,))
    want = oracle.swiglu(g, u)
    assert np.allclose(want, g / (1 + np.exp(-g.astype(np.float64))) * u, rtol=1e-5, atol=1e-6)
    got = np.empty_like(want)
    oracle.fma_lib().smf_swiglu(g.ctypes.data, u.ctypes.data, got.ctypes.data, 1000)
    assert np.allclose(got, want, atol=1e-5)  # the reference accepts 5 decimals between tiers
    sm_s = oracle.softmax_rows(g)
    sm_v = np.empty_like(sm_s)
    oracle.fma_lib().smf_softmax_row(g.ctypes.data, sm_v.ctypes.data, 1000)
    assert np.allclose(sm_s, sm_v, atol=1e-6)


def test_argmax_first_maximum_wins(oracle):
    assert oracle.argmax(np.array([1, 5, 5, 2], np.float32)) == 1


def test_sdpa_flash_matches_plain_softmax_attention(oracle):
    hd, kv = 16, 150  # crosses two 64-key tiles and a ragged third
    q = synth.normal("pins", "sq", (1, hd))
    k = synth.normal("pins", "sk", (kv, hd))
    v = synth.normal("pins", "sv", (kv, hd))
    got = oracle.sdpa_flash(q, k, v, 0.25)
    s = (k.astype(np.float64) @ q[0].astype(np.float64)) * 0.25
    p = np.exp(s - s.max())
    want = (p / p.sum()) @ v.astype(np.float64)
    assert np.allclose(got[0], want, rtol=1e-5, atol=1e-6)


def test_medusa_head_transform_and_acceptance_rule(oracle):
    """The oracle's Medusa restatement against a literal Python loop of MedusaHeads.PredictQuantized's head transform
    (small case), and the acceptance rule on hand-written cases."""
    rng = np.random.default_rng(7)
    k, H = 2, 12
    hidden = rng.standard_normal(H).astype(np.float32)
    w = rng.standard_normal((k, H, H)).astype(np.float32)
    b = rng.standard_normal((k, H)).astype(np.float32)
    got = oracle.medusa_heads(hidden, w, b)
    for h in range(k):
        for i in range(H):
            s = np.float32(b[h, i])
            for j in range(H):
                s = np.float32(s + np.float32(hidden[j] * w[h, j, i]))
            want = np.float32(s / np.float32(np.float32(1.0) + np.exp(np.float32(-s), dtype=np.float32)))
            assert abs(got[h, i] - want) <= 2e-7 * max(1.0, abs(want))
    assert oracle.verify_greedy([5, 6, 7, 8], [1, 5, 6, 7]) == 4          # every guess right (the 4th pick is the bonus)
    assert oracle.verify_greedy([5, 9, 7, 8], [1, 5, 6, 7]) == 2          # second guess wrong: later matches do not count
    assert oracle.verify_greedy([4, 6, 7, 8], [1, 5, 6, 7]) == 1          # token 0 alone
    assert oracle.verify_greedy([4], [1]) == 1                            # no heads
