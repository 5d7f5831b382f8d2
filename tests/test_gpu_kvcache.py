"""Device KV cache objects (IKVCache surface) against the oracle: Update / Truncate / TrimToLast / Snapshot / Restore and
attention over an fp32 cache (KVCache + ScaledDotProductFlash*) and a Q8_0 cache (QuantizedKVCache +
ScaledDotProductFlashQ8_0*).

Q8_0 rows must be bit-exact with QuantizedKVCache.QuantizeRowQ8_0 (the snapshot speaks the reference's 34-byte block
layout, so it is compared byte for byte with the oracle's row quantiser); attention outputs within 1e-5 relative of the
oracle's restatement of the scalar flash kernels on the same (quantised) rows.
"""
import numpy as np
import pytest

from sharpmind_b200 import ops, synth
from tests.gpu_util import to_dev

pytestmark = pytest.mark.gpu


def _rows_q8(oracle, x):
    """x [..., headDim] fp32 -> [..., headDim/32*34] uint8, QuantizeRowQ8_0 per row."""
    hd = x.shape[-1]
    flat = x.reshape(-1, hd)
    q = oracle.quantize_rows_q8_0(flat, flat.shape[0], hd)
    return np.asarray(q, np.uint8).reshape(*x.shape[:-1], hd // 32 * 34)


def _oracle_attention(oracle, kind, q, kc, vc, length, scale):
    """q [B, S, H, D]; kc / vc [B, KVH, length, row] (fp32 rows or Q8_0 byte rows); returns [B, S, H, D]."""
    B, S, H, D = q.shape
    KVH = kc.shape[1]
    out = np.zeros_like(q)
    for b in range(B):
        for h in range(H):
            kh = h // (H // KVH)
            qq = np.ascontiguousarray(q[b, :, h, :])
            if kind == ops.KVCache.Q8_0:
                out[b, :, h, :] = oracle.sdpa_flash_q8(qq, kc[b, kh, :length], vc[b, kh, :length], scale)
            else:
                out[b, :, h, :] = oracle.sdpa_flash(qq, kc[b, kh, :length], vc[b, kh, :length], scale)
    return out


@pytest.mark.parametrize("kind", [ops.KVCache.F32, ops.KVCache.Q8_0])
@pytest.mark.parametrize("hd,heads,kvh", [(128, 8, 2), (64, 4, 4)])
def test_kv_cache_update_attention_truncate_snapshot(oracle, cuda, kind, hd, heads, kvh):
    B, max_seq = 2, 96
    kv = ops.KVCache(cuda, B, kvh, max_seq, hd, kind)
    assert kv.Length == 0 and kv.MaxSeqLen == max_seq and not kv.IsFull and kv.Snapshot() is None
    scale = 1.0 / np.sqrt(hd)
    # the oracle's cache: rows as the reference stores them
    row = hd // 32 * 34 if kind == ops.KVCache.Q8_0 else hd
    kc = np.zeros((B, kvh, max_seq, row), np.uint8 if kind == ops.KVCache.Q8_0 else np.float32)
    vc = np.zeros_like(kc)
    length = 0

    def append(tag, s):
        nonlocal length
        k = synth.normal("kv", f"k{tag}{hd}", (B, s, kvh, hd))
        v = synth.normal("kv", f"v{tag}{hd}", (B, s, kvh, hd))
        if tag == "z":
            k[:, 0, 0, :32] = 0.0  # an all-zero block takes d = 1
        kv.Update(to_dev(k), to_dev(v))
        kr, vr = (_rows_q8(oracle, k), _rows_q8(oracle, v)) if kind == ops.KVCache.Q8_0 else (k, v)
        kc[:, :, length:length + s] = kr.transpose(0, 2, 1, 3)
        vc[:, :, length:length + s] = vr.transpose(0, 2, 1, 3)
        length += s

    def check_attention(tag, s):
        q = synth.normal("kv", f"q{tag}{hd}", (B, s, heads, hd))
        got = kv.attention(to_dev(q), scale).cpu().numpy()
        want = _oracle_attention(oracle, kind, q, kc, vc, length, scale)
        assert np.max(np.abs(got - want)) <= 1e-5 * np.max(np.abs(want)), (tag, float(np.max(np.abs(got - want)) / np.max(np.abs(want))))

    append("a", 37)                 # a prompt chunk
    assert kv.Length == 37
    check_attention("a", 5)         # the last five positions as queries (several rows: prompt / verification shape)
    append("z", 1)
    check_attention("b", 1)         # one decode step
    # the stored rows are the reference's rows, byte for byte
    pos, sk, sv = kv.Snapshot()
    assert pos == length
    assert np.array_equal(sk.view(kc.dtype).reshape(B, kvh, length, row), kc[:, :, :length])
    assert np.array_equal(sv.view(vc.dtype).reshape(B, kvh, length, row), vc[:, :, :length])
    # speculative rollback: append draft positions, truncate them away, carry on
    snap = (pos, sk.copy(), sv.copy())
    saved_k, saved_v, saved_len = kc.copy(), vc.copy(), length
    append("d", 4)
    check_attention("d", 4)
    kv.Truncate(saved_len)
    kv.Truncate(saved_len + 100)    # never grows (Math.Min)
    assert kv.Length == saved_len
    kc, vc, length = saved_k, saved_v, saved_len
    append("e", 1)
    check_attention("e", 1)
    # Restore brings the snapshot back, on this object or a fresh one
    other = ops.KVCache(cuda, B, kvh, max_seq, hd, kind)
    other.Restore(snap)
    assert other.Length == saved_len
    kc2, vc2 = saved_k.copy(), saved_v.copy()
    q = synth.normal("kv", f"qr{hd}", (B, 1, heads, hd))
    got = other.attention(to_dev(q), scale).cpu().numpy()
    want = _oracle_attention(oracle, kind, q, kc2, vc2, saved_len, scale)
    assert np.max(np.abs(got - want)) <= 1e-5 * np.max(np.abs(want))
    other.Dispose()
    # sliding window: the last 20 positions move to the front
    kv.TrimToLast(20)
    assert kv.Length == 20
    kc[:, :, :20] = kc[:, :, length - 20:length].copy()
    vc[:, :, :20] = vc[:, :, length - 20:length].copy()
    length = 20
    check_attention("t", 1)
    kv.TrimToLast(50)               # keep >= length: nothing happens
    assert kv.Length == 20
    kv.Reset()
    assert kv.Length == 0
    # overflow is refused (KVCache.Update throws)
    with pytest.raises(ops.ArgumentOutOfRangeException):
        kv.Update(to_dev(np.zeros((B, max_seq + 1, kvh, hd), np.float32)), to_dev(np.zeros((B, max_seq + 1, kvh, hd), np.float32)))
    kv.Dispose()
    assert cuda.device_status() == 0


def test_q8_cache_long_context_decode(oracle, cuda):
    """The benchmark's context length: 2049 positions of a Q8_0 cache, 16 query heads over 8 cached heads."""
    B, kvh, heads, hd, n = 1, 8, 16, 128, 2049
    kv = ops.KVCache(cuda, B, kvh, n + 7, hd, ops.KVCache.Q8_0)
    k = synth.normal("kv", "klong", (B, n, kvh, hd))
    v = synth.normal("kv", "vlong", (B, n, kvh, hd))
    kv.Update(to_dev(k), to_dev(v))
    q = synth.normal("kv", "qlong", (B, 1, heads, hd))
    scale = 1.0 / np.sqrt(hd)
    got = kv.attention(to_dev(q), scale).cpu().numpy()
    kc, vc = _rows_q8(oracle, k).transpose(0, 2, 1, 3), _rows_q8(oracle, v).transpose(0, 2, 1, 3)
    want = _oracle_attention(oracle, ops.KVCache.Q8_0, q, np.ascontiguousarray(kc), np.ascontiguousarray(vc), n, scale)
    assert np.max(np.abs(got - want)) <= 1e-5 * np.max(np.abs(want))
    kv.Dispose()


@pytest.mark.parametrize("hd,heads,kvh", [(128, 8, 4), (128, 6, 2), (64, 4, 4), (64, 8, 1)])
def test_prompt_attention_on_tensor_cores(oracle, cuda, hd, heads, kvh):
    """Causal attention of a chunk of query rows over an fp32 cache with both contractions as bf16 MMAs on operands split
    three ways: within 1e-5 of the oracle's scalar flash attention (the bound of the fp32 kernel), for chunks that end
    inside a 64-row tile, start after an earlier chunk, and for query-head groups of 1, 2, 3 and 8; and the fp32
    CUDA-core kernel it replaces gives the same result to that bound."""
    B, max_seq = 2, 320
    kv = ops.KVCache(cuda, B, kvh, max_seq, hd, ops.KVCache.F32)
    scale = 1.0 / np.sqrt(hd)
    kc = np.zeros((B, kvh, max_seq, hd), np.float32)
    vc = np.zeros_like(kc)
    length = 0
    for tag, s in (("p", 150), ("q", 77), ("r", 1), ("s", 64)):
        k = synth.normal("kvmma", f"k{tag}{hd}", (B, s, kvh, hd))
        v = synth.normal("kvmma", f"v{tag}{hd}", (B, s, kvh, hd))
        if tag == "p":
            k *= 4.0  # sharper softmax: scores of a few units
        kv.Update(to_dev(k), to_dev(v))
        kc[:, :, length:length + s] = k.transpose(0, 2, 1, 3)
        vc[:, :, length:length + s] = v.transpose(0, 2, 1, 3)
        length += s
        q = synth.normal("kvmma", f"q{tag}{hd}", (B, s, heads, hd))
        got = kv.attention(to_dev(q), scale).cpu().numpy()
        want = _oracle_attention(oracle, ops.KVCache.F32, q, kc, vc, length, scale)
        err = float(np.max(np.abs(got - want)) / np.max(np.abs(want)))
        assert err <= 1e-5, (tag, err)
        if s > 1:
            cuda.set_option("prompt_attention_mma", 0)
            try:
                old = kv.attention(to_dev(q), scale).cpu().numpy()
            finally:
                cuda.set_option("prompt_attention_mma", 1)
            assert np.max(np.abs(old - got)) <= 2e-5 * np.max(np.abs(want))
            # one query head per CTA instead of two that share a KV head: every head's arithmetic is the same
            cuda.set_option("prompt_attention_heads_per_cta", 1)
            try:
                single = kv.attention(to_dev(q), scale).cpu().numpy()
            finally:
                cuda.set_option("prompt_attention_heads_per_cta", 0)
            assert np.array_equal(single.view(np.uint32), got.view(np.uint32))
    kv.Dispose()
    assert cuda.device_status() == 0


@pytest.mark.parametrize("hd,heads,kvh", [(128, 8, 4), (64, 6, 2)])
def test_prompt_attention_on_tensor_cores_over_a_q8_0_cache(oracle, cuda, hd, heads, kvh):
    """Chunks of 16 query rows and more over a Q8_0 cache take the tensor-core kernel with its K / V tiles staged as d * q
    (exact in the three bf16 parts): within 1e-5 of the oracle's ScaledDotProductFlashQ8_0 on the same quantised rows,
    and of the CUDA-core kernel it replaces; shorter chunks keep that kernel."""
    B, max_seq = 2, 320
    kv = ops.KVCache(cuda, B, kvh, max_seq, hd, ops.KVCache.Q8_0)
    scale = 1.0 / np.sqrt(hd)
    row = hd // 32 * 34
    kc = np.zeros((B, kvh, max_seq, row), np.uint8)
    vc = np.zeros_like(kc)
    length = 0
    for tag, s in (("p", 150), ("q", 77), ("r", 5), ("s", 64)):
        k = synth.normal("kvmmaq8", f"k{tag}{hd}", (B, s, kvh, hd))
        v = synth.normal("kvmmaq8", f"v{tag}{hd}", (B, s, kvh, hd))
        if tag == "p":
            k *= 4.0
        kv.Update(to_dev(k), to_dev(v))
        kc[:, :, length:length + s] = _rows_q8(oracle, k).transpose(0, 2, 1, 3)
        vc[:, :, length:length + s] = _rows_q8(oracle, v).transpose(0, 2, 1, 3)
        length += s
        q = synth.normal("kvmmaq8", f"q{tag}{hd}", (B, s, heads, hd))
        got = kv.attention(to_dev(q), scale).cpu().numpy()
        want = _oracle_attention(oracle, ops.KVCache.Q8_0, q, kc, vc, length, scale)
        err = float(np.max(np.abs(got - want)) / np.max(np.abs(want)))
        assert err <= 1e-5, (tag, err)
        cuda.set_option("prompt_attention_mma", 0)
        try:
            old = kv.attention(to_dev(q), scale).cpu().numpy()
        finally:
            cuda.set_option("prompt_attention_mma", 1)
        assert np.max(np.abs(old - got)) <= 2e-5 * np.max(np.abs(want))
        assert np.array_equal(old.view(np.uint32), got.view(np.uint32)) == (s < 16)  # which kernel ran
    kv.Dispose()
    assert cuda.device_status() == 0
