"""Decode attention over the fp32 KV cache and the `attention` slot, against the oracle's
restatement of ScaledDotProductFlashScalar (1e-5 relative to the output scale)."""
import numpy as np
import pytest

from sharpmind_b200 import synth
from tests.gpu_util import bits, to_dev

pytestmark = pytest.mark.gpu


def oracle_decode(oracle, q, kc, vc, kv_len, scale):
    batch, heads, hd = q.shape
    kvh = kc.shape[1]
    out = np.zeros_like(q)
    for b in range(batch):
        for h in range(heads):
            g = h // (heads // kvh)
            out[b, h] = oracle.sdpa_flash(q[b, h:h + 1], kc[b, g, :kv_len], vc[b, g, :kv_len], scale)[0]
    return out


@pytest.mark.parametrize("batch,heads,kvh,hd,kv_len,max_seq", [
    (1, 16, 8, 128, 2049, 2304),   # the full-decode configuration's shape
    (3, 16, 8, 128, 131, 256),
    (2, 8, 8, 64, 77, 128),
    (2, 8, 2, 128, 1, 64),         # a single key
    (1, 4, 2, 32, 100, 128),       # head size the split kernel does not take: reference-order kernel
    (1, 14, 2, 64, 300, 512),      # 7 query heads per KV head: one head per CTA, seven CTAs share a cached head
    (2, 32, 8, 128, 500, 512),     # 4 query heads per KV head, few sequences: run as 2 x 2
    (6, 32, 8, 128, 200, 256),     # 4 per KV head, more sequences
    (1, 64, 8, 128, 300, 512),     # 8 per KV head (70B-class): 4 x 2
    (5, 64, 8, 64, 90, 128),       # 8 per KV head, more sequences, head size 64
])
def test_sdpa_decode(oracle, dev, batch, heads, kvh, hd, kv_len, max_seq):
    q = synth.normal("gpua", f"q{batch}_{heads}_{hd}_{kv_len}", (batch, heads, hd))
    kc = synth.normal("gpua", f"k{batch}_{kvh}_{hd}_{max_seq}", (batch, kvh, max_seq, hd))
    vc = synth.normal("gpua", f"v{batch}_{kvh}_{hd}_{max_seq}", (batch, kvh, max_seq, hd))
    scale = 1.0 / np.sqrt(np.float32(hd))
    want = oracle_decode(oracle, q, kc, vc, kv_len, float(scale))
    got = dev.sdpa_decode(to_dev(q), to_dev(kc), to_dev(vc), kv_len, float(scale)).cpu().numpy()
    tol = 1e-5 * np.abs(want).max(axis=-1, keepdims=True)
    assert np.all(np.abs(got - want) <= tol + 1e-7), np.max(np.abs(got - want) / (tol + 1e-7))


def test_sdpa_decode_is_deterministic(dev):
    q = to_dev(synth.normal("gpua", "dq", (2, 16, 128)))
    kc = to_dev(synth.normal("gpua", "dk", (2, 8, 512, 128)))
    vc = to_dev(synth.normal("gpua", "dv", (2, 8, 512, 128)))
    first = dev.sdpa_decode(q, kc, vc, 400, 0.088).cpu().numpy()
    for _ in range(4):
        assert np.array_equal(bits(dev.sdpa_decode(q, kc, vc, 400, 0.088).cpu().numpy()), bits(first))


def test_kv_append_and_overflow(dev):
    import torch

    from sharpmind_b200 import ops

    kc = torch.zeros((2, 8, 16, 128), device="cuda")
    vc = torch.zeros_like(kc)
    k = to_dev(synth.normal("gpua", "ak", (2, 8, 128)))
    v = to_dev(synth.normal("gpua", "av", (2, 8, 128)))
    dev.kv_append(k, v, kc, vc, 5)
    assert torch.equal(kc[:, :, 5], k) and torch.equal(vc[:, :, 5], v)
    assert kc[:, :, :5].abs().sum() == 0 and kc[:, :, 6:].abs().sum() == 0
    with pytest.raises(ops.ArgumentOutOfRangeException):  # KVCache overflow (KVCache.cs:89-91)
        dev.kv_append(k, v, kc, vc, 16)


@pytest.mark.parametrize("seq,kv,hd,causal", [(1, 150, 16, True), (5, 70, 64, True), (4, 9, 128, False), (3, 3, 256, True)])
def test_attention_slot_reference_order(oracle, cuda, seq, kv, hd, causal):
    """ScaledDotProduct(q, k, v, o, ...) on host pointers with strided q / o rows."""
    from sharpmind_b200.ops import ActivationOps

    a = ActivationOps(cuda)
    heads = 3
    q = synth.normal("gpua", f"sq{seq}_{hd}", (seq, heads, hd))
    k = synth.normal("gpua", f"sk{kv}_{hd}", (kv, hd))
    v = synth.normal("gpua", f"sv{kv}_{hd}", (kv, hd))
    o = np.full((seq, heads, hd), 7.0, np.float32)
    h = 1
    a.ScaledDotProduct(q.reshape(-1)[h * hd:], k, v, o.reshape(-1)[h * hd:], seq, kv, hd, 0.3, causal,
                       heads * hd, heads * hd, 0.0)
    want = oracle.sdpa_flash(np.ascontiguousarray(q[:, h]), k, v, 0.3, causal)
    tol = 2e-6 * np.abs(want).max()
    assert np.all(np.abs(o[:, h] - want) <= tol)
    assert np.all(o[:, 0] == 7.0) and np.all(o[:, 2] == 7.0)  # other heads' rows untouched


def test_attention_slot_rejects_large_heads(cuda):
    from sharpmind_b200 import ops

    a = ops.ActivationOps(cuda)
    z = np.zeros((1, 260), np.float32)
    with pytest.raises(ops.ArgumentOutOfRangeException):
        a.ScaledDotProduct(z, z, z, z.copy(), 1, 1, 260, 1.0, True, 260, 260, 0.0)
