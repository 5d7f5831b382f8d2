"""Draft verification on the device: Transformer.Forward over a draft's tokens with logits for every position, the
acceptance rule of MedusaGenerator (MedusaGenerator.cs:259-283), the heads' own prediction (MedusaHeads.cs:64-130), and
the cache roll-back after a rejected suffix (IKVCache.Truncate, MedusaGenerator.cs:394-398): the caller's next `pos`.

The oracle has no batched pass: it reaches the same numbers one token at a time, which is what makes the check a
check of the causal masking and cache writes of the batched pass too.
"""
import numpy as np
import pytest

from sharpmind_b200 import ops, synth
from sharpmind_b200.decoder import Decoder
from tests.gpu_util import to_dev

pytestmark = pytest.mark.gpu

CFG = dict(n_layers=3, hidden=256, n_heads=4, n_kv_heads=2, head_dim=128, ffn=512, vocab=2048,
           max_seq=64, dtype=8, eps=1e-6, rope_theta=1.0e6, neox=True, qk_norm=True)
NAME = "spec_small"


def _prefix(oracle, ref, toks):
    out = None
    for p, t in enumerate(toks):
        out = ref.step(np.array([t], dtype=np.int32), p)
    return out


@pytest.mark.parametrize("mode", [ops.Mode.ACT_F32, ops.Mode.REF_ORDER])
@pytest.mark.parametrize("n_right", [0, 2, 4])
def test_draft_verification_round(oracle, cuda, mode, n_right):
    """A prompt, then a draft of K + 1 = 5 tokens of which the first n_right head guesses are what the model would
    pick and the next is not.  Logits of all five positions match the oracle's token-by-token pass, the accepted count
    is 1 + n_right, and decoding on from pos + accepted (the rejected rows still in the cache) matches an oracle that
    never saw the rejected tokens."""
    n_prompt, K = 9, 4
    w = synth.make_decoder_weights(CFG, NAME, oracle.quantize)
    prompt = synth.token_ids(NAME, "spec_prompt", (n_prompt,), CFG["vocab"])
    ref = oracle.Decoder(CFG, w, 1)
    last = _prefix(oracle, ref, prompt)
    # the model's own greedy continuation: what a perfect draft would hold
    true_next, pos, lg = [], n_prompt, last
    probe = oracle.Decoder(CFG, w, 1)
    _prefix(oracle, probe, prompt)
    for i in range(K + 1):
        t = int(lg[0].argmax())
        true_next.append(t)
        lg = probe.step(np.array([t], dtype=np.int32), pos + i)
    draft = np.array(true_next, dtype=np.int32)
    for i in range(1 + n_right, K + 1):
        draft[i] = (draft[i] + 17 + i) % CFG["vocab"]  # a wrong guess, and everything after it
    # oracle: the same five tokens one by one
    want = np.stack([ref.step(draft[i:i + 1], n_prompt + i)[0] for i in range(K + 1)])
    dec = Decoder(cuda, CFG, w, max_batch=1, keep_raw=(mode == ops.Mode.REF_ORDER))
    dec.forward_last_logits(to_dev(prompt), 0, 0, mode)
    logits, picks, hidden = dec.forward_logits(to_dev(draft), n_prompt, 0, mode, want_hidden=True)
    got = logits.cpu().numpy()
    scale = np.abs(want).max()
    assert np.max(np.abs(got - want)) <= 1e-4 * scale, float(np.max(np.abs(got - want)) / scale)
    picks = picks.cpu().numpy()
    assert np.array_equal(picks, got.argmax(axis=1).astype(np.int32))
    accepted = dec.verify_greedy(to_dev(picks), to_dev(draft))
    assert accepted == oracle.verify_greedy(want.argmax(axis=1), draft) == 1 + n_right
    # roll back: the next round starts at n_prompt + accepted with the token the model picked after the last accepted one
    clean = oracle.Decoder(CFG, w, 1)
    _prefix(oracle, clean, np.concatenate([prompt, draft[:accepted]]))
    tok = np.array([int(want[accepted - 1].argmax())], dtype=np.int32)
    for step in range(3):
        p = n_prompt + accepted + step
        w_l = clean.step(tok, p)
        g_l, g_t = dec.step(to_dev(tok), p, mode)
        assert np.max(np.abs(g_l.cpu().numpy() - w_l)) <= 1e-4 * np.abs(w_l).max()
        tok = np.array([int(w_l[0].argmax())], dtype=np.int32)
    # the hidden rows are the final-normed states the LM head saw: the LM head applied to them gives the logits back
    again = ops.DeviceOps(cuda).qmatmul(hidden, dec.embedding, mode)
    assert np.array_equal(again.cpu().numpy(), got)
    dec.close()
    assert cuda.device_status() == 0


@pytest.mark.parametrize("k", [1, 4])
def test_medusa_heads_predict(oracle, cuda, k):
    """h' = SiLU(hidden W + b) summed in the reference's order, then the shared Q8_0 LM head and a first-maximum argmax."""
    H, V = CFG["hidden"], CFG["vocab"]
    w = synth.make_decoder_weights(CFG, NAME, oracle.quantize)
    rng = synth.rng(NAME, f"medusa{k}")
    hidden = rng.standard_normal(H).astype(np.float32)
    head_w = (rng.standard_normal((k, H, H)) / np.sqrt(H)).astype(np.float32)
    head_b = (0.1 * rng.standard_normal((k, H))).astype(np.float32)
    want_tok, want_logits = oracle.medusa_predict(hidden, head_w, head_b, w["embedding"], V)
    dec = Decoder(cuda, CFG, w, max_batch=1, keep_raw=True)
    got = dec.medusa_predict(to_dev(hidden), to_dev(head_w), to_dev(head_b)).cpu().numpy()
    # the exponential differs in the last place between libm and the device, so a near-tie may flip: a pick must be
    # the oracle's, or one whose oracle logit is within 1e-5 of the oracle's best
    for i in range(k):
        if got[i] != want_tok[i]:
            assert want_logits[i, want_tok[i]] - want_logits[i, got[i]] <= 1e-5 * np.abs(want_logits[i]).max()
    assert (got == want_tok).sum() >= k - 1
    dec.close()
    assert cuda.device_status() == 0


def test_verification_rejects_bad_arguments(oracle, cuda):
    w = synth.make_decoder_weights(CFG, NAME, oracle.quantize)
    dec = Decoder(cuda, CFG, w, max_batch=1)
    toks = to_dev(np.arange(8, dtype=np.int32))
    with pytest.raises(ops.SharpMindCudaError):
        dec.forward_logits(toks, CFG["max_seq"] - 3, 0)   # runs past the cache
    with pytest.raises(ops.SharpMindCudaError):
        dec.forward_logits(toks, 0, 1)                    # no such sequence slot
    dec.close()
