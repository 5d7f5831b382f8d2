"""Device-resident decode step against the oracle's restatement of the decoder forward
(Transformer.ForwardLastLogits with one new token per sequence, greedy sampling).

The model is a reduced Qwen3-shaped decoder (QK-norm, NEOX RoPE, GQA, SwiGLU, tied Q8_0 LM head) with
seeded random weights; the bar is top-1 token agreement over a run of greedy steps and logits within
1e-4 of the logit scale (the sum of ~10 ops per layer each held to 1e-5).
"""
import numpy as np
import pytest

from sharpmind_b200 import ops, synth
from sharpmind_b200.decoder import Decoder
from tests.gpu_util import to_dev

pytestmark = pytest.mark.gpu

SMALL = dict(n_layers=3, hidden=256, n_heads=4, n_kv_heads=2, head_dim=128, ffn=512, vocab=2048,
             max_seq=64, dtype=8, eps=1e-6, rope_theta=1.0e6, neox=True, qk_norm=True)
LLAMA_LIKE = dict(n_layers=2, hidden=256, n_heads=8, n_kv_heads=8, head_dim=64, ffn=768, vocab=1024,
                  max_seq=48, dtype=8, eps=1e-5, rope_theta=1.0e4, neox=False, qk_norm=False)


def _weights(oracle, cfg, name):
    return synth.make_decoder_weights(cfg, name, oracle.quantize)


def _greedy(oracle, cuda, cfg, name, batch, steps, mode):
    import torch

    w = _weights(oracle, cfg, name)
    ref = oracle.Decoder(cfg, w, batch)
    dec = Decoder(cuda, cfg, w, max_batch=batch, keep_raw=(mode == ops.Mode.REF_ORDER))
    tok_ref = synth.token_ids(name, "prompt", (batch,), cfg["vocab"])
    tok_dev = torch.from_numpy(tok_ref.copy()).cuda()
    worst, match = 0.0, 0
    for pos in range(steps):
        want = ref.step(tok_ref, pos)
        logits, nxt = dec.step(tok_dev, pos, mode)
        got = logits.cpu().numpy()
        scale = np.abs(want).max(axis=1, keepdims=True)
        worst = max(worst, float(np.max(np.abs(got - want) / scale)))
        pick = want.argmax(axis=1).astype(np.int32)
        assert np.array_equal(nxt.cpu().numpy(), got.argmax(axis=1).astype(np.int32))  # device argmax = first max
        match += int(np.array_equal(nxt.cpu().numpy(), pick))
        # teacher forcing on the oracle's token keeps both sides on one trajectory
        tok_ref = pick
        tok_dev = torch.from_numpy(pick.copy()).cuda()
    dec.close()
    return worst, match


@pytest.mark.parametrize("cfg,name", [(SMALL, "dec_small"), (LLAMA_LIKE, "dec_llama")])
@pytest.mark.parametrize("mode", [ops.Mode.ACT_F32, ops.Mode.REF_ORDER])
@pytest.mark.parametrize("batch", [1, 3])
def test_decode_matches_oracle_tokens(oracle, cuda, cfg, name, mode, batch):
    steps = 20
    worst, match = _greedy(oracle, cuda, cfg, name, batch, steps, mode)
    assert match == steps, f"top-1 matched on {match}/{steps} steps"
    assert worst <= 1e-4, worst


@pytest.mark.parametrize("batch", [1, 4])
def test_decode_quantised_activations_track_oracle(oracle, cuda, batch):
    """ACT_Q8 re-quantises every activation row to Q8_0, so logits move by ~1e-2 of their scale; the
    greedy token still has to agree wherever the oracle's top-2 margin exceeds that noise."""
    import torch

    cfg, name, steps = SMALL, "dec_small", 16
    w = _weights(oracle, cfg, name)
    ref = oracle.Decoder(cfg, w, batch)
    dec = Decoder(cuda, cfg, w, max_batch=batch)
    tok = synth.token_ids(name, "prompt", (batch,), cfg["vocab"])
    for pos in range(steps):
        want = ref.step(tok, pos)
        logits, nxt = dec.step(torch.from_numpy(tok.copy()).cuda(), pos, ops.Mode.ACT_Q8)
        got = logits.cpu().numpy()
        scale = np.abs(want).max(axis=1)
        assert np.all(np.abs(got - want).max(axis=1) <= 0.05 * scale)
        top2 = np.sort(want, axis=1)[:, -2:]
        clear = (top2[:, 1] - top2[:, 0]) > 0.1 * scale
        pick = want.argmax(axis=1).astype(np.int32)
        assert np.array_equal(nxt.cpu().numpy()[clear], pick[clear])
        tok = pick
    dec.close()


def test_decode_batch_rows_are_independent(oracle, cuda):
    """Lock-step sequences do not interact: row b of a batch of 4 equals the same sequence decoded alone."""
    import torch

    cfg, name = SMALL, "dec_small"
    w = _weights(oracle, cfg, name)
    toks = synth.token_ids(name, "rows", (6, 4), cfg["vocab"])
    both = Decoder(cuda, cfg, w, max_batch=4)
    outs = [both.step(to_dev(toks[p]), p, ops.Mode.ACT_F32)[0].cpu().numpy() for p in range(6)]
    both.close()
    solo = Decoder(cuda, cfg, w, max_batch=1)
    for p in range(6):
        got = solo.step(to_dev(toks[p, 2:3]), p, ops.Mode.ACT_F32)[0].cpu().numpy()
        scale = np.abs(got).max()
        assert np.max(np.abs(got[0] - outs[p][2])) <= 1e-5 * scale
    solo.close()


def test_decode_kv_load_equals_stepping(oracle, cuda):
    """A context installed with kv_load gives the same next-token logits as the oracle that stepped through it."""
    import torch

    cfg, name, batch, ctx_len = SMALL, "dec_small", 2, 9
    w = _weights(oracle, cfg, name)
    ref = oracle.Decoder(cfg, w, batch)
    toks = synth.token_ids(name, "kvload", (ctx_len + 1, batch), cfg["vocab"])
    for p in range(ctx_len):
        ref.step(toks[p], p)
    want = ref.step(toks[ctx_len], ctx_len)
    dec = Decoder(cuda, cfg, w, max_batch=batch)
    dec.load_kv(to_dev(ref.kcache[:, :, :, :ctx_len]), to_dev(ref.vcache[:, :, :, :ctx_len]))
    got = dec.step(to_dev(toks[ctx_len]), ctx_len, ops.Mode.ACT_F32)[0].cpu().numpy()
    assert np.max(np.abs(got - want)) <= 1e-4 * np.abs(want).max()
    dec.close()


def test_decode_rejects_bad_arguments(oracle, cuda):
    cfg, name = LLAMA_LIKE, "dec_llama"
    dec = Decoder(cuda, cfg, _weights(oracle, cfg, name), max_batch=2)
    tok = to_dev(np.zeros(3, np.int32))
    with pytest.raises(ops.SharpMindCudaError):
        dec.step(tok, 0)                       # batch 3 > max_batch 2
    with pytest.raises(ops.SharpMindCudaError):
        dec.step(tok[:2], cfg["max_seq"])      # position past the cache (KVCache.Update throws)
    dec.close()


WIDE = dict(n_layers=2, hidden=1024, n_heads=8, n_kv_heads=4, head_dim=128, ffn=2048, vocab=2048,
            max_seq=32, dtype=8, eps=1e-6, rope_theta=1.0e6, neox=True, qk_norm=True)


def test_decode_one_sequence_fused_path(oracle, cuda):
    """Hidden sizes the TMA GEMV takes put a single sequence on the path where the residual add, the RMSNorms and
    the SiLU-gate ride in the staging of the following matmul: same tolerance as the unfused quantised-activation
    path, and it agrees with row 0 of a two-sequence step (which runs the separate kernels) on the same tokens."""
    import torch

    cfg, name, steps = WIDE, "dec_wide", 8
    w = _weights(oracle, cfg, name)
    ref = oracle.Decoder(cfg, w, 1)
    one = Decoder(cuda, cfg, w, max_batch=1)
    # a host buffer registered twice replaces its first device copy: the second decoder gets its own arrays
    w2 = {k: ([a.copy() for a in v] if isinstance(v, list) else v.copy()) for k, v in w.items()}
    two = Decoder(cuda, cfg, w2, max_batch=2)
    tok = synth.token_ids(name, "prompt", (1,), cfg["vocab"])
    for pos in range(steps):
        want = ref.step(tok, pos)
        t1 = torch.from_numpy(tok.copy()).cuda()
        l1, n1 = one.step(t1, pos, ops.Mode.ACT_Q8)
        l2, _ = two.step(torch.cat([t1, t1]), pos, ops.Mode.ACT_Q8)
        got, pair = l1.cpu().numpy(), l2.cpu().numpy()
        scale = np.abs(want).max()
        assert np.abs(got - want).max() <= 0.05 * scale
        assert np.abs(got[0] - pair[0]).max() <= 2e-3 * scale, float(np.abs(got[0] - pair[0]).max() / scale)
        top2 = np.sort(want[0])[-2:]
        pick = want.argmax(axis=1).astype(np.int32)
        if top2[1] - top2[0] > 0.1 * scale:
            assert n1.cpu().numpy()[0] == pick[0]
        tok = pick
    one.close()
    two.close()
    assert cuda.device_status() == 0


@pytest.mark.parametrize("cfg,name", [(SMALL, "dec_small"), (LLAMA_LIKE, "dec_llama")])
@pytest.mark.parametrize("mode", [ops.Mode.ACT_F32, ops.Mode.REF_ORDER])
def test_prompt_in_one_pass_matches_oracle_stepping(oracle, cuda, cfg, name, mode):
    """ForwardLastLogits over a whole prompt (all tokens in one pass, causal attention among them) gives the logits
    the oracle reaches token by token, leaves a cache that later decode steps continue from, and chunked feeding
    (a second sequence slot, chunks of 5) agrees with the one-pass result."""
    import torch

    n_prompt, n_more = 19, 4
    w = _weights(oracle, cfg, name)
    ref = oracle.Decoder(cfg, w, 1)
    toks = synth.token_ids(name, "prompt_pass", (n_prompt + n_more,), cfg["vocab"])
    for p in range(n_prompt):
        want = ref.step(toks[p:p + 1], p)
    dec = Decoder(cuda, cfg, w, max_batch=2, keep_raw=(mode == ops.Mode.REF_ORDER))
    logits, pick = dec.forward_last_logits(to_dev(toks[:n_prompt]), 0, 0, mode)
    got = logits.cpu().numpy()
    scale = np.abs(want).max()
    assert np.max(np.abs(got - want[0])) <= 1e-4 * scale, float(np.max(np.abs(got - want[0])) / scale)
    assert int(pick.cpu()[0]) == int(got.argmax())
    chunked, _ = dec.forward_last_logits(to_dev(toks[:n_prompt]), 0, 1, mode, chunk=5)
    assert np.max(np.abs(chunked.cpu().numpy() - got)) <= 1e-5 * scale
    # decode continues from the cache the prompt pass wrote (both slots hold the same sequence)
    for p in range(n_prompt, n_prompt + n_more):
        want = ref.step(toks[p:p + 1], p)
        pair = to_dev(np.repeat(toks[p:p + 1], 2))
        out, _ = dec.step(pair, p, mode)
        out = out.cpu().numpy()
        for b in range(2):
            assert np.max(np.abs(out[b] - want[0])) <= 1e-4 * np.abs(want).max()
    dec.close()
    assert cuda.device_status() == 0


def test_prompt_pass_quantised_activations_and_guards(oracle, cuda):
    cfg, name = WIDE, "dec_wide"
    w = _weights(oracle, cfg, name)
    ref = oracle.Decoder(cfg, w, 1)
    toks = synth.token_ids(name, "prompt_q8", (12,), cfg["vocab"])
    for p in range(12):
        want = ref.step(toks[p:p + 1], p)
    dec = Decoder(cuda, cfg, w, max_batch=1)
    got = dec.forward_last_logits(to_dev(toks), 0, 0, ops.Mode.ACT_Q8)[0].cpu().numpy()
    assert np.max(np.abs(got - want[0])) <= 0.05 * np.abs(want).max()
    with pytest.raises(ops.SharpMindCudaError):
        dec.forward_last_logits(to_dev(toks), cfg["max_seq"] - 5, 0)      # runs past the cache
    with pytest.raises(ops.SharpMindCudaError):
        dec.forward_last_logits(to_dev(toks), 0, 1)                       # slot 1 of a one-sequence model
    dec.close()


# Formats mixed per tensor as GGUF K-quant files do: Q4_K attention and gate||up, Q6_K down, Q8_0 embedding / LM head.
MIXED = dict(n_layers=2, hidden=2048, n_heads=16, n_kv_heads=8, head_dim=128, ffn=2048, vocab=1024, max_seq=96,
             dtype=12, down_dtype=14, head_dtype=8, eps=1e-5, rope_theta=5.0e5, neox=False, qk_norm=False)


def test_mixed_format_decoder_prompt_and_decode(oracle, cuda):
    """K-quant decoder: a 70-token prompt in one pass (fp32 activations: Q4_K matmuls of 64 rows and more run on the
    tcgen05 kernel), then decode steps in every mode; one sequence with quantised activations takes the path with the
    norms and the SiLU-gate folded into the one-row Q4_K / Q6_K matmuls."""
    cfg, name, n_prompt = MIXED, "dec_mixed", 70
    w = _weights(oracle, cfg, name)
    ref = oracle.Decoder(cfg, w, 1)
    toks = synth.token_ids(name, "prompt", (n_prompt + 3,), cfg["vocab"])
    for p in range(n_prompt):
        want = ref.step(toks[p:p + 1], p)
    dec = Decoder(cuda, cfg, w, max_batch=1, keep_raw=True)
    got = dec.forward_last_logits(to_dev(toks[:n_prompt]), 0, 0, ops.Mode.ACT_F32, chunk=128)[0].cpu().numpy()
    scale = np.abs(want).max()
    assert np.max(np.abs(got - want[0])) <= 2e-4 * scale, float(np.max(np.abs(got - want[0])) / scale)
    assert int(got.argmax()) == int(want[0].argmax())
    for p, mode, tol in ((n_prompt, ops.Mode.ACT_F32, 2e-4), (n_prompt + 1, ops.Mode.REF_ORDER, 2e-4),
                         (n_prompt + 2, ops.Mode.ACT_Q8, 0.05)):
        want = ref.step(toks[p:p + 1], p)
        out = dec.step(to_dev(toks[p:p + 1]), p, mode)[0].cpu().numpy()
        assert np.max(np.abs(out[0] - want[0])) <= tol * np.abs(want).max(), (mode, float(np.max(np.abs(out[0] - want[0])) / np.abs(want).max()))
    dec.close()
    assert cuda.device_status() == 0


WIDE_FFN = dict(n_layers=2, hidden=1024, n_heads=8, n_kv_heads=2, head_dim=128, ffn=10240, vocab=1024, max_seq=16,
                dtype=8, eps=1e-5, rope_theta=1.0e4, neox=False, qk_norm=False)


def test_decode_one_sequence_wide_ffn(oracle, cuda):
    """An FFN wider than 8192 (Llama-3-8B has 14336): the one-sequence path keeps the norms in the matmul staging but
    runs the SiLU-gate as its own launch; same bars as the fused path, four query heads per KV head."""
    import torch

    cfg, name = WIDE_FFN, "dec_wideffn"
    w = _weights(oracle, cfg, name)
    ref = oracle.Decoder(cfg, w, 1)
    one = Decoder(cuda, cfg, w, max_batch=1)
    w2 = {k: ([a.copy() for a in v] if isinstance(v, list) else v.copy()) for k, v in w.items()}
    two = Decoder(cuda, cfg, w2, max_batch=2)
    tok = synth.token_ids(name, "prompt", (1,), cfg["vocab"])
    for pos in range(6):
        want = ref.step(tok, pos)
        t1 = torch.from_numpy(tok.copy()).cuda()
        got = one.step(t1, pos, ops.Mode.ACT_Q8)[0].cpu().numpy()
        pair = two.step(torch.cat([t1, t1]), pos, ops.Mode.ACT_Q8)[0].cpu().numpy()
        scale = np.abs(want).max()
        assert np.abs(got - want).max() <= 0.05 * scale
        # The two paths take the norm's sum of squares in different orders; a last-bit difference flips the Q8_0
        # rounding of the activations that sit next to a rounding boundary (a few per cent of 10240 elements), which
        # moves an output by a few 1e-3 of its scale per matmul: a looser bar than for the narrow FFN above.
        assert np.abs(got[0] - pair[0]).max() <= 2e-2 * scale
        tok = want.argmax(axis=1).astype(np.int32)
    one.close()
    two.close()
    assert cuda.device_status() == 0
