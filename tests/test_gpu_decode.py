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


# SMC_ACT_Q8 against the oracle run in the same arithmetic (every matmul input quantised to Q8_0 and dequantised,
# oracle.Decoder.step(act_q8=True)).  The two sides differ by fp32 rounding only, and where no activation sits on a
# rounding boundary their logits agree to 1e-7 of the logit scale (measured).  But rounding to int8 is not continuous:
# an activation whose quotient x/d lies within that fp32 noise of a half is quantised one step apart on the two sides
# ("a flip"), which moves the outputs of that matmul by about d * w.  Every later matmul re-quantises the perturbed
# activations, where more of them now flip, so one early flip grows into a difference of the size of the Q8_0
# quantisation noise itself: measured 3e-3 .. 9e-3 of the logit scale on the two- and three-layer models here, 1.6e-2 on
# a two-layer model of the benchmark's widths (worst of 151 936 logits), 6e-2 .. 8e-2 after 28 layers.  No
# implementation of this mode can be pinned tighter against another one; what can be pinned is that the arithmetic
# model is right (flip-free steps agree to 1e-7) and that nothing exceeds the noise.  The bars therefore are
#   * shallow models: every step within 3e-2, and at least three quarters of the steps of the small models flip-free
#     (within 1e-5);
#   * the 28-layer configuration: within 1.2e-1 in SMC_ACT_Q8, while the same model is held to 1e-4 (measured 6e-6)
#     with an exact top-1 match in SMC_ACT_F32 and SMC_REF_ORDER;
#   * in SMC_ACT_Q8 top-1 agrees wherever the oracle's margin between its two best tokens exceeds twice the bar (the
#     bar itself for the deep model).
Q8_SHALLOW_TOL, Q8_DEEP_TOL, Q8_EXACT = 3e-2, 1.2e-1, 1e-5


def _q8_step_check(want, got, picked, worst, tol=Q8_SHALLOW_TOL, margin=2.0):
    """Returns (worst error so far, the oracle's greedy tokens, rows whose top-1 was decidable, rows that were flip-free)."""
    scale = np.abs(want).max(axis=1)
    err = np.abs(got - want).max(axis=1) / scale
    assert np.all(err <= tol), err
    top2 = np.sort(want, axis=1)[:, -2:]
    clear = (top2[:, 1] - top2[:, 0]) > margin * tol * scale
    pick = want.argmax(axis=1).astype(np.int32)
    assert np.array_equal(picked[clear], pick[clear])
    return max(worst, float(err.max())), pick, int(clear.sum()), int((err <= Q8_EXACT).sum())


@pytest.mark.parametrize("cfg,name", [(SMALL, "dec_small"), (LLAMA_LIKE, "dec_llama")])
@pytest.mark.parametrize("batch", [1, 4])
def test_decode_quantised_activations_match_q8_oracle(oracle, cuda, cfg, name, batch):
    import torch

    steps = 16
    w = _weights(oracle, cfg, name)
    ref = oracle.Decoder(cfg, w, batch)
    dec = Decoder(cuda, cfg, w, max_batch=batch)
    tok = synth.token_ids(name, "prompt", (batch,), cfg["vocab"])
    worst, decided, exact = 0.0, 0, 0
    for pos in range(steps):
        want = ref.step(tok, pos, act_q8=True)
        logits, nxt = dec.step(torch.from_numpy(tok.copy()).cuda(), pos, ops.Mode.ACT_Q8)
        worst, tok, n, ex = _q8_step_check(want, logits.cpu().numpy(), nxt.cpu().numpy(), worst)
        decided += n
        exact += ex
    dec.close()
    print(f"ACT_Q8 decode vs Q8 oracle, {name} batch {batch}: worst logit error {worst:.2e} of scale, "
          f"{exact}/{steps * batch} flip-free, {decided} decidable")
    assert exact >= steps * batch * 3 // 4, "too many steps differ by more than rounding"
    assert decided >= steps * batch // 2, "too few steps had a decidable top-1"


def _qwen3_device_weights(dev, cfg, seed):
    import torch

    g = torch.Generator(device="cuda").manual_seed(seed)
    L, H, hd = cfg["n_layers"], cfg["hidden"], cfg["head_dim"]
    q_dim, kv_dim, F, V = cfg["n_heads"] * hd, cfg["n_kv_heads"] * hd, cfg["ffn"], cfg["vocab"]

    def mat(n, k):
        return dev.quantize_weights(cfg["dtype"], torch.randn((n, k), generator=g, device="cuda") * 0.02)

    def vec(n):
        return torch.randn(n, generator=g, device="cuda") * 0.1 + 1.0

    wd = {k: [] for k in ("wq", "wk", "wv", "wo", "wgu", "wdown", "norm1", "norm2", "qnorm", "knorm")}
    for _ in range(L):
        wd["wq"].append(mat(q_dim, H)), wd["wk"].append(mat(kv_dim, H)), wd["wv"].append(mat(kv_dim, H))
        wd["wo"].append(mat(H, q_dim)), wd["wgu"].append(mat(2 * F, H)), wd["wdown"].append(mat(H, F))
        wd["norm1"].append(vec(H)), wd["norm2"].append(vec(H)), wd["qnorm"].append(vec(hd)), wd["knorm"].append(vec(hd))
    wd["final_norm"] = vec(H)
    wd["embedding"] = mat(V, H)
    wh = {k: ([t.cpu().numpy() for t in v] if isinstance(v, list) else v.cpu().numpy()) for k, v in wd.items()}
    return wd, wh, g


@pytest.mark.parametrize("n_layers", [2, 28])
def test_decode_full_qwen3_0_6b_shape_against_oracle(oracle, cuda, dev, n_layers):
    """The benchmarked decode configuration itself: hidden 1024, 16 / 8 heads of 128, FFN 3072, vocabulary 151 936, all
    matrices Q8_0 drawn on the device (the oracle gets the same bytes), a seeded 2048-position context installed on both
    sides, then greedy steps with teacher forcing.  Batch 1 (the one-sequence path with its fused staging) in
    SMC_ACT_Q8, SMC_ACT_F32 and SMC_REF_ORDER, and rows 0 and 21 of a batch of 32 (the small-batch kernels) in
    SMC_ACT_Q8.  28 layers is the configuration; the two-layer cut keeps SMC_ACT_Q8 clear of the flip cascade
    described above and is held to the shallow bar."""
    import torch

    cfg = dict(synth.QWEN3_0_6B)
    cfg["n_layers"] = n_layers
    deep = n_layers > 4
    ctx_len, steps_q8, steps_f32 = 2048, (16 if deep else 6), (16 if deep else 3)
    q8_tol, q8_margin = (Q8_DEEP_TOL, 1.0) if deep else (Q8_SHALLOW_TOL, 2.0)
    wd, wh, g = _qwen3_device_weights(dev, cfg, 20240611)
    L, hd, V = n_layers, cfg["head_dim"], cfg["vocab"]
    # context: the same seeded K / V rows for the sequences that are compared (rows 0 and 21 of the batch of 32)
    rows = (0, 21)
    kv_shape = (L, 32, cfg["n_kv_heads"], ctx_len, hd)
    kd, vd = torch.randn(kv_shape, generator=g, device="cuda"), torch.randn(kv_shape, generator=g, device="cuda")
    tok32 = synth.token_ids("qwen3_full", "tok32", (32,), V)

    def oracle_with_context(sel):
        ref = oracle.Decoder(cfg, wh, len(sel))
        for i, r in enumerate(sel):
            ref.kcache[:, i, :, :ctx_len] = kd[:, r].cpu().numpy()
            ref.vcache[:, i, :, :ctx_len] = vd[:, r].cpu().numpy()
        return ref

    # ---- batch 1, every mode
    for mode, steps in ((ops.Mode.ACT_F32, steps_f32), (ops.Mode.REF_ORDER, steps_f32), (ops.Mode.ACT_Q8, steps_q8)):
        ref = oracle_with_context((0,))
        dec = Decoder(cuda, cfg, wd, max_batch=1, keep_raw=(mode == ops.Mode.REF_ORDER))
        dec.load_kv(kd[:, 0:1].contiguous(), vd[:, 0:1].contiguous())
        tok = tok32[0:1].copy()
        worst = 0.0
        for s in range(steps):
            pos = ctx_len + s
            want = ref.step(tok, pos, act_q8=(mode == ops.Mode.ACT_Q8))
            logits, nxt = dec.step(to_dev(tok), pos, mode)
            got, picked = logits.cpu().numpy(), nxt.cpu().numpy()
            if mode == ops.Mode.ACT_Q8:
                worst, tok, _, _ = _q8_step_check(want, got, picked, worst, q8_tol, q8_margin)
            else:
                scale = np.abs(want).max()
                worst = max(worst, float(np.abs(got - want).max() / scale))
                assert np.abs(got - want).max() <= 1e-4 * scale, (mode, worst)
                top2 = np.sort(want[0])[-2:]
                tok = want.argmax(axis=1).astype(np.int32)
                if top2[1] - top2[0] > 2e-4 * scale:
                    assert picked[0] == tok[0]
        print(f"Qwen3-0.6B shape, {n_layers} layers, batch 1, mode {int(mode)}: worst logit error {worst:.2e} of scale over {steps} steps")
        dec.close()
        del ref
    # ---- batch 32 (lock-step sequences, the small-batch kernels), two of its rows against the oracle
    ref = oracle_with_context(rows)
    dec = Decoder(cuda, cfg, wd, max_batch=32)
    dec.load_kv(kd, vd)
    del kd, vd
    tok = tok32.copy()
    worst = 0.0
    for s in range(4):
        pos = ctx_len + s
        want = ref.step(tok[list(rows)], pos, act_q8=True)
        logits, nxt = dec.step(to_dev(tok), pos, ops.Mode.ACT_Q8)
        got, picked = logits.cpu().numpy(), nxt.cpu().numpy()
        worst, pick, _, _ = _q8_step_check(want, got[list(rows)], picked[list(rows)], worst, q8_tol, q8_margin)
        tok = picked.copy()          # the other sequences follow their own greedy tokens
        tok[list(rows)] = pick       # the compared ones are teacher-forced on the oracle's
    print(f"Qwen3-0.6B shape, {n_layers} layers, batch 32 rows {rows}: worst logit error {worst:.2e} of scale")
    dec.close()
    assert cuda.device_status() == 0


@pytest.mark.parametrize("which", ["qkv", "all"])
@pytest.mark.parametrize("mode", [ops.Mode.ACT_F32, ops.Mode.REF_ORDER, ops.Mode.ACT_Q8])
def test_decode_with_linear_biases(oracle, cuda, which, mode):
    """Linear layers with a bias (InferenceLinearLayer.Forward -> LinearLayer.AddBiasInPlace): the attention
    projections only, as Qwen2-class checkpoints have them, or every linear layer; decode steps and a prompt pass."""
    cfg, name, batch = SMALL, "dec_small", 2
    w = dict(_weights(oracle, cfg, name))
    L, H, hd = cfg["n_layers"], cfg["hidden"], cfg["head_dim"]
    q_dim, kv_dim, F = cfg["n_heads"] * hd, cfg["n_kv_heads"] * hd, cfg["ffn"]
    sizes = {"bq": q_dim, "bk": kv_dim, "bv": kv_dim, "bo": H, "bgu": 2 * F, "bdown": H}
    for bname, n in sizes.items():
        if which == "qkv" and bname not in ("bq", "bk", "bv"):
            continue
        # one layer keeps a missing vector: entries may be null
        w[bname] = [None if (bname == "bo" and i == 1) else synth.normal(name, f"l{i}.{bname}", (n,), 0.05) for i in range(L)]
    ref = oracle.Decoder(cfg, w, batch)
    dec = Decoder(cuda, cfg, w, max_batch=batch, keep_raw=(mode == ops.Mode.REF_ORDER))
    tok = synth.token_ids(name, "bias_prompt", (batch,), cfg["vocab"])
    q8 = mode == ops.Mode.ACT_Q8
    for pos in range(6):
        want = ref.step(tok, pos, act_q8=q8)
        logits, _ = dec.step(to_dev(tok), pos, mode)
        got = logits.cpu().numpy()
        scale = np.abs(want).max()
        assert np.abs(got - want).max() <= (Q8_SHALLOW_TOL if q8 else 1e-4) * scale, float(np.abs(got - want).max() / scale)
        tok = want.argmax(axis=1).astype(np.int32)
    # a prompt pass of sequence 0 over its own six tokens lands on the oracle's next logits
    if not q8:
        ref1 = oracle.Decoder(cfg, w, 1)
        toks = synth.token_ids(name, "bias_pass", (7,), cfg["vocab"])
        for p in range(7):
            want1 = ref1.step(toks[p:p + 1], p)
        got1 = dec.forward_last_logits(to_dev(toks), 0, 1, mode)[0].cpu().numpy()
        assert np.abs(got1 - want1[0]).max() <= 1e-4 * np.abs(want1).max()
    dec.close()


@pytest.mark.parametrize("cfg0,name", [(SMALL, "dec_small"), (LLAMA_LIKE, "dec_llama")])
@pytest.mark.parametrize("mode", [ops.Mode.ACT_F32, ops.Mode.REF_ORDER])
def test_decode_with_q8_0_kv_cache(oracle, cuda, cfg0, name, mode):
    """kv_dtype = Q8_0 (QuantizedKVCache): a prompt pass writes quantised K / V rows, decode steps (one sequence and
    two) append to them and attend over them; against the oracle whose cache holds what those rows decode to.  A K or V
    element whose quotient sits on a rounding boundary may quantise one step apart on the two sides (one element of one
    cached row: a few 1e-5 of the attention output), hence 1e-3 rather than the 1e-4 of the fp32 cache."""
    cfg = dict(cfg0, kv_dtype=8)
    w = _weights(oracle, cfg, name)
    n_prompt = 9
    toks = synth.token_ids(name, "q8kv", (n_prompt + 5, 2), cfg["vocab"])
    ref = oracle.Decoder(cfg, w, 2)
    for p in range(n_prompt):
        want = ref.step(toks[p], p)
    dec = Decoder(cuda, cfg, w, max_batch=2, keep_raw=(mode == ops.Mode.REF_ORDER))
    for seq in range(2):
        got = dec.forward_last_logits(to_dev(np.ascontiguousarray(toks[:n_prompt, seq])), 0, seq, mode)[0].cpu().numpy()
        assert np.abs(got - want[seq]).max() <= 1e-3 * np.abs(want).max(), float(np.abs(got - want[seq]).max() / np.abs(want).max())
    for p in range(n_prompt, n_prompt + 5):
        want = ref.step(toks[p], p)
        got = dec.step(to_dev(toks[p]), p, mode)[0].cpu().numpy()
        assert np.abs(got - want).max() <= 1e-3 * np.abs(want).max(), (p, float(np.abs(got - want).max() / np.abs(want).max()))
    dec.close()
    # one sequence with quantised activations takes the fused one-row path over the same cache format
    ref1 = oracle.Decoder(cfg, w, 1)
    dec1 = Decoder(cuda, cfg, w, max_batch=1)
    tok = toks[0, :1].copy()
    for p in range(6):
        want = ref1.step(tok, p, act_q8=True)
        got = dec1.step(to_dev(tok), p, ops.Mode.ACT_Q8)[0].cpu().numpy()
        assert np.abs(got - want).max() <= Q8_SHALLOW_TOL * np.abs(want).max()
        tok = want.argmax(axis=1).astype(np.int32)
    dec1.close()
    assert cuda.device_status() == 0


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
    worst = 0.0
    for pos in range(steps):
        want = ref.step(tok, pos, act_q8=True)
        t1 = torch.from_numpy(tok.copy()).cuda()
        l1, n1 = one.step(t1, pos, ops.Mode.ACT_Q8)
        l2, _ = two.step(torch.cat([t1, t1]), pos, ops.Mode.ACT_Q8)
        got, pair = l1.cpu().numpy(), l2.cpu().numpy()
        scale = np.abs(want).max()
        assert np.abs(got[0] - pair[0]).max() <= 2e-3 * scale, float(np.abs(got[0] - pair[0]).max() / scale)
        worst, tok, _, _ = _q8_step_check(want, got, n1.cpu().numpy(), worst)
    print(f"fused one-sequence path vs Q8 oracle: worst logit error {worst:.2e} of scale")
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
        want = ref.step(toks[p:p + 1], p, act_q8=True)
    dec = Decoder(cuda, cfg, w, max_batch=1)
    got = dec.forward_last_logits(to_dev(toks), 0, 0, ops.Mode.ACT_Q8)[0].cpu().numpy()
    assert np.max(np.abs(got - want[0])) <= Q8_SHALLOW_TOL * np.abs(want).max(), float(np.max(np.abs(got - want[0])) / np.abs(want).max())
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
                         (n_prompt + 2, ops.Mode.ACT_Q8, Q8_SHALLOW_TOL)):
        want = ref.step(toks[p:p + 1], p, act_q8=(mode == ops.Mode.ACT_Q8))
        out = dec.step(to_dev(toks[p:p + 1]), p, mode)[0].cpu().numpy()
        assert np.max(np.abs(out[0] - want[0])) <= tol * np.abs(want).max(), (mode, float(np.max(np.abs(out[0] - want[0])) / np.abs(want).max()))
    dec.close()
    assert cuda.device_status() == 0


WIDE_FFN = dict(n_layers=2, hidden=1024, n_heads=8, n_kv_heads=2, head_dim=128, ffn=10240, vocab=1024, max_seq=16,
                dtype=8, eps=1e-5, rope_theta=1.0e4, neox=False, qk_norm=False)


def test_decode_one_sequence_wide_ffn(oracle, cuda):
    """An FFN wider than 8192 (Llama-3-8B has 14336): the one-sequence path keeps the norms in the matmul staging and,
    up to `decode_gate_in_staging_max_ffn` (default 16384), the SiLU-gate in the down projection's staging too (the two
    SMs of a pair share that work); above it the gate is a launch of its own.  Both forms give the same bits (the
    staged row is quantised by the same code), same bars as the narrow FFN, four query heads per KV head."""
    import torch

    cfg, name = WIDE_FFN, "dec_wideffn"
    w = _weights(oracle, cfg, name)
    # the two forms of the gate, bit for bit
    runs = []
    for limit in (16384, 8192):
        cuda.set_option("decode_gate_in_staging_max_ffn", limit)
        try:
            d = Decoder(cuda, cfg, {k: ([a.copy() for a in v] if isinstance(v, list) else v.copy()) for k, v in w.items()}, max_batch=1)
            tk = torch.from_numpy(synth.token_ids(name, "prompt", (1,), cfg["vocab"]).copy()).cuda()
            outs = []
            for pos in range(5):
                lg, tk = d.step(tk, pos, ops.Mode.ACT_Q8)
                outs.append(lg.clone())
                tk = tk.clone()
            d.close()
            runs.append(torch.stack(outs))
        finally:
            cuda.set_option("decode_gate_in_staging_max_ffn", 16384)
    assert torch.equal(runs[0], runs[1])
    ref = oracle.Decoder(cfg, w, 1)
    one = Decoder(cuda, cfg, w, max_batch=1)
    w2 = {k: ([a.copy() for a in v] if isinstance(v, list) else v.copy()) for k, v in w.items()}
    two = Decoder(cuda, cfg, w2, max_batch=2)
    tok = synth.token_ids(name, "prompt", (1,), cfg["vocab"])
    for pos in range(6):
        want = ref.step(tok, pos, act_q8=True)
        t1 = torch.from_numpy(tok.copy()).cuda()
        got = one.step(t1, pos, ops.Mode.ACT_Q8)[0].cpu().numpy()
        pair = two.step(torch.cat([t1, t1]), pos, ops.Mode.ACT_Q8)[0].cpu().numpy()
        scale = np.abs(want).max()
        assert np.abs(got - want).max() <= 2e-2 * scale, float(np.abs(got - want).max() / scale)
        # The two paths take the norm's sum of squares in different orders; a last-bit difference flips the Q8_0
        # rounding of the activations that sit next to a rounding boundary (a few per cent of 10240 elements), which
        # moves an output by a few 1e-3 of its scale per matmul: a looser bar than for the narrow FFN above.
        assert np.abs(got[0] - pair[0]).max() <= 2e-2 * scale
        tok = want.argmax(axis=1).astype(np.int32)
    one.close()
    two.close()
    assert cuda.device_status() == 0
