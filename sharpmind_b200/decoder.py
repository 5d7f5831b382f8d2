"""Device-resident decoder step: host mirror of `Transformer.ForwardLastLogits` for one new token per sequence.

The model is described by the same dictionary `synth.make_decoder_weights` produces (per-layer GGUF byte arrays
for wq / wk / wv / wo / wgu / wdown, fp32 norm vectors, the Q8_0 embedding that doubles as the tied LM head).
Everything runs in the CUDA library (`smc_decode_step`); this class only registers weights and owns handles.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import ops


class _Desc(C.Structure):
    _fields_ = [
        ("n_layers", C.c_int), ("hidden", C.c_int), ("n_heads", C.c_int), ("n_kv_heads", C.c_int),
        ("head_dim", C.c_int), ("ffn", C.c_int), ("vocab", C.c_int), ("max_seq", C.c_int),
        ("eps", C.c_float), ("rope_theta", C.c_float), ("neox", C.c_int), ("qk_norm", C.c_int),
        ("wq", C.POINTER(C.c_void_p)), ("wk", C.POINTER(C.c_void_p)), ("wv", C.POINTER(C.c_void_p)),
        ("wo", C.POINTER(C.c_void_p)), ("wgu", C.POINTER(C.c_void_p)), ("wdown", C.POINTER(C.c_void_p)),
        ("norm1", C.POINTER(C.c_void_p)), ("norm2", C.POINTER(C.c_void_p)),
        ("qnorm", C.POINTER(C.c_void_p)), ("knorm", C.POINTER(C.c_void_p)),
        ("final_norm", C.c_void_p), ("lm_head", C.c_void_p),
        ("bq", C.POINTER(C.c_void_p)), ("bk", C.POINTER(C.c_void_p)), ("bv", C.POINTER(C.c_void_p)),
        ("bo", C.POINTER(C.c_void_p)), ("bgu", C.POINTER(C.c_void_p)), ("bdown", C.POINTER(C.c_void_p)),
        ("kv_dtype", C.c_int),
    ]


class Decoder:
    def __init__(self, ctx: ops.CudaContext, cfg: dict, weights: dict, max_batch: int, keep_raw: bool = False):
        import torch

        self.torch, self.ctx, self.cfg, self.max_batch = torch, ctx, cfg, max_batch
        L, H, hd = cfg["n_layers"], cfg["hidden"], cfg["head_dim"]
        q_dim, kv_dim, F, V, dt = cfg["n_heads"] * hd, cfg["n_kv_heads"] * hd, cfg["ffn"], cfg["vocab"], cfg["dtype"]
        shapes = {"wq": (q_dim, H), "wk": (kv_dim, H), "wv": (kv_dim, H), "wo": (H, q_dim), "wgu": (2 * F, H),
                  "wdown": (H, F)}
        self.w = {}
        self._keep = []

        def reg(raw, n, k, fmt=dt):
            if isinstance(raw, ops.Weight):  # registered already (e.g. straight from a GGUF file)
                if (raw.N, raw.K) != (n, k):
                    raise ops.InvalidOperationException(f"weight is [{raw.N}, {raw.K}], the model needs [{n}, {k}]")
                return raw
            if isinstance(raw, np.ndarray):
                return ctx.register(raw, fmt, n, k, repack=True, keep_raw=keep_raw)
            return ctx.register_dev(raw, fmt, n, k, repack=True, keep_raw=keep_raw)

        # GGUF files mix formats per tensor: the down projection and the embedding may name their own
        fmts = {"wdown": cfg.get("down_dtype") or dt}
        for name, (n, k) in shapes.items():
            self.w[name] = [reg(weights[name][i], n, k, fmts.get(name, dt)) for i in range(L)]
        self.embedding = reg(weights["embedding"], V, H, cfg.get("head_dtype") or dt)
        self.norms = {}
        for name in ("norm1", "norm2", "qnorm", "knorm"):
            self.norms[name] = [self._dev(weights[name][i]) for i in range(L)]
        self.final_norm = self._dev(weights["final_norm"])

        def handles(ws):
            a = (C.c_void_p * L)(*[w.handle for w in ws])
            self._keep.append(a)
            return C.cast(a, C.POINTER(C.c_void_p))

        def ptrs(ts):
            a = (C.c_void_p * L)(*[t.data_ptr() for t in ts])
            self._keep.append(a)
            return C.cast(a, C.POINTER(C.c_void_p))

        d = _Desc()
        d.n_layers, d.hidden, d.n_heads, d.n_kv_heads = L, H, cfg["n_heads"], cfg["n_kv_heads"]
        d.head_dim, d.ffn, d.vocab, d.max_seq = hd, F, V, cfg["max_seq"]
        d.eps, d.rope_theta, d.neox, d.qk_norm = cfg["eps"], cfg["rope_theta"], int(cfg["neox"]), int(cfg["qk_norm"])
        d.wq, d.wk, d.wv, d.wo = handles(self.w["wq"]), handles(self.w["wk"]), handles(self.w["wv"]), handles(self.w["wo"])
        d.wgu, d.wdown = handles(self.w["wgu"]), handles(self.w["wdown"])
        d.norm1, d.norm2 = ptrs(self.norms["norm1"]), ptrs(self.norms["norm2"])
        d.qnorm, d.knorm = ptrs(self.norms["qnorm"]), ptrs(self.norms["knorm"])
        d.final_norm = self.final_norm.data_ptr()
        d.lm_head = self.embedding.handle
        d.kv_dtype = int(cfg.get("kv_dtype", 0))  # 0 = fp32 cache, 8 = Q8_0 rows (QuantizedKVCache)
        # optional bias vectors of the linear layers: weights["bq"] ... ["bdown"], lists of n_layers arrays (or None)
        self.biases = {}
        for name in ("bq", "bk", "bv", "bo", "bgu", "bdown"):
            if weights.get(name) is None:
                continue
            ts = [None if b is None else self._dev(b) for b in weights[name]]
            self.biases[name] = ts
            a = (C.c_void_p * L)(*[None if t_ is None else t_.data_ptr() for t_ in ts])
            self._keep.append(a)
            setattr(d, name, C.cast(a, C.POINTER(C.c_void_p)))
        self._desc = d
        h = C.c_void_p()
        ctx.check(ctx.lib.smc_model_create(ctx.h, C.byref(d), max_batch, C.byref(h)))
        self.h = h

    def _dev(self, a):
        t = self.torch
        if isinstance(a, np.ndarray):
            return t.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).cuda()
        return a.contiguous()

    def load_kv(self, k, v):
        """k, v: CUDA fp32 [layers, batch, kv_heads, len, head_dim]; become cache positions [0, len)."""
        L, B, kvh, ln, hd = k.shape
        self.ctx.check(self.ctx.lib.smc_model_kv_load(self.ctx.h, self.h, k.contiguous().data_ptr(),
                                                      v.contiguous().data_ptr(), B, ln,
                                                      C.c_void_p(self.torch.cuda.current_stream().cuda_stream)))

    def step(self, tokens, pos: int, mode: int = ops.Mode.ACT_Q8, logits=None, argmax=None):
        """tokens: CUDA int32 [batch]. Returns (logits [batch, vocab], greedy token ids [batch])."""
        t = self.torch
        B = tokens.numel()
        if logits is None:
            logits = t.empty((B, self.cfg["vocab"]), dtype=t.float32, device="cuda")
        if argmax is None:
            argmax = t.empty(B, dtype=t.int32, device="cuda")
        self.ctx.check(self.ctx.lib.smc_decode_step(self.ctx.h, self.h, tokens.data_ptr(), B, pos, int(mode),
                                                    logits.data_ptr(), argmax.data_ptr(),
                                                    C.c_void_p(t.cuda.current_stream().cuda_stream)))
        return logits, argmax

    def forward_last_logits(self, tokens, pos: int = 0, seq: int = 0, mode: int = ops.Mode.ACT_Q8, chunk: int = 2048):
        """Prompt processing (Transformer.ForwardLastLogits with seqLen > 1): tokens is CUDA int32 [seqLen], one
        sequence, placed at positions pos .. pos + seqLen - 1 of cache slot `seq`, fed in chunks of `chunk` tokens.
        Returns (logits [vocab] of the last token, its greedy pick [1])."""
        t = self.torch
        n = tokens.numel()
        logits = t.empty(self.cfg["vocab"], dtype=t.float32, device="cuda")
        argmax = t.empty(1, dtype=t.int32, device="cuda")
        if n == 0:
            raise ValueError("forward_last_logits: empty prompt")
        for start in range(0, n, chunk):
            part = tokens[start:start + chunk].contiguous()
            self.ctx.check(self.ctx.lib.smc_forward_last_logits(self.ctx.h, self.h, part.data_ptr(), part.numel(), seq,
                                                                pos + start, int(mode), logits.data_ptr(), argmax.data_ptr(),
                                                                C.c_void_p(t.cuda.current_stream().cuda_stream)))
        return logits, argmax

    def forward_logits(self, tokens, pos: int, seq: int = 0, mode: int = ops.Mode.ACT_Q8, want_hidden: bool = False):
        """Transformer.Forward over the tokens of one sequence (a verification round's K + 1 draft tokens): returns
        (logits [seqLen, vocab], greedy pick per row [seqLen], final-normed hidden states [seqLen, hidden] or None)."""
        t = self.torch
        n = tokens.numel()
        logits = t.empty((n, self.cfg["vocab"]), dtype=t.float32, device="cuda")
        argmax = t.empty(n, dtype=t.int32, device="cuda")
        hidden = t.empty((n, self.cfg["hidden"]), dtype=t.float32, device="cuda") if want_hidden else None
        self.ctx.check(self.ctx.lib.smc_forward_logits(self.ctx.h, self.h, tokens.contiguous().data_ptr(), n, seq, pos, int(mode),
                                                       logits.data_ptr(), argmax.data_ptr(),
                                                       None if hidden is None else hidden.data_ptr(),
                                                       C.c_void_p(t.cuda.current_stream().cuda_stream)))
        return logits, argmax, hidden

    def verify_greedy(self, argmax, draft):
        """1 + the number of leading head guesses the model agrees with (MedusaGenerator's acceptance rule)."""
        t = self.torch
        acc = t.zeros(1, dtype=t.int32, device="cuda")
        self.ctx.check(self.ctx.lib.smc_verify_greedy_dev(self.ctx.h, argmax.data_ptr(), draft.contiguous().data_ptr(), draft.numel() - 1,
                                                          acc.data_ptr(), C.c_void_p(t.cuda.current_stream().cuda_stream)))
        return int(acc.item())

    def medusa_predict(self, hidden, head_w, head_b):
        """MedusaHeads.Predict: hidden [hidden] (final-normed), head_w [k, hidden, hidden], head_b [k, hidden] -> tokens [k]."""
        t = self.torch
        k, H = head_w.shape[0], self.cfg["hidden"]
        work = t.empty(k * (H + self.cfg["vocab"]), dtype=t.float32, device="cuda")
        out = t.empty(k, dtype=t.int32, device="cuda")
        self.ctx.check(self.ctx.lib.smc_medusa_predict_dev(self.ctx.h, hidden.contiguous().data_ptr(), head_w.contiguous().data_ptr(),
                                                           head_b.contiguous().data_ptr(), k, H, self.embedding.handle, work.data_ptr(),
                                                           out.data_ptr(), C.c_void_p(t.cuda.current_stream().cuda_stream)))
        return out

    def close(self):
        if self.h:
            self.ctx.lib.smc_model_destroy(self.ctx.h, self.h)
            self.h = None
