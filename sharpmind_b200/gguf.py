"""GGUF files to device-resident weights: host mirror of the reference's GgufLoader for the tensors of the hot path.

`GgufFile` wraps the library's memory-mapped reader (smc_gguf_*); `load_decoder` maps the tensor names llama.cpp
writes (token_embd, blk.N.attn_q / attn_k / attn_v / attn_output / ffn_gate / ffn_up / ffn_down, the norm vectors,
output_norm) onto a `Decoder` (SharpMind.Model/Format/GgufLoader.cs:435-510 resolves the same names onto
TransformerWeights).  Only Q8_0, Q4_K and Q6_K matrices have kernels; a file that holds another format for one of
them is refused with NotSupportedException.
"""
from __future__ import annotations

import ctypes as C

from . import ops


class GgufFile:
    def __init__(self, ctx: ops.CudaContext, path: str):
        self.ctx, self.lib = ctx, ctx.lib
        h = C.c_void_p()
        ctx.check(self.lib.smc_gguf_open(ctx.h, path.encode(), C.byref(h)))
        self.h = h
        self.tensors = {}
        for i in range(self.lib.smc_gguf_tensor_count(h)):
            name, dt, nd, nbytes = C.c_char_p(), C.c_int(), C.c_int(), C.c_int64()
            dims = (C.c_int64 * 4)()
            self.lib.smc_gguf_tensor_info(h, i, C.byref(name), C.byref(dt), C.byref(nd), dims, C.byref(nbytes))
            self.tensors[name.value.decode()] = dict(index=i, dtype=dt.value, dims=list(dims)[:nd.value], bytes=nbytes.value)

    def close(self):
        if self.h:
            self.lib.smc_gguf_close(self.ctx.h, self.h)
            self.h = None

    def meta_int(self, key: str, default=None):
        v = C.c_int64()
        return v.value if self.lib.smc_gguf_meta_int(self.h, key.encode(), C.byref(v)) == 0 else default

    def meta_float(self, key: str, default=None):
        v = C.c_double()
        return v.value if self.lib.smc_gguf_meta_float(self.h, key.encode(), C.byref(v)) == 0 else default

    def meta_string(self, key: str, default=None):
        s = self.lib.smc_gguf_meta_string(self.h, key.encode())
        return s.decode() if s is not None else default

    def register(self, name: str, keep_raw: bool = False) -> ops.Weight:
        t = self.tensors[name]
        h = C.c_void_p()
        flags = ops.W_REPACK | (ops.W_KEEP_RAW if keep_raw else 0)
        self.ctx.check(self.lib.smc_gguf_register(self.ctx.h, self.h, t["index"], flags, C.byref(h)))
        return ops.Weight(h, t["dtype"], t["dims"][1], t["dims"][0], None)

    def read_f32(self, name: str):
        import torch

        t = self.tensors[name]
        n = 1
        for d in t["dims"]:
            n *= d
        out = torch.empty(n, dtype=torch.float32, device=f"cuda:{self.ctx.device}")
        self.ctx.check(self.lib.smc_gguf_read_f32(self.ctx.h, self.h, t["index"], out.data_ptr(), n))
        return out


def decoder_config(f: GgufFile, max_seq: int) -> dict:
    """ModelConfig fields of the hot path from the file's metadata (GgufLoader.LoadConfig, GgufLoader.cs:180-283)."""
    arch = f.meta_string("general.architecture", "llama")
    heads = f.meta_int(f"{arch}.attention.head_count")
    hidden = f.meta_int(f"{arch}.embedding_length")
    head_dim = f.meta_int(f"{arch}.attention.key_length", hidden // heads)
    emb = f.tensors["token_embd.weight"]
    return dict(
        n_layers=f.meta_int(f"{arch}.block_count"), hidden=hidden, n_heads=heads,
        n_kv_heads=f.meta_int(f"{arch}.attention.head_count_kv", heads), head_dim=head_dim,
        ffn=f.meta_int(f"{arch}.feed_forward_length"), vocab=emb["dims"][1], max_seq=max_seq,
        dtype=f.tensors["blk.0.attn_q.weight"]["dtype"], down_dtype=f.tensors["blk.0.ffn_down.weight"]["dtype"],
        head_dtype=emb["dtype"], eps=f.meta_float(f"{arch}.attention.layer_norm_rms_epsilon", 1e-5),
        rope_theta=f.meta_float(f"{arch}.rope.freq_base", 10000.0),
        # AttentionLayer.cs:132-144: llama pairs adjacent elements, qwen / gemma / phi the two halves
        neox=arch not in ("llama", "mistral"), qk_norm="blk.0.attn_q_norm.weight" in f.tensors)


def load_decoder(ctx: ops.CudaContext, path: str, max_seq: int, max_batch: int = 1):
    """Opens `path`, registers every matrix of the decoder from the mapped file and returns (Decoder, config)."""
    import torch

    from .decoder import Decoder

    f = GgufFile(ctx, path)
    try:
        cfg = decoder_config(f, max_seq)
        L = cfg["n_layers"]
        w = {k: [] for k in ("wq", "wk", "wv", "wo", "wgu", "wdown", "norm1", "norm2", "qnorm", "knorm")}
        hd = cfg["head_dim"]
        for i in range(L):
            b = f"blk.{i}."
            w["wq"].append(f.register(b + "attn_q.weight")), w["wk"].append(f.register(b + "attn_k.weight"))
            w["wv"].append(f.register(b + "attn_v.weight")), w["wo"].append(f.register(b + "attn_output.weight"))
            gate, up = f.register(b + "ffn_gate.weight"), f.register(b + "ffn_up.weight")
            joined = C.c_void_p()  # gate rows followed by up rows: the fused matrix FfnKernels.Gated multiplies by
            parts = (C.c_void_p * 2)(gate.handle, up.handle)
            ctx.check(ctx.lib.smc_weight_concat_rows(ctx.h, parts, 2, C.byref(joined)))
            w["wgu"].append(ops.Weight(joined, gate.dtype, gate.N + up.N, gate.K, None))
            ctx.release(gate), ctx.release(up)
            w["wdown"].append(f.register(b + "ffn_down.weight"))
            w["norm1"].append(f.read_f32(b + "attn_norm.weight")), w["norm2"].append(f.read_f32(b + "ffn_norm.weight"))
            if cfg["qk_norm"]:
                w["qnorm"].append(f.read_f32(b + "attn_q_norm.weight")), w["knorm"].append(f.read_f32(b + "attn_k_norm.weight"))
            else:
                one = torch.ones(hd, device=f"cuda:{ctx.device}")
                w["qnorm"].append(one), w["knorm"].append(one)
            for bname, tname in (("bq", "attn_q.bias"), ("bk", "attn_k.bias"), ("bv", "attn_v.bias")):
                if b + tname in f.tensors:
                    w.setdefault(bname, [None] * L)[i] = f.read_f32(b + tname)
        w["final_norm"] = f.read_f32("output_norm.weight")
        w["embedding"] = f.register("token_embd.weight")
        return Decoder(ctx, cfg, w, max_batch=max_batch), cfg
    finally:
        f.close()
