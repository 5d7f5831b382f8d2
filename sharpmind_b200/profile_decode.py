"""Times the device-resident decode step on the Qwen3-0.6B-shaped configuration (Q8_0 weights, fp32 KV), or with
`--model llama8b` on a Llama-3-8B shape with K-quant weights; `--prompt N` times the multi-token prompt pass.

    python -m sharpmind_b200.profile_decode [--batches 1,8,32] [--ctx 2048] [--steps 64] [--modes q8,f32]
                                            [--layers 28] [--once] [--model qwen3|llama8b] [--prompt N --chunk C]

Weights are seeded normal(0, 0.02) values quantised on the device, the context is `ctx` positions of
seeded normal K/V installed with kv_load (no prompt is run: the step's cost depends on the context length
only), and every timed step decodes one token per sequence at position `ctx`.  Two timings are printed per
(batch, mode): plain launches on a stream, and the same step captured once in a CUDA graph and replayed.
`--once` runs a single untimed step per case (for a profiler).
"""
from __future__ import annotations

import argparse
import json

from . import ops, synth
from .decoder import Decoder

MODES = {"q8": ops.Mode.ACT_Q8, "f32": ops.Mode.ACT_F32}


def device_weights(dev: ops.DeviceOps, cfg: dict, seed: int = 1234) -> dict:
    import torch

    g = torch.Generator(device="cuda")
    g.manual_seed(seed)
    L, H, hd = cfg["n_layers"], cfg["hidden"], cfg["head_dim"]
    q_dim, kv_dim, F, V, dt = cfg["n_heads"] * hd, cfg["n_kv_heads"] * hd, cfg["ffn"], cfg["vocab"], cfg["dtype"]

    def mat(n, k, fmt=None):
        return dev.quantize_weights(fmt or dt, torch.randn((n, k), generator=g, device="cuda") * 0.02)

    def vec(n):
        return torch.randn(n, generator=g, device="cuda") * 0.1 + 1.0

    w = {k: [] for k in ("wq", "wk", "wv", "wo", "wgu", "wdown", "norm1", "norm2", "qnorm", "knorm")}
    for _ in range(L):
        w["wq"].append(mat(q_dim, H)), w["wk"].append(mat(kv_dim, H)), w["wv"].append(mat(kv_dim, H))
        w["wo"].append(mat(H, q_dim)), w["wgu"].append(mat(2 * F, H)), w["wdown"].append(mat(H, F, cfg.get("down_dtype")))
        w["norm1"].append(vec(H)), w["norm2"].append(vec(H)), w["qnorm"].append(vec(hd)), w["knorm"].append(vec(hd))
    w["final_norm"] = vec(H)
    w["embedding"] = mat(V, H, cfg.get("head_dtype"))
    return w


def step_bytes(cfg: dict, batch: int, ctx: int) -> dict:
    """Bytes one step has to read: every weight block once, and the K/V rows of the context per sequence."""
    L, H, hd = cfg["n_layers"], cfg["hidden"], cfg["head_dim"]
    q_dim, kv_dim, F, V = cfg["n_heads"] * hd, cfg["n_kv_heads"] * hd, cfg["ffn"], cfg["vocab"]
    bpe = {8: 34 / 32, 12: 144 / 256, 14: 210 / 256}  # bytes per element of each block format
    dt = cfg["dtype"]
    per_layer = (q_dim * H + 2 * kv_dim * H + H * q_dim + 2 * F * H) * bpe[dt] + H * F * bpe[cfg.get("down_dtype") or dt]
    weights = int(L * per_layer + V * H * bpe[cfg.get("head_dtype") or dt])
    kv = L * batch * 2 * cfg["n_kv_heads"] * (ctx + 1) * hd * 4
    return {"weights": weights, "kv": kv}


def time_decode(ctx, dev, cfg: dict, batches, ctx_len: int, steps: int, modes=("q8",), once: bool = False) -> list:
    """Builds the model, installs a `ctx_len`-position context and times one-token steps; one dict per case."""
    import torch

    w = device_weights(dev, cfg)
    dec = Decoder(ctx, cfg, w, max_batch=max(batches))
    del w
    g = torch.Generator(device="cuda")
    g.manual_seed(99)
    shape = (cfg["n_layers"], max(batches), cfg["n_kv_heads"], ctx_len, cfg["head_dim"])
    k, v = torch.randn(shape, generator=g, device="cuda"), torch.randn(shape, generator=g, device="cuda")
    dec.load_kv(k, v)
    torch.cuda.synchronize()
    del k, v
    torch.cuda.empty_cache()
    rows = []
    for B in batches:
        tok = torch.randint(0, cfg["vocab"], (B,), generator=g, device="cuda", dtype=torch.int32)
        logits = torch.empty((B, cfg["vocab"]), device="cuda")
        nxt = torch.empty(B, dtype=torch.int32, device="cuda")
        for name in modes:
            mode = MODES[name]
            if once:
                dec.step(tok, ctx_len, mode, logits, nxt)
                torch.cuda.synchronize()
                continue
            for _ in range(3):
                dec.step(tok, ctx_len, mode, logits, nxt)
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(steps):
                dec.step(tok, ctx_len, mode, logits, nxt)
            e1.record()
            torch.cuda.synchronize()
            plain_ms = e0.elapsed_time(e1) / steps
            side = torch.cuda.Stream()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.stream(side):
                dec.step(tok, ctx_len, mode, logits, nxt)
                side.synchronize()
                with torch.cuda.graph(graph, stream=side):
                    dec.step(tok, ctx_len, mode, logits, nxt)
            torch.cuda.synchronize()
            for _ in range(3):
                graph.replay()
            e0.record()
            for _ in range(steps):
                graph.replay()
            e1.record()
            torch.cuda.synchronize()
            graph_ms = e0.elapsed_time(e1) / steps
            by = step_bytes(cfg, B, ctx_len)
            rows.append({
                "batch": B, "mode": name, "ctx": ctx_len, "layers": cfg["n_layers"],
                "plain_ms_per_step": round(plain_ms, 4), "graph_ms_per_step": round(graph_ms, 4),
                "tokens_per_s_plain": round(B / plain_ms * 1e3, 1), "tokens_per_s_graph": round(B / graph_ms * 1e3, 1),
                "weight_MB": round(by["weights"] / 1e6, 1), "kv_MB": round(by["kv"] / 1e6, 1),
                "GBps_graph": round((by["weights"] + by["kv"]) / graph_ms / 1e6, 1),
                "device_status": ctx.device_status(),
            })
    dec.close()
    return rows


def time_prompt(ctx, dev, cfg: dict, n_tokens: int, chunk: int = 1024, mode: str = "q8", reps: int = 3) -> dict:
    """Times ForwardLastLogits over a seeded random prompt of `n_tokens` (one sequence, chunks of `chunk` tokens)."""
    import torch

    w = device_weights(dev, cfg)
    dec = Decoder(ctx, cfg, w, max_batch=1)
    del w
    g = torch.Generator(device="cuda")
    g.manual_seed(7)
    tok = torch.randint(0, cfg["vocab"], (n_tokens,), generator=g, device="cuda", dtype=torch.int32)
    dec.forward_last_logits(tok, 0, 0, MODES[mode], chunk)  # grows the scratch, warms up
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        dec.forward_last_logits(tok, 0, 0, MODES[mode], chunk)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / reps
    row = {"prompt_tokens": n_tokens, "chunk": chunk, "mode": mode, "layers": cfg["n_layers"], "ms": round(ms, 3),
           "tokens_per_s": round(n_tokens / ms * 1e3, 1), "device_status": ctx.device_status()}
    dec.close()
    return row


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--prompt", type=int, default=0, help="time a prompt pass of this many tokens instead of decode steps")
    ap.add_argument("--chunk", type=int, default=1024)
    ap.add_argument("--batches", default="1,8,32")
    ap.add_argument("--ctx", type=int, default=2048)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--modes", default="q8,f32")
    ap.add_argument("--layers", type=int, default=0)
    ap.add_argument("--once", action="store_true")
    ap.add_argument("--model", default="qwen3", choices=("qwen3", "llama8b"),
                    help="qwen3 = Qwen3-0.6B shape, Q8_0; llama8b = Llama-3-8B shape, Q4_K / Q6_K down / Q8_0 head")
    a = ap.parse_args()
    cfg = dict(synth.QWEN3_0_6B if a.model == "qwen3" else synth.LLAMA3_8B)
    if a.layers:
        cfg["n_layers"] = a.layers
    ctx = ops.CudaContext(0)
    dev = ops.DeviceOps(ctx)
    if a.prompt:
        for name in a.modes.split(","):
            print(json.dumps(time_prompt(ctx, dev, cfg, a.prompt, a.chunk, name)), flush=True)
        ctx.close()
        return
    for row in time_decode(ctx, dev, cfg, [int(b) for b in a.batches.split(",")], a.ctx, a.steps,
                           tuple(a.modes.split(",")), a.once):
        print(json.dumps(row), flush=True)
    ctx.close()


if __name__ == "__main__":
    main()
