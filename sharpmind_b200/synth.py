"""Seeded synthetic tensors for the benchmark configurations.

Every tensor is drawn from a counter-based generator (Philox) keyed by a stable hash of
(config name, tensor name), so the same bytes feed the CUDA path and any checker on any host.
No dataset or checkpoint is involved: the reference's headline configurations only name shapes
and distributions (weights N(0, 0.02) before quantisation, activations N(0, 1)).
"""
from __future__ import annotations

import hashlib

import numpy as np


def _key(config: str, name: str) -> int:
    h = hashlib.sha256(f"{config}/{name}".encode()).digest()
    return int.from_bytes(h[:8], "little")


def rng(config: str, name: str) -> np.random.Generator:
    return np.random.Generator(np.random.Philox(key=_key(config, name)))


def normal(config: str, name: str, shape, sigma: float = 1.0, mean: float = 0.0) -> np.ndarray:
    g = rng(config, name)
    out = g.standard_normal(size=shape, dtype=np.float32)
    if sigma != 1.0:
        out *= np.float32(sigma)
    if mean != 0.0:
        out += np.float32(mean)
    return out


def uniform(config: str, name: str, shape, lo: float = -1.0, hi: float = 1.0) -> np.ndarray:
    g = rng(config, name)
    return (g.random(size=shape, dtype=np.float32) * np.float32(hi - lo) + np.float32(lo)).astype(np.float32)


def token_ids(config: str, name: str, shape, vocab: int) -> np.ndarray:
    return rng(config, name).integers(0, vocab, size=shape, dtype=np.int32)


# Qwen3-0.6B-shaped decoder of the full-decode configuration.  rope_theta is not given by the
# configuration text; 1e6 (the value Qwen3 checkpoints carry) is used and recorded here.
QWEN3_0_6B = dict(
    n_layers=28, hidden=1024, n_heads=16, n_kv_heads=8, head_dim=128, ffn=3072, vocab=151936,
    max_seq=2304, dtype=8, eps=1e-6, rope_theta=1.0e6, neox=True, qk_norm=True,
)


# Llama-3-8B shape with the formats a Q4_K_M-style GGUF file mixes: Q4_K attention and gate||up, Q6_K down;
# the embedding / tied LM head is Q8_0 (the decoder's embedding gather reads Q8_0 rows).
LLAMA3_8B = dict(
    n_layers=32, hidden=4096, n_heads=32, n_kv_heads=8, head_dim=128, ffn=14336, vocab=128256,
    max_seq=2304, dtype=12, down_dtype=14, head_dtype=8, eps=1e-5, rope_theta=5.0e5, neox=False, qk_norm=False,
)


def make_decoder_weights(cfg: dict, config_name: str, quantize) -> dict:
    """Random-init weights of a decoder shaped by `cfg`.

    `quantize(dtype, fp32_values) -> uint8 array` turns N(0, 0.02) matrices into GGUF blocks; the
    caller chooses which quantiser (the CUDA one in the product, a CPU checker in tests).
    Layout per layer follows the reference's linear layers: wq [nH*hd, H], wk/wv [nKV*hd, H],
    wo [H, nH*hd], wgu = gate rows followed by up rows [2F, H], wdown [H, F]; the embedding
    [vocab, H] doubles as the tied LM head.  cfg["dtype"] is the format of every matrix unless
    cfg["down_dtype"] / cfg["head_dtype"] name another one for the down projection / the embedding.
    """
    L, H, hd = cfg["n_layers"], cfg["hidden"], cfg["head_dim"]
    q_dim, kv_dim, F, V = cfg["n_heads"] * hd, cfg["n_kv_heads"] * hd, cfg["ffn"], cfg["vocab"]
    dt = cfg["dtype"]

    def mat(name, n, k, fmt=None):
        return quantize(fmt or dt, normal(config_name, name, (n, k), 0.02))

    w = {k: [] for k in ("wq", "wk", "wv", "wo", "wgu", "wdown", "norm1", "norm2", "qnorm", "knorm")}
    for i in range(L):
        w["wq"].append(mat(f"l{i}.wq", q_dim, H))
        w["wk"].append(mat(f"l{i}.wk", kv_dim, H))
        w["wv"].append(mat(f"l{i}.wv", kv_dim, H))
        w["wo"].append(mat(f"l{i}.wo", H, q_dim))
        w["wgu"].append(mat(f"l{i}.wgu", 2 * F, H))
        w["wdown"].append(mat(f"l{i}.wdown", H, F, cfg.get("down_dtype")))
        w["norm1"].append(normal(config_name, f"l{i}.norm1", (H,), 0.1, 1.0))
        w["norm2"].append(normal(config_name, f"l{i}.norm2", (H,), 0.1, 1.0))
        w["qnorm"].append(normal(config_name, f"l{i}.qnorm", (hd,), 0.1, 1.0))
        w["knorm"].append(normal(config_name, f"l{i}.knorm", (hd,), 0.1, 1.0))
    w["final_norm"] = normal(config_name, "final_norm", (H,), 0.1, 1.0)
    w["embedding"] = mat("embedding", V, H, cfg.get("head_dtype"))
    return w
