"""GGUF file -> device weights -> decode: a file written by the test with the tensor names llama.cpp uses is loaded
through the library's memory-mapped reader, every matrix registered straight from the mapping, and the decoder built
from it is compared with the oracle decoder fed the very bytes that were written."""
import numpy as np
import pytest

from sharpmind_b200 import gguf, ops, synth
from tests.gguf_writer import write_gguf
from tests.gpu_util import to_dev

pytestmark = pytest.mark.gpu

CFG = dict(n_layers=2, hidden=256, n_heads=4, n_kv_heads=2, head_dim=128, ffn=512, vocab=512, max_seq=32, dtype=12,
           down_dtype=14, head_dtype=8, eps=1e-6, rope_theta=1.0e6, neox=True, qk_norm=True)


def _file(oracle, tmp_path, f16_norms: bool):
    cfg = CFG
    w = synth.make_decoder_weights(cfg, "gguf_dec", oracle.quantize)
    H, hd, F = cfg["hidden"], cfg["head_dim"], cfg["ffn"]
    q_dim, kv_dim = cfg["n_heads"] * hd, cfg["n_kv_heads"] * hd
    tensors = [("token_embd.weight", 8, [H, cfg["vocab"]], w["embedding"])]

    def vec(name, a):
        if f16_norms:  # norm vectors stored as F16: the oracle gets the rounded values
            h = a.astype(np.float16)
            a[:] = h.astype(np.float32)
            tensors.append((name, 1, [a.size], h))
        else:
            tensors.append((name, 0, [a.size], a))

    per_row = len(w["wgu"][0]) // (2 * F)
    for i in range(cfg["n_layers"]):
        b = f"blk.{i}."
        tensors += [(b + "attn_q.weight", 12, [H, q_dim], w["wq"][i]), (b + "attn_k.weight", 12, [H, kv_dim], w["wk"][i]),
                    (b + "attn_v.weight", 12, [H, kv_dim], w["wv"][i]), (b + "attn_output.weight", 12, [q_dim, H], w["wo"][i]),
                    (b + "ffn_gate.weight", 12, [H, F], w["wgu"][i][:F * per_row]),
                    (b + "ffn_up.weight", 12, [H, F], w["wgu"][i][F * per_row:]),
                    (b + "ffn_down.weight", 14, [F, H], w["wdown"][i])]
        vec(b + "attn_norm.weight", w["norm1"][i]), vec(b + "ffn_norm.weight", w["norm2"][i])
        vec(b + "attn_q_norm.weight", w["qnorm"][i]), vec(b + "attn_k_norm.weight", w["knorm"][i])
    vec("output_norm.weight", w["final_norm"])
    meta = {"general.architecture": "qwen3", "general.name": "synthetic", "qwen3.block_count": cfg["n_layers"],
            "qwen3.embedding_length": H, "qwen3.attention.head_count": cfg["n_heads"],
            "qwen3.attention.head_count_kv": cfg["n_kv_heads"], "qwen3.attention.key_length": hd,
            "qwen3.feed_forward_length": F, "qwen3.attention.layer_norm_rms_epsilon": float(cfg["eps"]),
            "qwen3.rope.freq_base": float(cfg["rope_theta"])}
    path = str(tmp_path / "model.gguf")
    write_gguf(path, meta, tensors)
    return path, w


@pytest.mark.parametrize("f16_norms", [False, True])
def test_gguf_to_device_decoder_matches_oracle(oracle, cuda, tmp_path, f16_norms):
    path, w = _file(oracle, tmp_path, f16_norms)
    dec, cfg = gguf.load_decoder(cuda, path, max_seq=CFG["max_seq"], max_batch=2)
    for k in ("n_layers", "hidden", "n_heads", "n_kv_heads", "head_dim", "ffn", "vocab", "dtype", "down_dtype", "head_dtype",
              "neox", "qk_norm"):
        assert cfg[k] == CFG[k], k
    assert abs(cfg["rope_theta"] - CFG["rope_theta"]) < 1 and abs(cfg["eps"] - CFG["eps"]) < 1e-12
    ref = oracle.Decoder(CFG, w, 2)
    tok = synth.token_ids("gguf_dec", "prompt", (2,), CFG["vocab"])
    for pos in range(5):
        want = ref.step(tok, pos)
        logits, nxt = dec.step(to_dev(tok), pos, ops.Mode.ACT_F32)
        got = logits.cpu().numpy()
        assert np.abs(got - want).max() <= 1e-4 * np.abs(want).max()
        tok = want.argmax(axis=1).astype(np.int32)
        assert np.array_equal(nxt.cpu().numpy(), tok)
    dec.close()


def test_gguf_reader_reports_and_refuses(oracle, cuda, tmp_path):
    path, _ = _file(oracle, tmp_path, False)
    f = gguf.GgufFile(cuda, path)
    assert f.meta_string("general.architecture") == "qwen3" and f.meta_int("qwen3.block_count") == 2
    assert f.meta_int("no.such.key") is None
    t = f.tensors["blk.1.ffn_down.weight"]
    assert t["dtype"] == 14 and t["dims"] == [512, 256] and t["bytes"] == 256 * 512 // 256 * 210
    with pytest.raises(ops.NotSupportedException):
        f.register("output_norm.weight")          # an F32 vector is not a quantized matrix
    with pytest.raises(ops.SharpMindCudaError):
        f.read_f32("blk.0.attn_q.weight")         # and a Q4_K matrix is not read as floats
    f.close()
    bad = tmp_path / "bad.gguf"
    bad.write_bytes(b"GGML" + b"\0" * 64)
    with pytest.raises(ops.SharpMindCudaError):
        gguf.GgufFile(cuda, str(bad))
    # a file cut short inside a tensor is refused at open (the reference's loader would read past its stream)
    whole = open(path, "rb").read()
    cut = tmp_path / "cut.gguf"
    cut.write_bytes(whole[:len(whole) - 4096])
    with pytest.raises(ops.InvalidOperationException):
        gguf.GgufFile(cuda, str(cut))
