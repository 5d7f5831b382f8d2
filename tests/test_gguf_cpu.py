"""The GGUF header parser needs no device: files written by the test are opened through the C ABI with a null context."""
import ctypes as C

import numpy as np

from sharpmind_b200 import _lib
from tests.gguf_writer import write_gguf


def _open(lib, path):
    h = C.c_void_p()
    return lib.smc_gguf_open(None, str(path).encode(), C.byref(h)), h


def test_gguf_header_tensor_infos_and_metadata(tmp_path):
    lib = _lib.load()
    tensors = [("token_embd.weight", 8, [256, 512], np.zeros(512 * 8 * 34, np.uint8)),
               ("blk.0.attn_norm.weight", 0, [256], np.arange(256, dtype=np.float32)),
               ("blk.0.ffn_norm.weight", 1, [256], np.arange(256).astype(np.float16)),
               ("blk.0.ffn_down.weight", 14, [512, 256], np.zeros(256 * 2 * 210, np.uint8)),
               ("blk.0.exotic.weight", 30, [64], np.zeros(64, np.uint8))]
    path = tmp_path / "m.gguf"
    write_gguf(path, {"general.architecture": "qwen3", "qwen3.block_count": 28, "qwen3.rope.freq_base": 1e6,
                      "general.file_size": 2 ** 33}, tensors, alignment=64)
    rc, h = _open(lib, path)
    assert rc == 0 and lib.smc_gguf_tensor_count(h) == 5
    want = {"token_embd.weight": (8, [256, 512], 139264), "blk.0.attn_norm.weight": (0, [256], 1024),
            "blk.0.ffn_norm.weight": (1, [256], 512), "blk.0.ffn_down.weight": (14, [512, 256], 107520),
            "blk.0.exotic.weight": (30, [64], -1)}
    for name, (dt, dims, nbytes) in want.items():
        i = lib.smc_gguf_find(h, name.encode())
        assert i >= 0
        n, d, nd, nb = C.c_char_p(), C.c_int(), C.c_int(), C.c_int64()
        dm = (C.c_int64 * 4)()
        assert lib.smc_gguf_tensor_info(h, i, C.byref(n), C.byref(d), C.byref(nd), dm, C.byref(nb)) == 0
        assert (n.value.decode(), d.value, list(dm)[:nd.value], nb.value) == (name, dt, dims, nbytes)
    assert lib.smc_gguf_find(h, b"no.such.tensor") == -1
    v, f = C.c_int64(), C.c_double()
    assert lib.smc_gguf_meta_int(h, b"qwen3.block_count", C.byref(v)) == 0 and v.value == 28
    assert lib.smc_gguf_meta_int(h, b"general.file_size", C.byref(v)) == 0 and v.value == 2 ** 33
    assert lib.smc_gguf_meta_float(h, b"qwen3.rope.freq_base", C.byref(f)) == 0 and f.value == 1e6
    assert lib.smc_gguf_meta_int(h, b"general.alignment", C.byref(v)) == 0 and v.value == 64
    assert lib.smc_gguf_meta_string(h, b"general.architecture") == b"qwen3"
    assert lib.smc_gguf_meta_int(h, b"absent", C.byref(v)) != 0 and lib.smc_gguf_meta_string(h, b"absent") is None
    assert lib.smc_gguf_close(None, h) == 0


def test_gguf_refuses_foreign_and_truncated_files(tmp_path):
    lib = _lib.load()
    bad = tmp_path / "bad.gguf"
    bad.write_bytes(b"GGML" + b"\0" * 64)
    assert _open(lib, bad)[0] != 0
    assert _open(lib, tmp_path / "missing.gguf")[0] != 0
    path = tmp_path / "m.gguf"
    write_gguf(path, {"general.architecture": "llama"}, [("a", 0, [1024], np.ones(1024, np.float32)),
                                                          ("b", 0, [1024], np.ones(1024, np.float32))])
    whole = path.read_bytes()
    for cut in (len(whole) - 100, 40, 12):  # inside the last tensor, inside the header, inside the counts
        part = tmp_path / f"cut{cut}.gguf"
        part.write_bytes(whole[:cut])
        assert _open(lib, part)[0] != 0, cut
