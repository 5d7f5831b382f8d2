"""ctypes front end of the CPU checkers in this directory.

TEST INFRASTRUCTURE ONLY.  The scalar restatement (`sm_oracle.c`), the AVX2/FMA port
(`sm_cpu_fma.c`) and, when it has been built, the reference's own C oracle
(`_ref/libvecdot_ref.so`, compiled from SharpMind's tools/ReferenceDataGenerator/vecdot_ref.c)
are loaded here for the test suite, the smoke check and the benchmark's CPU-baseline leg.
Nothing in the shipped package imports this module.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))

Q8_0, Q4_K, Q6_K = 8, 12, 14  # SharpMind.Core/Quantization/QuantDType.cs:2-18
BLOCK_ELEMS = {Q8_0: 32, Q4_K: 256, Q6_K: 256}
BLOCK_BYTES = {Q8_0: 34, Q4_K: 144, Q6_K: 210}
# dtype numbering private to the reference's C tool (vecdot_ref.c:24-38)
_REF_TOOL_FN = {Q8_0: "vecdot_q8_0", Q4_K: "vecdot_q4_K", Q6_K: "vecdot_q6_K"}

_f32p = C.POINTER(C.c_float)
_u8p = C.POINTER(C.c_uint8)
_i32p = C.POINTER(C.c_int32)


def build(reference_root: str | None = None) -> None:
    """Compile the checkers; also the reference's own C oracle when its tree is present."""
    subprocess.run(["make", "-s", "-C", HERE], check=True)
    if reference_root and os.path.isfile(
        os.path.join(reference_root, "tools", "ReferenceDataGenerator", "vecdot_ref.c")
    ):
        subprocess.run(["make", "-s", "-C", HERE, "ref", f"REF={reference_root}"], check=True)


def _load(name: str) -> C.CDLL:
    path = os.path.join(HERE, name)
    if not os.path.exists(path):
        build()
    return C.CDLL(path)


_lib = None
_fma = None
_ref = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        _lib = _load("libsm_oracle.so")
        L = _lib
        L.smo_half_to_float.restype = C.c_float
        L.smo_half_to_float.argtypes = [C.c_uint16]
        L.smo_float_to_half.restype = C.c_uint16
        L.smo_float_to_half.argtypes = [C.c_float]
        L.smo_float_to_half_trunc.restype = C.c_uint16
        L.smo_float_to_half_trunc.argtypes = [C.c_float]
        L.smo_raw_bytes.restype = C.c_int64
        L.smo_raw_bytes.argtypes = [C.c_int, C.c_int64, C.c_int64]
        L.smo_vecdot.restype = C.c_float
        L.smo_vecdot.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_int, C.c_int]
        L.smo_qmatmul.restype = C.c_int
        L.smo_qmatmul.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int]
        L.smo_qmatmul_cols.restype = C.c_int
        L.smo_qmatmul_cols.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int,
                                       C.c_int, C.c_int, C.c_int]
        for fn in ("smo_read_q8_0", "smo_read_q4_K", "smo_read_q6_K"):
            getattr(L, fn).restype = None
            getattr(L, fn).argtypes = [C.c_void_p, C.c_void_p, C.c_int64]
        L.smo_quantize.restype = C.c_int
        L.smo_quantize.argtypes = [C.c_int, C.c_void_p, C.c_int64, C.c_void_p]
        L.smo_quantize_row_q8_0.restype = None
        L.smo_quantize_row_q8_0.argtypes = [C.c_void_p, C.c_void_p, C.c_int]
        L.smo_block_isums.restype = C.c_int
        L.smo_block_isums.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_void_p]
        L.smo_scale_min_k4.restype = None
        L.smo_scale_min_k4.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p]
        L.smo_rmsnorm_param.restype = C.c_float
        L.smo_rmsnorm_param.argtypes = [C.c_void_p, C.c_int, C.c_float]
        L.smo_rmsnorm_row.restype = None
        L.smo_rmsnorm_row.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_float]
        L.smo_rmsnorm.restype = None
        L.smo_rmsnorm.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_float]
        L.smo_silu.restype = None
        L.smo_silu.argtypes = [C.c_void_p, C.c_void_p, C.c_int64]
        L.smo_swiglu.restype = None
        L.smo_swiglu.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64]
        L.smo_softmax_row.restype = None
        L.smo_softmax_row.argtypes = [C.c_void_p, C.c_void_p, C.c_int]
        L.smo_rope_tables.restype = None
        L.smo_rope_tables.argtypes = [C.c_float, C.c_int, C.c_int, C.c_void_p, C.c_void_p]
        L.smo_rope_apply.restype = None
        L.smo_rope_apply.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p,
                                     C.c_void_p, C.c_int]
        L.smo_add_inplace.restype = None
        L.smo_add_inplace.argtypes = [C.c_void_p, C.c_void_p, C.c_int64]
        L.smo_argmax.restype = C.c_int
        L.smo_argmax.argtypes = [C.c_void_p, C.c_int]
        L.smo_medusa_heads.restype = None
        L.smo_medusa_heads.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int]
        L.smo_verify_greedy.restype = C.c_int
        L.smo_verify_greedy.argtypes = [C.c_void_p, C.c_void_p, C.c_int]
        L.smo_sdpa_flash.restype = None
        L.smo_sdpa_flash.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int,
                                     C.c_float, C.c_int, C.c_int, C.c_int]
        L.smo_sdpa_flash_q8.restype = None
        L.smo_sdpa_flash_q8.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int,
                                        C.c_float, C.c_int, C.c_int, C.c_int]
        L.smo_sample.restype = C.c_int
        L.smo_sample.argtypes = [C.c_void_p, C.c_int, C.c_float, C.c_int, C.c_float, C.c_float, C.c_float]
        L.smo_sample_ex.restype = C.c_int
        L.smo_sample_ex.argtypes = [C.c_void_p, C.c_int, C.c_float, C.c_int, C.c_float, C.c_float, C.c_float, C.c_void_p]
        L.smo_repetition_penalty.restype = None
        L.smo_repetition_penalty.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_float]
        L.smo_decode_step.restype = C.c_int
        L.smo_decode_step.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_void_p,
                                      C.c_void_p]
        L.smo_decode_step_ex.restype = C.c_int
        L.smo_decode_step_ex.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_void_p,
                                         C.c_void_p, C.c_int]
    return _lib


def fma_lib() -> C.CDLL:
    global _fma
    if _fma is None:
        _fma = _load("libsm_cpu_fma.so")
        F = _fma
        for fn in ("smf_vecdot_q8_0", "smf_vecdot_q4_K", "smf_vecdot_q6_K"):
            getattr(F, fn).restype = C.c_float
            getattr(F, fn).argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int]
        F.smf_num_threads.restype = C.c_int
        F.smf_qmatmul_parallel.restype = C.c_int
        F.smf_qmatmul_parallel.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int,
                                           C.c_int]
        F.smf_swiglu.restype = None
        F.smf_swiglu.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int]
        F.smf_swiglu_rows.restype = None
        F.smf_swiglu_rows.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int]
        F.smf_softmax_row.restype = None
        F.smf_softmax_row.argtypes = [C.c_void_p, C.c_void_p, C.c_int]
        F.smf_rmsnorm.restype = None
        F.smf_rmsnorm.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_float]
        F.smf_add_inplace.restype = None
        F.smf_add_inplace.argtypes = [C.c_void_p, C.c_void_p, C.c_int64]
    return _fma


def ref_lib() -> C.CDLL | None:
    """The reference's own C oracle, or None when `_ref/` was never built."""
    global _ref
    if _ref is None:
        path = os.path.join(HERE, "_ref", "libvecdot_ref.so")
        if not os.path.exists(path):
            return None
        _ref = C.CDLL(path)
        for fn in _REF_TOOL_FN.values():
            getattr(_ref, fn).restype = C.c_float
            getattr(_ref, fn).argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int]
    return _ref


def _p(a: np.ndarray) -> C.c_void_p:
    return C.c_void_p(a.ctypes.data)


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def _u8(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.uint8)


# ------------------------------------------------------------------ scalars / sizes
def half_to_float(h: int) -> float:
    return float(lib().smo_half_to_float(h))


def half_bits_to_float_bits(h: int) -> int:
    return int(np.float32(lib().smo_half_to_float(h)).view(np.uint32))


def float_to_half(f: float) -> int:
    return int(lib().smo_float_to_half(C.c_float(f)))


def float_to_half_trunc(f: float) -> int:
    return int(lib().smo_float_to_half_trunc(C.c_float(f)))


def raw_bytes(dtype: int, n: int, k: int) -> int:
    return int(lib().smo_raw_bytes(dtype, n, k))


# ------------------------------------------------------------------ quantised path
def quantize(dtype: int, values) -> np.ndarray:
    v = _f32(values).ravel()
    be, bb = BLOCK_ELEMS[dtype], BLOCK_BYTES[dtype]
    if v.size % be:
        raise ValueError(f"length {v.size} is not a multiple of {be}")
    out = np.zeros(v.size // be * bb, dtype=np.uint8)
    rc = lib().smo_quantize(dtype, _p(v), v.size, _p(out))
    if rc:
        raise ValueError("quantize failed")
    return out


def dequantize(dtype: int, raw, n: int) -> np.ndarray:
    raw = _u8(raw)
    out = np.zeros(n, dtype=np.float32)
    fn = {Q8_0: "smo_read_q8_0", Q4_K: "smo_read_q4_K", Q6_K: "smo_read_q6_K"}[dtype]
    getattr(lib(), fn)(_p(raw), _p(out), n)
    return out


def vecdot(dtype: int, x, raw, col: int, k: int) -> float:
    x, raw = _f32(x), _u8(raw)
    return float(lib().smo_vecdot(dtype, _p(x), _p(raw), col, k))


def vecdot_fma(dtype: int, x, raw, col: int, k: int) -> float:
    x, raw = _f32(x), _u8(raw)
    fn = {Q8_0: "smf_vecdot_q8_0", Q4_K: "smf_vecdot_q4_K", Q6_K: "smf_vecdot_q6_K"}[dtype]
    return float(getattr(fma_lib(), fn)(_p(x), _p(raw), col, k))


def vecdot_ref(dtype: int, x, raw, col: int, k: int) -> float:
    """Calls the reference's own compiled C function."""
    r = ref_lib()
    if r is None:
        raise RuntimeError("oracle/_ref was not built")
    x, raw = _f32(x), _u8(raw)
    return float(getattr(r, _REF_TOOL_FN[dtype])(_p(x), _p(raw), col, k))


def qmatmul(dtype: int, x, raw, m: int, k: int, n: int, cols: tuple[int, int] | None = None) -> np.ndarray:
    x, raw = _f32(x).reshape(m, k), _u8(raw)
    out = np.zeros((m, n), dtype=np.float32)
    if cols is None:
        rc = lib().smo_qmatmul(dtype, _p(x), _p(raw), _p(out), m, k, n)
    else:
        rc = lib().smo_qmatmul_cols(dtype, _p(x), _p(raw), _p(out), m, k, n, cols[0], cols[1])
    if rc:
        raise ValueError("unsupported dtype")
    return out


def qmatmul_fma(dtype: int, x, raw, m: int, k: int, n: int) -> np.ndarray:
    x, raw = _f32(x).reshape(m, k), _u8(raw)
    out = np.zeros((m, n), dtype=np.float32)
    rc = fma_lib().smf_qmatmul_parallel(dtype, _p(x), _p(raw), _p(out), m, k, n)
    if rc:
        raise ValueError("unsupported dtype")
    return out


def quantize_rows_q8_0(x, m: int, k: int) -> np.ndarray:
    """Run-time activation quantiser: [m, k] fp32 -> [m, ceil(k/32)*34] bytes."""
    x = _f32(x).reshape(m, k)
    nb = (k + 31) // 32
    out = np.zeros((m, nb * 34), dtype=np.uint8)
    for r in range(m):
        lib().smo_quantize_row_q8_0(_p(x[r]), C.c_void_p(out[r].ctypes.data), k)
    return out


def split_q8_rows(xq: np.ndarray) -> tuple[np.ndarray, np.ndarray]:
    """[m, nb*34] bytes -> (int8 [m, nb*32], fp16-bit scales uint16 [m, nb])."""
    m = xq.shape[0]
    blocks = xq.reshape(m, -1, 34)
    d = blocks[:, :, :2].copy().view(np.uint16).reshape(m, -1)
    q = blocks[:, :, 2:].copy().view(np.int8).reshape(m, -1)
    return q, d


def block_isums(dtype: int, raw, xq_row, col: int, k: int) -> np.ndarray:
    raw, xq_row = _u8(raw), _u8(xq_row)
    out = np.zeros(k // 32, dtype=np.int32)
    rc = lib().smo_block_isums(dtype, _p(raw), _p(xq_row), col, k, _p(out))
    if rc:
        raise ValueError("unsupported shape")
    return out


def scale_min_k4(sc12) -> tuple[np.ndarray, np.ndarray]:
    sc12 = _u8(sc12)
    s = np.zeros(8, dtype=np.int32)
    m = np.zeros(8, dtype=np.int32)
    lib().smo_scale_min_k4(_p(sc12), _p(s), _p(m))
    return s, m


# ------------------------------------------------------------------ fp32 ops
def rmsnorm_param(row, eps: float) -> float:
    row = _f32(row)
    return float(lib().smo_rmsnorm_param(_p(row), row.size, C.c_float(eps)))


def rmsnorm(x, w, eps: float) -> np.ndarray:
    x, w = _f32(x), _f32(w)
    n = x.shape[-1]
    out = np.empty_like(x)
    lib().smo_rmsnorm(_p(x), _p(w), _p(out), x.size // n, n, C.c_float(eps))
    return out


def rmsnorm_row(src, w, rms_inv: float) -> np.ndarray:
    src, w = _f32(src), _f32(w)
    out = np.empty_like(src)
    lib().smo_rmsnorm_row(_p(src), _p(w), _p(out), src.size, C.c_float(rms_inv))
    return out


def silu(x) -> np.ndarray:
    x = _f32(x)
    out = np.empty_like(x)
    lib().smo_silu(_p(x), _p(out), x.size)
    return out


def swiglu(gate, up) -> np.ndarray:
    gate, up = _f32(gate), _f32(up)
    out = np.empty_like(gate)
    lib().smo_swiglu(_p(gate), _p(up), _p(out), gate.size)
    return out


def softmax_rows(x) -> np.ndarray:
    x = _f32(x)
    n = x.shape[-1]
    x2 = x.reshape(-1, n)
    out = np.empty_like(x2)
    for r in range(x2.shape[0]):
        lib().smo_softmax_row(C.c_void_p(x2[r].ctypes.data), C.c_void_p(out[r].ctypes.data), n)
    return out.reshape(x.shape)


def rope_tables(theta: float, rope_dim: int, max_seq: int) -> tuple[np.ndarray, np.ndarray]:
    cos = np.zeros((max_seq, rope_dim // 2), dtype=np.float32)
    sin = np.zeros_like(cos)
    lib().smo_rope_tables(C.c_float(theta), rope_dim, max_seq, _p(cos), _p(sin))
    return cos, sin


def rope_apply(x, pos_offset: int, cos, sin, neox: bool, rope_dim: int | None = None) -> np.ndarray:
    """x [seq, heads, head_dim]; returns the rotated copy."""
    x = _f32(x).copy()
    seq, heads, hd = x.shape
    lib().smo_rope_apply(_p(x), seq, heads, hd, rope_dim or hd, pos_offset, _p(_f32(cos)), _p(_f32(sin)),
                         1 if neox else 0)
    return x


def add(x, y) -> np.ndarray:
    x = _f32(x).copy()
    y = _f32(y)
    lib().smo_add_inplace(_p(x), _p(y), x.size)
    return x


def argmax(logits) -> int:
    logits = _f32(logits)
    return int(lib().smo_argmax(_p(logits), logits.size))


def medusa_heads(hidden, w, b) -> np.ndarray:
    """MedusaHeads.PredictQuantized's head transform: hidden [H], w [k, H, H], b [k, H] -> SiLU(b + hidden W) [k, H]."""
    hidden, w, b = _f32(hidden), _f32(w), _f32(b)
    k, H = b.shape
    out = np.empty((k, H), dtype=np.float32)
    lib().smo_medusa_heads(_p(hidden), _p(w), _p(b), _p(out), k, H)
    return out


def medusa_predict(hidden, w, b, lm_head_raw, vocab: int) -> tuple[np.ndarray, np.ndarray]:
    """MedusaHeads.Predict on a Q8_0 LM head: the tokens the k heads pick and their logits [k, vocab]."""
    h = medusa_heads(hidden, w, b)
    k, H = h.shape
    logits = qmatmul(8, h, lm_head_raw, k, H, vocab)
    return np.array([argmax(logits[i]) for i in range(k)], dtype=np.int32), logits


def verify_greedy(argmax_rows, draft) -> int:
    a = np.ascontiguousarray(argmax_rows, dtype=np.int32)
    d = np.ascontiguousarray(draft, dtype=np.int32)
    return int(lib().smo_verify_greedy(_p(a), _p(d), d.size - 1))


def sdpa_flash_q8(q, k_rows, v_rows, scale: float, causal: bool = True) -> np.ndarray:
    """ScaledDotProductFlashQ8_0Scalar for one head: q [seqLen, headDim] fp32, k_rows / v_rows [kvLen, headDim/32 * 34]
    uint8 (Q8_0 blocks as QuantizedKVCache stores them)."""
    q = _f32(q)
    seq, hd = q.shape
    k, v = _u8(k_rows), _u8(v_rows)
    out = np.zeros_like(q)
    lib().smo_sdpa_flash_q8(_p(q), _p(k), _p(v), _p(out), seq, k.shape[0], hd, scale, int(causal), hd, hd)
    return out


def sample(logits, temperature: float, top_k: int, top_p: float, min_p: float, r: float) -> int:
    """Sampler.Sample on one row of logits with the uniform draw `r` supplied by the caller."""
    x = _f32(logits)
    return int(lib().smo_sample(_p(x), x.size, temperature, top_k, top_p, min_p, r))


def sample_probs(logits, temperature: float, top_k: int, top_p: float, min_p: float, r: float):
    """(token, probabilities the draw was made from) of Sampler.Sample; temperature must be > 0."""
    x = _f32(logits)
    probs = np.zeros(x.size, np.float32)
    tok = int(lib().smo_sample_ex(_p(x), x.size, temperature, top_k, top_p, min_p, r, _p(probs)))
    return tok, probs


def repetition_penalty(logits, ids, penalty: float) -> np.ndarray:
    """RepetitionPenalty.Apply on a copy of one row of logits."""
    x = _f32(logits).copy()
    i = np.ascontiguousarray(ids, dtype=np.int32)
    lib().smo_repetition_penalty(_p(x), x.size, _p(i), i.size, penalty)
    return x


def sdpa_flash(q, k, v, scale: float, causal: bool = True) -> np.ndarray:
    """q [seq, head_dim] (contiguous rows), k/v [kv, head_dim]."""
    q, k, v = _f32(q), _f32(k), _f32(v)
    seq, hd = q.shape
    out = np.zeros_like(q)
    lib().smo_sdpa_flash(_p(q), _p(k), _p(v), _p(out), seq, k.shape[0], hd, C.c_float(scale),
                         1 if causal else 0, hd, hd)
    return out


# ------------------------------------------------------------------ decoder
class _Model(C.Structure):
    _fields_ = [
        ("n_layers", C.c_int), ("hidden", C.c_int), ("n_heads", C.c_int), ("n_kv_heads", C.c_int),
        ("head_dim", C.c_int), ("ffn", C.c_int), ("vocab", C.c_int), ("max_seq", C.c_int),
        ("dtype", C.c_int), ("eps", C.c_float), ("rope_theta", C.c_float), ("neox", C.c_int),
        ("qk_norm", C.c_int),
        ("wq", C.POINTER(C.c_void_p)), ("wk", C.POINTER(C.c_void_p)), ("wv", C.POINTER(C.c_void_p)),
        ("wo", C.POINTER(C.c_void_p)), ("wgu", C.POINTER(C.c_void_p)), ("wdown", C.POINTER(C.c_void_p)),
        ("norm1", C.POINTER(C.c_void_p)), ("norm2", C.POINTER(C.c_void_p)),
        ("qnorm", C.POINTER(C.c_void_p)), ("knorm", C.POINTER(C.c_void_p)),
        ("final_norm", C.c_void_p), ("lm_head", C.c_void_p), ("embedding", C.c_void_p),
        ("cosT", C.c_void_p), ("sinT", C.c_void_p),
        ("down_dtype", C.c_int), ("head_dtype", C.c_int),
        ("bq", C.POINTER(C.c_void_p)), ("bk", C.POINTER(C.c_void_p)), ("bv", C.POINTER(C.c_void_p)),
        ("bo", C.POINTER(C.c_void_p)), ("bgu", C.POINTER(C.c_void_p)), ("bdown", C.POINTER(C.c_void_p)),
        ("kv_q8", C.c_int),
    ]


class Decoder:
    """Oracle decoder over host weights.

    `weights` is the dict produced by `sharpmind_b200.synth.make_decoder_weights`: per-layer raw
    byte arrays wq/wk/wv/wo/wgu/wdown, fp32 norm vectors, the raw embedding (also the tied LM head).
    """

    def __init__(self, cfg: dict, weights: dict, batch: int):
        self.cfg = cfg
        self.w = weights
        L = cfg["n_layers"]
        self.batch = batch
        hd, nkv, ms = cfg["head_dim"], cfg["n_kv_heads"], cfg["max_seq"]
        self.kcache = np.zeros((L, batch, nkv, ms, hd), dtype=np.float32)
        self.vcache = np.zeros_like(self.kcache)
        self.cos, self.sin = rope_tables(cfg["rope_theta"], hd, ms)
        head_dt = cfg.get("head_dtype", cfg["dtype"])
        self.embedding = dequantize(head_dt, weights["embedding"], cfg["vocab"] * cfg["hidden"])
        self._keep = []

        def arr(name):
            a = (C.c_void_p * L)(*[weights[name][i].ctypes.data for i in range(L)])
            self._keep.append(a)
            return C.cast(a, C.POINTER(C.c_void_p))

        m = _Model()
        m.n_layers, m.hidden, m.n_heads, m.n_kv_heads = L, cfg["hidden"], cfg["n_heads"], nkv
        m.head_dim, m.ffn, m.vocab, m.max_seq = hd, cfg["ffn"], cfg["vocab"], ms
        m.dtype, m.eps, m.rope_theta = cfg["dtype"], cfg["eps"], cfg["rope_theta"]
        m.neox, m.qk_norm = int(cfg["neox"]), int(cfg["qk_norm"])
        m.down_dtype, m.head_dtype = cfg.get("down_dtype", 0), cfg.get("head_dtype", 0)
        m.wq, m.wk, m.wv, m.wo = arr("wq"), arr("wk"), arr("wv"), arr("wo")
        m.wgu, m.wdown = arr("wgu"), arr("wdown")
        m.norm1, m.norm2 = arr("norm1"), arr("norm2")
        m.qnorm, m.knorm = arr("qnorm"), arr("knorm")
        for name in ("bq", "bk", "bv", "bo", "bgu", "bdown"):  # optional bias vectors (entries may be None)
            if weights.get(name) is None:
                continue
            a = (C.c_void_p * L)(*[None if b is None else b.ctypes.data for b in weights[name]])
            self._keep.append(a)
            setattr(m, name, C.cast(a, C.POINTER(C.c_void_p)))
        m.kv_q8 = 1 if cfg.get("kv_dtype", 0) == 8 else 0  # QuantizedKVCache with Q8_0 rows
        m.final_norm = weights["final_norm"].ctypes.data
        m.lm_head = weights["embedding"].ctypes.data
        m.embedding = self.embedding.ctypes.data
        m.cosT, m.sinT = self.cos.ctypes.data, self.sin.ctypes.data
        self._m = m

    def step(self, tokens, pos: int, act_q8: bool = False) -> np.ndarray:
        """One decode step.  act_q8: every matmul input is quantised to Q8_0 and dequantised first (the arithmetic
        the CUDA library's SMC_ACT_Q8 mode is specified to have)."""
        tok = np.ascontiguousarray(tokens, dtype=np.int32)
        logits = np.zeros((self.batch, self.cfg["vocab"]), dtype=np.float32)
        rc = lib().smo_decode_step_ex(C.byref(self._m), _p(tok), self.batch, pos, _p(self.kcache),
                                      _p(self.vcache), _p(logits), int(act_q8))
        if rc:
            raise RuntimeError(f"oracle decode_step failed: {rc}")
        return logits
