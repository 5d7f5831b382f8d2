"""Host-side mirror of the reference's operator interface for the quantized hot path.

Two layers, both thin wrappers over the C ABI (no compute happens in Python):

* `QuantizationOps` / `ActivationOps` keep the reference's slot names and argument order
  (SharpMind.Core/Quantization/QuantizationOps.cs:8-9,176-235; SharpMind.Core/Activations/
  ActivationOps.cs:36-160): host arrays in, host arrays out, one synchronous call per op.
* `DeviceOps` works on CUDA tensors (torch is used only as the owner of device memory and
  streams) and is what the decoder, the benchmark and the sharded runner call.

Error behaviour follows the reference: a byte-count mismatch raises InvalidOperationException
(InferenceLinearLayer.cs:162-171), headDim > 256 and out-of-range indices raise
ArgumentOutOfRangeException (AttentionKernels.cs:225-227), unsupported dtype/shape combinations raise
NotSupportedException.
"""
from __future__ import annotations

import ctypes as C
from enum import IntEnum

import numpy as np

from . import _lib


class SharpMindCudaError(RuntimeError):
    pass


class InvalidOperationException(SharpMindCudaError):
    pass


class ArgumentOutOfRangeException(SharpMindCudaError, ValueError):
    pass


class NotSupportedException(SharpMindCudaError):
    pass


class ArgumentException(SharpMindCudaError, ValueError):
    pass


class QuantDType(IntEnum):  # SharpMind.Core/Quantization/QuantDType.cs:2-18
    Q8_0 = 8
    Q4_K = 12
    Q6_K = 14


class Mode(IntEnum):
    ACT_F32 = 0
    ACT_Q8 = 1
    REF_ORDER = 2


W_REPACK, W_KEEP_RAW = 1, 2
_STATUS_EXC = {
    1: ArgumentException, 2: NotSupportedException, 3: InvalidOperationException, 4: SharpMindCudaError,
    5: InvalidOperationException, 6: SharpMindCudaError, 7: ArgumentOutOfRangeException,
}


def raw_tensor_bytes(dtype: int, n: int, k: int) -> int:
    """QuantizationOps.GetRawTensorByteCount for a [n, k] tensor."""
    r = _lib.load().smc_raw_tensor_bytes(int(dtype), n, k)
    if r < 0:
        raise ArgumentOutOfRangeException(f"dtype {dtype}")
    return int(r)


class Weight:
    """A registered weight tensor: device copy owned by the library, host bytes kept alive here."""

    def __init__(self, handle, dtype, n, k, host=None):
        self.handle, self.dtype, self.N, self.K, self.host = handle, int(dtype), n, k, host

    @property
    def raw_bytes(self) -> int:
        return raw_tensor_bytes(self.dtype, self.N, self.K)


class CudaContext:
    def __init__(self, device: int = 0):
        self.lib = _lib.load()
        h = C.c_void_p()
        rc = self.lib.smc_init(device, C.byref(h))
        if rc:
            raise SharpMindCudaError(f"smc_init(device={device}) failed with status {rc}: no usable CUDA device")
        self.h = h
        self.device = device
        self._weights = []

    def close(self):
        if getattr(self, "h", None):
            self.lib.smc_destroy(self.h)
            self.h = None

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()

    def check(self, rc: int):
        if rc:
            msg = self.lib.smc_last_error(self.h).decode(errors="replace")
            raise _STATUS_EXC.get(rc, SharpMindCudaError)(msg or f"status {rc}")

    def synchronize(self):
        self.check(self.lib.smc_synchronize(self.h))

    def host_register(self, a: np.ndarray):
        """Page-locks a host array in place (smc_host_register): the host slots then copy from / to it directly."""
        self.check(self.lib.smc_host_register(self.h, a.ctypes.data, a.nbytes))

    def host_unregister(self, a: np.ndarray):
        self.check(self.lib.smc_host_unregister(self.h, a.ctypes.data))

    def set_option(self, name: str, value: int):
        """smc_set_option: per-context tuning and kernel-selection switches (the names and their meaning are listed
        with the entry point in the C header); none of them changes a result beyond its mode's bound."""
        self.check(self.lib.smc_set_option(self.h, name.encode(), int(value)))

    def device_status(self) -> int:
        """Waits for the device; raises if a kernel abandoned a bounded wait since the last call."""
        st = C.c_int(0)
        self.check(self.lib.smc_device_status(self.h, C.byref(st)))
        return st.value

    # ---- weights
    def register(self, raw: np.ndarray, dtype: int, n: int, k: int, repack: bool = True,
                 keep_raw: bool = True) -> Weight:
        raw = np.ascontiguousarray(raw, dtype=np.uint8)
        flags = (W_REPACK if repack else 0) | (W_KEEP_RAW if keep_raw else 0)
        h = C.c_void_p()
        self.check(self.lib.smc_weight_register(self.h, raw.ctypes.data, raw.size, int(dtype), n, k, flags, C.byref(h)))
        w = Weight(h, dtype, n, k, raw)
        self._weights.append(w)
        return w

    def register_dev(self, raw, dtype: int, n: int, k: int, repack: bool = True, keep_raw: bool = False) -> Weight:
        """`raw`: CUDA uint8 tensor holding the GGUF-layout bytes (copied by the library)."""
        flags = (W_REPACK if repack else 0) | (W_KEEP_RAW if keep_raw else 0)
        h = C.c_void_p()
        self.check(self.lib.smc_weight_register_dev(self.h, raw.data_ptr(), raw.numel(), int(dtype), n, k, flags,
                                                    C.byref(h)))
        return Weight(h, dtype, n, k, None)

    def lookup(self, raw: np.ndarray) -> C.c_void_p:
        h = C.c_void_p()
        self.check(self.lib.smc_weight_lookup(self.h, raw.ctypes.data, C.byref(h)))
        return h

    def release(self, w: Weight):
        self.check(self.lib.smc_weight_release(self.h, w.handle))
        w.handle = None
        if w in self._weights:
            self._weights.remove(w)


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


class QuantizationOps:
    """The `vecdot_*`, `qmatmul_*`, `linear` and `logit` slots on host pointers.

    `rawWeights` must be the numpy array that was passed to `CudaContext.register` (the library finds
    the device copy by its host address, as a backend that only receives `byte* rawWeights` must).
    """

    def __init__(self, ctx: CudaContext, mode: int = Mode.ACT_F32):
        self.ctx, self.mode = ctx, int(mode)

    GetRawTensorByteCount = staticmethod(lambda shape, dtype: raw_tensor_bytes(dtype, int(np.prod(shape[:-1])), shape[-1]))

    def _vecdot(self, dtype, input, rawWeights, col, inFeatures) -> float:
        x = _f32(input)
        out = C.c_float()
        self.ctx.check(self.ctx.lib.smc_vecdot_host(self.ctx.h, x.ctypes.data, rawWeights.ctypes.data, col,
                                                    inFeatures, int(dtype), C.byref(out)))
        return float(out.value)

    def VecDotQ8_0(self, input, rawWeights, col, inFeatures):
        return self._vecdot(QuantDType.Q8_0, input, rawWeights, col, inFeatures)

    def VecDotQ4K(self, input, rawWeights, col, inFeatures):
        return self._vecdot(QuantDType.Q4_K, input, rawWeights, col, inFeatures)

    def VecDotQ6K(self, input, rawWeights, col, inFeatures):
        return self._vecdot(QuantDType.Q6_K, input, rawWeights, col, inFeatures)

    def QuantizedMatMulFn(self, dtype, input, rawWeights, output, M, K, N, mode=None):
        """QuantizedMatMulFn(input, rawWeights, output, M, K, N); writes `output` in place."""
        x = _f32(input)
        if x.size != M * K:
            raise ArgumentException(f"input holds {x.size} values, expected M*K = {M * K}")
        if not (isinstance(output, np.ndarray) and output.dtype == np.float32 and output.flags.c_contiguous
                and output.size == M * N):
            raise ArgumentException("output must be a C-contiguous float32 array of M*N values")
        self.ctx.check(self.ctx.lib.smc_qmatmul_host(self.ctx.h, x.ctypes.data, rawWeights.ctypes.data,
                                                     output.ctypes.data, M, K, N, int(dtype),
                                                     self.mode if mode is None else int(mode)))
        return output

    def QuantizedMatMulHandle(self, input, weight: "Weight", output, M, K, N, mode=None):
        """The same slot for a layer that kept the `Weight` its registration returned (smc_qmatmul_host_w): host
        activations in, host results out, no lookup by pointer; works for weights registered from device memory."""
        # (a linear layer calls this once per matmul: the checks are kept to attribute reads, and the addresses come from
        # the array interface rather than from a ctypes view object)
        x = input if (type(input) is np.ndarray and input.dtype == np.float32 and input.flags.c_contiguous) else _f32(input)
        if x.size != M * K:
            raise ArgumentException(f"input holds {x.size} values, expected M*K = {M * K}")
        if not (type(output) is np.ndarray and output.dtype == np.float32 and output.flags.c_contiguous
                and output.size == M * N):
            raise ArgumentException("output must be a C-contiguous float32 array of M*N values")
        rc = self.ctx.lib.smc_qmatmul_host_w(self.ctx.h, x.__array_interface__["data"][0], weight.handle,
                                             output.__array_interface__["data"][0], M, K, N, self.mode if mode is None else int(mode))
        if rc:
            self.ctx.check(rc)
        return output

    def QuantizedMatMulQ8_0(self, input, rawWeights, output, M, K, N):
        return self.QuantizedMatMulFn(QuantDType.Q8_0, input, rawWeights, output, M, K, N)

    def QuantizedMatMulQ4K(self, input, rawWeights, output, M, K, N):
        return self.QuantizedMatMulFn(QuantDType.Q4_K, input, rawWeights, output, M, K, N)

    def QuantizedMatMulQ6K(self, input, rawWeights, output, M, K, N):
        return self.QuantizedMatMulFn(QuantDType.Q6_K, input, rawWeights, output, M, K, N)

    def QuantizedMatMulFor(self, dtype):
        return lambda input, rawWeights, output, M, K, N: self.QuantizedMatMulFn(dtype, input, rawWeights, output,
                                                                                  M, K, N)


class ActivationOps:
    """The `gate`, `pointwise`, `softmax`, `rmsnorm` and `attention` slots on host arrays."""

    def __init__(self, ctx: CudaContext):
        self.ctx = ctx

    @staticmethod
    def _dst(dst, n):
        if not (isinstance(dst, np.ndarray) and dst.dtype == np.float32 and dst.flags.c_contiguous and dst.size == n):
            raise ArgumentException("dst must be a C-contiguous float32 array of matching length")

    def ApplyGate(self, gate, up, dst):
        g, u = _f32(gate), _f32(up)
        self._dst(dst, g.size)
        self.ctx.check(self.ctx.lib.smc_swiglu_host(self.ctx.h, g.ctypes.data, u.ctypes.data, dst.ctypes.data, g.size))
        return dst

    def ApplyPointwise(self, src, dst):
        s = _f32(src)
        self._dst(dst, s.size)
        self.ctx.check(self.ctx.lib.smc_silu_host(self.ctx.h, s.ctypes.data, dst.ctypes.data, s.size))
        return dst

    def ApplySoftmaxRow(self, src, dst):
        s = _f32(src)
        self._dst(dst, s.size)
        self.ctx.check(self.ctx.lib.smc_softmax_row_host(self.ctx.h, s.ctypes.data, dst.ctypes.data, s.size))
        return dst

    def ApplyRMSNormRow(self, src, weight, dst, rmsInv):
        s, w = _f32(src), _f32(weight)
        self._dst(dst, s.size)
        self.ctx.check(self.ctx.lib.smc_rmsnorm_row_host(self.ctx.h, s.ctypes.data, w.ctypes.data, dst.ctypes.data,
                                                         s.size, C.c_float(rmsInv)))
        return dst

    def Softmax(self, x):
        x = _f32(x)
        out = np.empty_like(x)
        rows = x.reshape(-1, x.shape[-1])
        o = out.reshape(rows.shape)
        for r in range(rows.shape[0]):
            self.ApplySoftmaxRow(rows[r], o[r])
        return out

    def ScaledDotProduct(self, q, k, v, o, seqLen, kvLen, headDim, scale, causal, qStride, oStride, alibiSlope=0.0):
        q, k, v = _f32(q), _f32(k), _f32(v)
        self.ctx.check(self.ctx.lib.smc_sdpa_host(self.ctx.h, q.ctypes.data, k.ctypes.data, v.ctypes.data,
                                                  o.ctypes.data, seqLen, kvLen, headDim, C.c_float(scale),
                                                  1 if causal else 0, qStride, oStride, C.c_float(alibiSlope)))
        return o


class Q8Act:
    def __init__(self, ctx: CudaContext, max_rows: int, max_k: int):
        self.ctx = ctx
        h = C.c_void_p()
        ctx.check(ctx.lib.smc_q8act_create(ctx.h, max_rows, max_k, C.byref(h)))
        self.h, self.M, self.K = h, 0, 0

    def read(self):
        q = np.empty((self.M, self.K), np.int8)
        d = np.empty((self.M, self.K // 32), np.uint16)
        self.ctx.check(self.ctx.lib.smc_q8act_read(self.ctx.h, self.h, q.ctypes.data, d.ctypes.data))
        return q, d

    def close(self):
        if self.h:
            self.ctx.lib.smc_q8act_destroy(self.ctx.h, self.h)
            self.h = None


class DeviceOps:
    """Device-resident entry points over torch CUDA tensors (fp32, contiguous)."""

    def __init__(self, ctx: CudaContext):
        import torch

        self.torch = torch
        self.ctx = ctx
        self.lib = ctx.lib

    def _stream(self):
        return C.c_void_p(self.torch.cuda.current_stream().cuda_stream)

    def _chk(self, t, dtype=None):
        if not t.is_cuda or not t.is_contiguous():
            raise ArgumentException("expected a contiguous CUDA tensor")
        if dtype is not None and t.dtype != dtype:
            raise ArgumentException(f"expected dtype {dtype}, got {t.dtype}")
        return t.data_ptr()

    def qmatmul(self, x, w: Weight, mode: int = Mode.ACT_F32, out=None):
        t = self.torch
        M = x.numel() // w.K
        if x.numel() != M * w.K:
            raise ArgumentException(f"input of {x.numel()} values is not a multiple of K = {w.K}")
        if out is None:
            out = t.empty((M, w.N), dtype=t.float32, device=x.device)
        if M == 0:
            return out
        self.ctx.check(self.lib.smc_qmatmul_dev(self.ctx.h, self._chk(x, t.float32), w.handle, self._chk(out, t.float32),
                                                M, int(mode), self._stream()))
        return out

    def interleave_rows(self, gate: Weight, up: Weight) -> Weight:
        """gate and up [ffn, hidden] woven into one matrix [2 * ffn, hidden]: row 2i = gate i, row 2i + 1 = up i."""
        h = C.c_void_p()
        self.ctx.check(self.lib.smc_weight_interleave_rows(self.ctx.h, gate.handle, up.handle, C.byref(h)))
        return Weight(h, gate.dtype, 2 * gate.N, gate.K)

    def qmatmul_swiglu_pairs(self, x, w: Weight, out=None):
        """One activation row through an interleaved gate / up matrix; returns SiLU(gate . x) * (up . x), [1, N / 2]."""
        t = self.torch
        if out is None:
            out = t.empty((1, w.N // 2), dtype=t.float32, device=x.device)
        self.ctx.check(self.lib.smc_qmatmul_swiglu_pairs_dev(self.ctx.h, self._chk(x, t.float32), w.handle, self._chk(out, t.float32),
                                                            self._stream()))
        return out

    def qmatmul_tc(self, x, w: Weight, out=None):
        """Prefill-sized matmul on the tensor cores (Q4_K, N % 128 == 0, K % 256 == 0)."""
        t = self.torch
        M = x.numel() // w.K
        if x.numel() != M * w.K:
            raise ArgumentException(f"input of {x.numel()} values is not a multiple of K = {w.K}")
        if out is None:
            out = t.empty((M, w.N), dtype=t.float32, device=x.device)
        if M == 0:
            return out
        self.ctx.check(self.lib.smc_qmatmul_tc_dev(self.ctx.h, self._chk(x, t.float32), w.handle,
                                                   self._chk(out, t.float32), M, self._stream()))
        return out

    def quantize_q8(self, x, act: Q8Act, K: int):
        M = x.numel() // K
        self.ctx.check(self.lib.smc_quantize_q8_dev(self.ctx.h, self._chk(x, self.torch.float32), M, K, act.h,
                                                    self._stream()))
        act.M, act.K = M, K
        return act

    def swiglu_quantize_q8(self, gu, F: int, act: Q8Act):
        """act = Q8_0(SiLU(gate) * up) for a joined gate||up output gu [rows, 2 F]."""
        rows = gu.numel() // (2 * F)
        p = self._chk(gu, self.torch.float32)
        self.ctx.check(self.lib.smc_swiglu_quantize_q8_dev(self.ctx.h, p, p + 4 * F, rows, F, 2 * F, act.h, self._stream()))
        act.M, act.K = rows, F
        return act

    def add_rmsnorm_q8(self, x, y, w, eps: float, act: Q8Act, out=None):
        """x += y (y may be None), act = Q8_0(RMSNorm(x) * w) row by row; `out` also receives the fp32 rows."""
        rows, n = x.shape
        self.ctx.check(self.lib.smc_add_rmsnorm_q8_dev(self.ctx.h, self._chk(x, self.torch.float32), None if y is None else self._chk(y),
                                                       self._chk(w), None if out is None else self._chk(out), rows, n, eps, act.h,
                                                       self._stream()))
        act.M, act.K = rows, n
        return act

    def qmatmul_q8(self, act: Q8Act, w: Weight, out=None):
        t = self.torch
        if out is None:
            out = t.empty((act.M, w.N), dtype=t.float32, device="cuda")
        self.ctx.check(self.lib.smc_qmatmul_q8_dev(self.ctx.h, act.h, w.handle, self._chk(out, t.float32), self._stream()))
        return out

    def qmatmul_q8_noalloc(self, x, w: Weight, out=None):
        """SMC_ACT_Q8 matmul whose intermediate buffer is a fixed array inside the library: for hosts that
        may not allocate device memory while serving.  M * K is limited (SMC_NOALLOC_MAX_ELEMS)."""
        t = self.torch
        M = x.numel() // w.K
        if out is None:
            out = t.empty((M, w.N), dtype=t.float32, device=x.device)
        self.ctx.check(self.lib.smc_qmatmul_q8_noalloc(self.ctx.h, self._chk(x, t.float32), w.handle,
                                                       self._chk(out, t.float32), M, self._stream()))
        return out

    def block_isums(self, act: Q8Act, m: int, w: Weight, col0: int, col1: int):
        t = self.torch
        out = t.empty((col1 - col0, w.K // 32), dtype=t.int32, device="cuda")
        self.ctx.check(self.lib.smc_block_isums_dev(self.ctx.h, act.h, m, w.handle, col0, col1, out.data_ptr(),
                                                    self._stream()))
        return out

    def quantize_weights(self, dtype: int, values):
        """TensorQuantizer.Quantize on device: fp32 CUDA tensor -> uint8 CUDA tensor of GGUF blocks."""
        t = self.torch
        n = values.numel()
        be, bb = (32, 34) if int(dtype) == QuantDType.Q8_0 else (256, 144 if int(dtype) == QuantDType.Q4_K else 210)
        if n % be:
            raise InvalidOperationException(
                f"Cannot quantize buffer of {n} floats: length must be a multiple of {be}")
        raw = t.empty(n // be * bb, dtype=t.uint8, device=values.device)
        self.ctx.check(self.lib.smc_quantize_weights_dev(self.ctx.h, int(dtype), self._chk(values, t.float32), n,
                                                         raw.data_ptr(), self._stream()))
        return raw

    def rmsnorm(self, x, w, eps: float, out=None):
        n = x.shape[-1]
        if w.numel() != n:
            raise ArgumentException(f"Weight length {w.numel()} does not match last dim {n}.")
        if out is None:
            out = self.torch.empty_like(x)
        self.ctx.check(self.lib.smc_rmsnorm_dev(self.ctx.h, self._chk(x), self._chk(w), self._chk(out), x.numel() // n,
                                                n, C.c_float(eps), self._stream()))
        return out

    def swiglu_fused(self, gu, F: int, out=None):
        """gu [rows, 2F] = gate || up (the fused projection FfnKernels.Gated activates)."""
        t = self.torch
        rows = gu.numel() // (2 * F)
        if out is None:
            out = t.empty((rows, F), dtype=t.float32, device=gu.device)
        p = self._chk(gu, t.float32)
        self.ctx.check(self.lib.smc_swiglu_dev(self.ctx.h, p, p + 4 * F, self._chk(out), rows, F, 2 * F, self._stream()))
        return out

    def swiglu(self, gate, up, out=None):
        if out is None:
            out = self.torch.empty_like(gate)
        F = gate.shape[-1]
        self.ctx.check(self.lib.smc_swiglu_dev(self.ctx.h, self._chk(gate), self._chk(up), self._chk(out),
                                               gate.numel() // F, F, F, self._stream()))
        return out

    def silu(self, x, out=None):
        if out is None:
            out = self.torch.empty_like(x)
        self.ctx.check(self.lib.smc_silu_dev(self.ctx.h, self._chk(x), self._chk(out), x.numel(), self._stream()))
        return out

    def softmax(self, x, out=None):
        if out is None:
            out = self.torch.empty_like(x)
        n = x.shape[-1]
        self.ctx.check(self.lib.smc_softmax_dev(self.ctx.h, self._chk(x), self._chk(out), x.numel() // n, n,
                                                self._stream()))
        return out

    def rope_tables(self, theta: float, rope_dim: int, max_seq: int):
        t = self.torch
        cos = t.empty((max_seq, rope_dim // 2), dtype=t.float32, device="cuda")
        sin = t.empty_like(cos)
        self.ctx.check(self.lib.smc_rope_tables(self.ctx.h, C.c_float(theta), rope_dim, max_seq, cos.data_ptr(),
                                                sin.data_ptr()))
        return cos, sin

    def rope(self, x, pos_offset: int, cos, sin, neox: bool, rope_dim: int | None = None):
        """In place on x [seq, heads, head_dim]."""
        seq, heads, hd = x.shape
        if pos_offset + seq > cos.shape[0]:
            raise ArgumentOutOfRangeException(f"Position {pos_offset + seq} exceeds MaxSeqLen {cos.shape[0]}.")
        self.ctx.check(self.lib.smc_rope_dev(self.ctx.h, self._chk(x), seq, heads, hd, rope_dim or hd, pos_offset,
                                             self._chk(cos), self._chk(sin), 1 if neox else 0, self._stream()))
        return x

    def add_(self, x, y):
        if x.shape != y.shape:
            raise ArgumentException("AddInPlace: shapes differ")
        self.ctx.check(self.lib.smc_add_dev(self.ctx.h, self._chk(x), self._chk(y), x.numel(), self._stream()))
        return x

    def argmax(self, logits):
        t = self.torch
        n = logits.shape[-1]
        rows = logits.numel() // n
        out = t.empty(rows, dtype=t.int32, device=logits.device)
        self.ctx.check(self.lib.smc_argmax_dev(self.ctx.h, self._chk(logits), rows, n, out.data_ptr(), self._stream()))
        return out

    def sample(self, logits, temperature: float, top_k: int = 0, top_p: float = 1.0, min_p: float = 0.0, uniform=None,
               work=None):
        """Sampler.Sample per row of `logits` [rows, n]; `uniform` [rows] holds the host generator's NextSingle() per row."""
        t = self.torch

        class _Cfg(C.Structure):
            _fields_ = [("temperature", C.c_float), ("top_k", C.c_int), ("top_p", C.c_float), ("min_p", C.c_float)]

        rows, n = logits.shape
        cfg = _Cfg(temperature, top_k, top_p, min_p)
        out = t.empty(rows, dtype=t.int32, device=logits.device)
        if temperature > 0 and work is None:
            work = t.empty_like(logits)
        self.ctx.check(self.lib.smc_sample_dev(self.ctx.h, self._chk(logits, t.float32), rows, n, C.byref(cfg),
                                               None if uniform is None else self._chk(uniform, t.float32),
                                               None if work is None else self._chk(work, t.float32), out.data_ptr(),
                                               self._stream()))
        return out

    def repetition_penalty_(self, logits, ids, penalty: float):
        """RepetitionPenalty.Apply in place: `ids` [rows, window] int32 (pad with -1)."""
        t = self.torch
        rows, n = logits.shape
        self.ctx.check(self.lib.smc_repetition_penalty_dev(self.ctx.h, self._chk(logits, t.float32), rows, n,
                                                           self._chk(ids, t.int32), ids.shape[1], penalty, self._stream()))
        return logits

    def embed(self, table: Weight, tokens, out=None):
        t = self.torch
        if out is None:
            out = t.empty((tokens.numel(), table.K), dtype=t.float32, device=tokens.device)
        self.ctx.check(self.lib.smc_embed_q8_0_dev(self.ctx.h, table.handle, self._chk(tokens, t.int32), tokens.numel(),
                                                   self._chk(out), self._stream()))
        return out

    def sdpa_decode(self, q, kcache, vcache, kv_len: int, scale: float, out=None):
        """q [batch, heads, hd]; caches [batch, kv_heads, max_seq, hd]."""
        batch, heads, hd = q.shape
        _, kvh, max_seq, _ = kcache.shape
        if out is None:
            out = self.torch.empty_like(q)
        self.ctx.check(self.lib.smc_sdpa_decode_dev(self.ctx.h, self._chk(q), self._chk(kcache), self._chk(vcache),
                                                    self._chk(out), batch, heads, kvh, hd, kv_len, max_seq,
                                                    C.c_float(scale), self._stream()))
        return out

    def kv_append(self, k, v, kcache, vcache, pos: int):
        batch, kvh, max_seq, hd = kcache.shape
        self.ctx.check(self.lib.smc_kv_append_dev(self.ctx.h, self._chk(k), self._chk(v), self._chk(kcache),
                                                  self._chk(vcache), batch, kvh, hd, pos, max_seq, self._stream()))


class KVCache:
    """IKVCache on the device (SharpMind.Model/IKVCache.cs): an fp32 cache (KVCache) or a Q8_0 one (QuantizedKVCache),
    holding one attention layer's keys and values for `batch` lock-step sequences."""

    F32, Q8_0 = 0, 8

    def __init__(self, ctx: CudaContext, batch: int, kv_heads: int, max_seq: int, head_dim: int, kind: int = 0):
        import torch

        self.ctx, self.torch, self.kind = ctx, torch, kind
        self.batch, self.kv_heads, self.head_dim = batch, kv_heads, head_dim
        h = C.c_void_p()
        ctx.check(ctx.lib.smc_kv_create(ctx.h, batch, kv_heads, max_seq, head_dim, kind, C.byref(h)))
        self.h = h

    def _stream(self):
        return C.c_void_p(self.torch.cuda.current_stream().cuda_stream)

    @property
    def Length(self) -> int:
        return self.ctx.lib.smc_kv_length(self.h)

    @property
    def MaxSeqLen(self) -> int:
        return self.ctx.lib.smc_kv_max_seq(self.h)

    @property
    def IsFull(self) -> bool:
        return self.Length >= self.MaxSeqLen

    def Reset(self):
        self.ctx.check(self.ctx.lib.smc_kv_reset(self.ctx.h, self.h))

    def Truncate(self, length: int):
        self.ctx.check(self.ctx.lib.smc_kv_truncate(self.ctx.h, self.h, length))

    def TrimToLast(self, keep: int):
        self.ctx.check(self.ctx.lib.smc_kv_trim_to_last(self.ctx.h, self.h, keep, self._stream()))

    def Update(self, k, v):
        """k, v: CUDA fp32 [batch, seqLen, kvHeads, headDim]."""
        b, s = k.shape[0], k.shape[1]
        self.ctx.check(self.ctx.lib.smc_kv_update_dev(self.ctx.h, self.h, k.contiguous().data_ptr(), v.contiguous().data_ptr(),
                                                      b, s, self._stream()))

    def Snapshot(self):
        """(position, keys, values) as host arrays ([batch, kvHeads, position, row] bytes or floats), or None when empty."""
        n = self.ctx.lib.smc_kv_snapshot_bytes(self.h)
        if n == 0:
            return None
        k, v, pos = np.empty(n, np.uint8), np.empty(n, np.uint8), C.c_int()
        self.ctx.check(self.ctx.lib.smc_kv_snapshot(self.ctx.h, self.h, k.ctypes.data, v.ctypes.data, n, C.byref(pos)))
        return pos.value, k, v

    def Restore(self, snapshot):
        if snapshot is None:
            return
        pos, k, v = snapshot
        self.ctx.check(self.ctx.lib.smc_kv_restore(self.ctx.h, self.h, k.ctypes.data, v.ctypes.data, k.size, pos))

    def attention(self, q, scale: float):
        """q: CUDA fp32 [batch, seqLen, heads, headDim], the queries of the last seqLen positions; returns the same shape."""
        b, s, heads, hd = q.shape
        out = self.torch.empty_like(q)
        self.ctx.check(self.ctx.lib.smc_sdpa_kv_dev(self.ctx.h, self.h, q.contiguous().data_ptr(), out.data_ptr(), b, heads, s, scale,
                                                    self._stream()))
        return out

    def Dispose(self):
        if self.h:
            self.ctx.lib.smc_kv_destroy(self.ctx.h, self.h)
            self.h = None
