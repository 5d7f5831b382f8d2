"""Shared helpers of the GPU parity tests (everything here needs a CUDA device)."""
import numpy as np

Q8_0, Q4_K, Q6_K = 8, 12, 14
BLOCK = {Q8_0: 32, Q4_K: 256, Q6_K: 256}


def row_norm_bound(oracle, dtype, raw, n, k, x):
    """1e-5 * ||w_row|| * ||x_row|| per output element, w dequantised by the oracle readers."""
    if (n * k) % BLOCK[dtype] == 0 and (dtype != Q8_0 or k % 32 == 0):
        w = oracle.dequantize(dtype, raw, n * k).reshape(n, k).astype(np.float64)
        wn = np.linalg.norm(w, axis=1)
    else:  # ragged tensors: a loose per-tensor bound is enough for a tolerance
        wn = np.full(n, 1.0)
    xn = np.linalg.norm(np.asarray(x, np.float64).reshape(-1, k), axis=1)
    return 1e-5 * xn[:, None] * wn[None, :]


def to_dev(a):
    import torch

    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def bits(a):
    return np.ascontiguousarray(a, np.float32).view(np.uint32)
