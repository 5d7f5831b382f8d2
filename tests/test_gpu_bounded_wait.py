"""A bounded wait that runs out: the exchange of a row-split matmul whose peer never shows up.

Nothing here faults or hangs a GPU.  Two gather objects of a world of two live on ONE GPU in one process; object 0 is
connected to object 1's buffer (smc_gather_connect_local), and nothing ever runs on object 1, so its "ready" flag
and its packets never arrive.  With the wait limit set to a few milliseconds the fused GEMV + exchange kernel must
return by itself, the context's status word must read 2 (and be cleared by reading it), and the next call on the same
context must work and be correct.
"""
import ctypes as C
import time

import numpy as np
import pytest

from sharpmind_b200 import ops, synth
from tests.gpu_util import Q4_K, bits, to_dev

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("m", [1, 4])  # 1: the exchange rides in the one-row GEMV's tail; 4: the separate exchange kernel
def test_exchange_gives_up_when_the_peer_never_arrives(oracle, m):
    import torch

    ctx = ops.CudaContext(0)  # a context of its own: the status word it raises must not leak into the session's
    dev = ops.DeviceOps(ctx)
    lib = ctx.lib
    n, k = 512, 2048
    raw = oracle.quantize(Q4_K, synth.normal("wait", "w", (n, k), 0.02))
    w = ctx.register(raw, Q4_K, n, k)
    x = to_dev(synth.normal("wait", f"x{m}", (m, k)))
    want = dev.qmatmul(x, w, ops.Mode.ACT_Q8).cpu().numpy()

    ga, gb = C.c_void_p(), C.c_void_p()
    cap = 2 * m * n
    ctx.check(lib.smc_gather_create(ctx.h, 0, 2, cap, C.byref(ga)))
    ctx.check(lib.smc_gather_create(ctx.h, 1, 2, cap, C.byref(gb)))
    both = (C.c_void_p * 2)(ga, gb)
    ctx.check(lib.smc_gather_connect_local(ctx.h, ga, both))
    ctx.check(lib.smc_gather_set_wait_ns(ctx.h, ga, 5_000_000))  # 5 ms
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    t0 = time.perf_counter()
    ctx.check(lib.smc_qmatmul_gather_dev(ctx.h, ga, x.data_ptr(), w.handle, m, int(ops.Mode.ACT_Q8), stream))
    torch.cuda.synchronize()
    waited = time.perf_counter() - t0
    assert waited < 1.0, f"the kernel took {waited:.3f} s to give up a 5 ms wait"
    # the status word reports the abandoned wait once ...
    st = C.c_int(0)
    rc = lib.smc_device_status(ctx.h, C.byref(st))
    assert rc != 0 and st.value == 2
    assert b"bounded wait" in lib.smc_last_error(ctx.h)
    # ... and is clear afterwards: the context is usable and still correct
    assert ctx.device_status() == 0
    again = dev.qmatmul(x, w, ops.Mode.ACT_Q8).cpu().numpy()
    assert np.array_equal(bits(again), bits(want))
    # this rank's own chunk of the abandoned exchange was still computed (only the peer's half is invalid)
    buf = C.c_void_p()
    ctx.check(lib.smc_gather_buffer(ctx.h, ga, C.byref(buf)))
    mine_np = _read_floats(torch, buf.value, m * n).reshape(m, n)
    assert np.array_equal(bits(mine_np), bits(want))
    assert ctx.device_status() == 0
    ctx.check(lib.smc_gather_destroy(ctx.h, ga))
    ctx.check(lib.smc_gather_destroy(ctx.h, gb))
    ctx.release(w)
    ctx.close()


def _read_floats(torch, ptr, count):
    class _Holder:
        pass

    h = _Holder()
    h.__cuda_array_interface__ = {"shape": (count,), "typestr": "<f4", "data": (ptr, False), "version": 2}
    return torch.as_tensor(h, device="cuda").cpu().numpy()
