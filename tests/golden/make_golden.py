"""Regenerates tests/golden/vecdot_golden.npz.

Run in a checkout where the SharpMind tree is available and `make -C oracle ref REF=<tree>` has
built oracle/_ref/libvecdot_ref.so: the outputs stored here come from the REFERENCE'S OWN compiled
C vec-dots (tools/ReferenceDataGenerator/vecdot_ref.c), not from this repository's restatement.
Inputs are regenerated from seeds by the test, so only the outputs are stored.

    python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from oracle import sm_oracle as oracle  # noqa: E402
from sharpmind_b200 import synth  # noqa: E402
from tests.test_oracle_pins import _random_raw  # noqa: E402

SHAPES = [(8, 16, 1024), (8, 5, 137), (12, 16, 1024), (12, 6, 160), (14, 16, 1024), (14, 6, 160),
          (12, 8, 4096), (14, 4, 14336)]


def main():
    if oracle.ref_lib() is None:
        raise SystemExit("build oracle/_ref first: make -C oracle ref REF=<SharpMind tree>")
    out = {}
    for dtype, n, k in SHAPES:
        raw = _random_raw(dtype, oracle.raw_bytes(dtype, n, k) + 256, f"gold{dtype}_{n}_{k}")
        x = synth.uniform("pins", f"goldx{dtype}_{n}_{k}", (k,))
        out[f"out_{dtype}_{n}_{k}"] = np.array(
            [oracle.vecdot_ref(dtype, x, raw, c, k) for c in range(n)], np.float32)
        be = 32 if dtype == 8 else 256
        if (n * k) % be == 0 and k % 32 == 0:
            w = synth.normal("pins", f"goldw{dtype}_{n}_{k}", (n, k), 0.02)
            rawq = oracle.quantize(dtype, w)
            out[f"qout_{dtype}_{n}_{k}"] = np.array(
                [oracle.vecdot_ref(dtype, x, rawq, c, k) for c in range(n)], np.float32)
    np.savez(os.path.join(ROOT, "tests", "golden", "vecdot_golden.npz"), **out)
    print("wrote", len(out), "arrays")


if __name__ == "__main__":
    main()
