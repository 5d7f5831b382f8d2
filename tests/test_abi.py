"""The C ABI: every symbol the header declares is exported by the library and typed in the binding.
Runs without a GPU (no compute call is made)."""
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "sharpmind_cuda.h")


def declared_symbols():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"SMC_API\s+[\w\s\*]+?\b(smc_\w+)\s*\(", text)))


def test_header_declares_entry_points():
    syms = declared_symbols()
    assert "smc_qmatmul_host" in syms and "smc_qmatmul_dev" in syms and len(syms) >= 30


def test_library_exports_every_declared_symbol():
    from sharpmind_b200 import _lib

    lib = _lib.load()
    for name in declared_symbols():
        assert hasattr(lib, name), f"{name} is declared in the header but not exported"


def test_binding_covers_header_exactly():
    from sharpmind_b200 import _lib

    assert sorted(_lib.SIGNATURES) == declared_symbols()


def test_every_declaration_cites_the_reference():
    # each SMC_API declaration sits under a comment naming a SharpMind file (or says it has none)
    text = open(HEADER).read()
    assert text.count(".cs") >= 25


def test_byte_counts_without_gpu():
    from sharpmind_b200 import ops

    assert ops.raw_tensor_bytes(ops.QuantDType.Q8_0, 3072, 1024) == 3_342_336
    assert ops.raw_tensor_bytes(ops.QuantDType.Q4_K, 14336, 4096) == 33_030_144
    assert ops.raw_tensor_bytes(ops.QuantDType.Q6_K, 4096, 14336) == 48_168_960
    with pytest.raises(ops.ArgumentOutOfRangeException):
        ops.raw_tensor_bytes(3, 4, 32)


def test_no_device_fails_loudly():
    import torch

    from sharpmind_b200 import ops

    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(ops.SharpMindCudaError):
        ops.CudaContext(0)


def test_product_does_not_import_the_oracle():
    pkg = os.path.join(ROOT, "sharpmind_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                src = open(os.path.join(dirpath, f)).read()
                assert "sm_oracle" not in src and "oracle/" not in src and "import oracle" not in src, f


def test_every_option_is_documented_where_it_is_declared():
    """smc_set_option's names: each one the library accepts is described in the header and in the integration notes,
    and the header describes none the library does not know; the C# source binds every declared entry point."""
    api = open(os.path.join(ROOT, "sharpmind_b200", "csrc", "smc_api.cu")).read()
    accepted = set(re.findall(r'strcmp\(name, "([a-z0-9_]+)"\)', api))
    assert len(accepted) >= 10
    header = open(HEADER).read()
    block = header[header.index("smc_set_option") - 6000:header.index("SMC_API int smc_set_option")]
    documented = set(re.findall(r'^ \*\s+"([a-z0-9_]+)"', block, flags=re.M))
    assert accepted == documented, (sorted(accepted - documented), sorted(documented - accepted))
    notes = open(os.path.join(ROOT, "INTEGRATION.md")).read()
    for name in accepted:
        assert f"`{name}`" in notes, name
    native = open(os.path.join(ROOT, "sharpmind_b200", "dotnet", "SharpMind.Cuda", "Native.cs")).read()
    for sym in declared_symbols():
        assert re.search(rf"\b{sym}\(", native), f"{sym} has no P/Invoke declaration"
