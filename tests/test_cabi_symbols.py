"""CPU: the C-ABI library loads and exports every symbol that include/iex_b200.h declares.

No compute entry point is called here (there is no GPU); only the status helpers are.
"""
import ctypes
import os
import re

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(REPO, "include", "iex_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"IEX_API\s+[\w\s\*]+?\b(iex_\w+)\s*\(", text)))


def test_header_declares_entry_points():
    syms = declared_symbols()
    for must in ("iex_spmm_f32", "iex_spmm_f16_i16", "iex_spmm_f16_i32", "iex_sddmm_f32",
                 "iex_error_string"):
        assert must in syms


def test_library_exports_every_declared_symbol():
    from intrasm_engine_b200 import _lib
    raw = ctypes.CDLL(_lib.LIB_PATH)
    for name in declared_symbols():
        assert hasattr(raw, name), f"{name} declared in the header but not exported"
        assert name in _lib.SIGNATURES, f"{name} has no ctypes signature in _lib.py"
    assert sorted(_lib.SIGNATURES) == declared_symbols()


def test_status_helpers():
    from intrasm_engine_b200 import _lib
    assert _lib.lib.iex_compiled_sm() == 100
    assert _lib.error_string(0) == "success"
    assert "bad argument" in _lib.error_string(-1)
    assert _lib.error_string(-5)
    assert _lib.error_string(1)  # a cudaError_t text


def test_ops_registered_with_reference_schemas():
    import torch
    import intrasm_engine_b200  # noqa: F401
    from intrasm_engine_b200 import ops
    for name in ("spmm_sputnik_reuse_weight", "spmm_sputnik_atomic",
                 "spmm_sputnik_reuse_weight_half", "sddmm_sputnik_atomic_upd_weight"):
        assert name in ops.OP_NAMES
    for name in ops.OP_NAMES:
        assert hasattr(torch.ops.iex_ops, name)
        # compiled registration with a CUDA kernel and no CPU kernel
        assert torch._C._dispatch_has_kernel_for_dispatch_key(f"iex_ops::{name}", "CUDA")
        assert not torch._C._dispatch_has_kernel_for_dispatch_key(f"iex_ops::{name}", "CPU")
    schema = str(torch.ops.iex_ops.spmm_sputnik_reuse_weight.default._schema)
    assert "Tensor b, Tensor row_indices, Tensor values, Tensor row_offsets, Tensor column_indices, int m" in schema


def test_torch_extension_is_a_compiled_library():
    """The operators come from a shared object in the package, not from Python functions."""
    from intrasm_engine_b200 import ops
    raw = ctypes.CDLL(ops.EXT_PATH)
    assert os.path.dirname(ops.EXT_PATH) == os.path.join(REPO, "intrasm_engine_b200")
    assert raw is not None


def test_torch_extension_shares_the_process_cxx_runtime():
    """The extension must not carry its own copy of the C++ exception runtime (a toolchain that
    links libstdc++ statically does that): errors raised by its argument checks are thrown in
    torch's runtime and have to unwind through the extension's frames."""
    import subprocess
    from intrasm_engine_b200 import ops
    out = subprocess.run(["nm", "-D", "--defined-only", ops.EXT_PATH], capture_output=True, text=True).stdout
    assert "__cxa_allocate_exception" not in out and "__gxx_personality_v0" not in out


def test_no_cpu_fallback():
    """CPU tensors are refused: the operators exist for CUDA only."""
    import pytest
    import torch
    import intrasm_engine_b200  # noqa: F401
    z = torch.zeros(1, 2, 2)
    i = torch.zeros(2, dtype=torch.int32)
    with pytest.raises((NotImplementedError, RuntimeError)):
        torch.ops.iex_ops.spmm_sputnik_reuse_weight(z, i, torch.zeros(0), torch.zeros(3, dtype=torch.int32),
                                                    torch.zeros(0, dtype=torch.int32), 2)
