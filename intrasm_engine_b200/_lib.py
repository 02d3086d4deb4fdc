"""ctypes binding of ``libiex_b200.so`` (the C ABI declared in ``include/iex_b200.h``).

There is no fallback: if the library has not been built, importing this module raises.
Build it with ``python intrasm_engine_b200/build.py``.
"""
from __future__ import annotations

import ctypes
import os

_PKG_DIR = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG_DIR, "libiex_b200.so")

c_int = ctypes.c_int
c_ll = ctypes.c_longlong
c_ptr = ctypes.c_void_p
c_size = ctypes.c_size_t

# name -> (restype, argtypes); must list every symbol the header declares.
SIGNATURES = {
    "iex_error_string": (ctypes.c_char_p, [c_int]),
    "iex_version": (c_int, []),
    "iex_compiled_sm": (c_int, []),
    # m k n nnz row_indices values vstride row_offsets cols dense bias out batch accumulate stream
    "iex_spmm_f32": (c_int, [c_int, c_int, c_int, c_int, c_ptr, c_ptr, c_ll, c_ptr, c_ptr,
                             c_ptr, c_ptr, c_ptr, c_int, c_int, c_ptr]),
    # m k n nnz row_indices values row_offsets cols dense bias out batch stream
    "iex_spmm_f16_i16": (c_int, [c_int, c_int, c_int, c_int, c_ptr, c_ptr, c_ptr, c_ptr,
                                 c_ptr, c_ptr, c_ptr, c_int, c_ptr]),
    "iex_spmm_f16_i32": (c_int, [c_int, c_int, c_int, c_int, c_ptr, c_ptr, c_ptr, c_ptr,
                                 c_ptr, c_ptr, c_ptr, c_int, c_ptr]),
    # m k n nnz row_indices row_offsets cols lhs rhs out batch accumulate stream
    "iex_sddmm_f32": (c_int, [c_int, c_int, c_int, c_int, c_ptr, c_ptr, c_ptr, c_ptr, c_ptr,
                              c_ptr, c_int, c_int, c_ptr]),
    # m k n nnz row_indices row_offsets cols index_bits lhs rhs out batch stream
    "iex_sddmm_f16": (c_int, [c_int, c_int, c_int, c_int, c_ptr, c_ptr, c_ptr, c_int, c_ptr, c_ptr,
                              c_ptr, c_int, c_ptr]),
    # count m k n nnz[] plans[] lhs[] rhs[] outs[] accumulate stream
    "iex_sddmm_f32_tc_batched": (c_int, [c_int, c_int, c_int, c_int, ctypes.POINTER(c_int), ctypes.POINTER(c_ptr),
                                         ctypes.POINTER(c_ptr), ctypes.POINTER(c_ptr), ctypes.POINTER(c_ptr),
                                         c_int, c_ptr]),
    "iex_sddmm_f32_tc_max_batch": (c_int, []),
    # m n nnz
    "iex_sddmm_plan_bytes": (c_size, [c_int, c_int, c_int]),
    # m n nnz row_offsets cols plan plan_bytes stream
    "iex_sddmm_plan_build": (c_int, [c_int, c_int, c_int, c_ptr, c_ptr, c_ptr, c_size, c_ptr]),
    # m n nnz tile_cols
    "iex_tile_plan_bytes": (c_size, [c_int, c_int, c_int, c_int]),
    # m n nnz tile_cols row_offsets cols plan plan_bytes stream
    "iex_tile_plan_build": (c_int, [c_int, c_int, c_int, c_int, c_ptr, c_ptr, c_ptr, c_size, c_ptr]),
    # m k n nnz plan values dense out workspace workspace_bytes stream
    "iex_spmm_f32_tc": (c_int, [c_int, c_int, c_int, c_int, c_ptr, c_ptr, c_ptr, c_ptr, c_ptr, c_size, c_ptr]),
    "iex_spmm_f32_tc_workspace_bytes": (c_size, [c_int, c_int, c_int]),
    "iex_spmm_f32_tc_supported": (c_int, [c_int, c_int, c_int]),
    "iex_spmm_f32_prefers_tc": (c_int, [c_int, c_int, c_int, c_int]),
    # m k n nnz plan lhs rhs out accumulate stream
    "iex_sddmm_f32_tc": (c_int, [c_int, c_int, c_int, c_int, c_ptr, c_ptr, c_ptr, c_ptr, c_int, c_ptr]),
    "iex_sddmm_f32_tc_supported": (c_int, [c_int, c_int, c_int, c_int]),
    "iex_sddmm_f32_prefers_tc": (c_int, [c_int, c_int, c_int, c_int, c_int]),
    # tokens in_features out_features input weight out stream
    "iex_linear_f16": (c_int, [c_int, c_int, c_int, c_ptr, c_ptr, c_ptr, c_ptr]),
    # tokens in_features out_features grad weight|input dinput|dweight stream
    "iex_linear_f16_dgrad": (c_int, [c_int, c_int, c_int, c_ptr, c_ptr, c_ptr, c_ptr]),
    "iex_linear_f16_wgrad": (c_int, [c_int, c_int, c_int, c_ptr, c_ptr, c_ptr, c_ptr]),
    # m k n nnz row_offsets cols index_bits values dense out stream
    "iex_spmm_f16_tc": (c_int, [c_int, c_int, c_int, c_int, c_ptr, c_ptr, c_int, c_ptr, c_ptr,
                                c_ptr, c_ptr]),
    # m k n nnz row_offsets cols index_bits values dense bias out stream
    "iex_spmm_f16_tc_bias_relu": (c_int, [c_int, c_int, c_int, c_int, c_ptr, c_ptr, c_int, c_ptr, c_ptr,
                                          c_ptr, c_ptr, c_ptr]),
    # m_sparse m_dense k n nnz row_offsets cols index_bits values weight x out_sparse out_dense
    # dense_out_tokens_major stream
    "iex_fused_spmm_linear_f16": (c_int, [c_int, c_int, c_int, c_int, c_int, c_ptr, c_ptr, c_int,
                                          c_ptr, c_ptr, c_ptr, c_ptr, c_ptr, c_int, c_ptr]),
    "iex_tc_workspace_bytes": (c_size, [c_int, c_int, c_int, c_int, c_int]),
    # ... parts workspace workspace_bytes stream
    "iex_linear_f16_splitk": (c_int, [c_int, c_int, c_int, c_ptr, c_ptr, c_ptr, c_int, c_ptr, c_size, c_ptr]),
    "iex_spmm_f16_tc_splitk": (c_int, [c_int, c_int, c_int, c_int, c_ptr, c_ptr, c_int, c_ptr, c_ptr,
                                       c_ptr, c_int, c_ptr, c_size, c_ptr]),
    "iex_fused_spmm_linear_f16_splitk": (c_int, [c_int, c_int, c_int, c_int, c_int, c_ptr, c_ptr, c_int,
                                                 c_ptr, c_ptr, c_ptr, c_ptr, c_ptr, c_int, c_int, c_int,
                                                 c_ptr, c_size, c_ptr]),
    "iex_static_workspace_capacity": (c_size, []),
    # tokens in_features out_features input weight out parts stream
    "iex_linear_f16_splitk_static": (c_int, [c_int, c_int, c_int, c_ptr, c_ptr, c_ptr, c_int, c_ptr]),
    # m k row_offsets cols index_bits values out stream
    # tokens in_features out_features input weight outs world rank ld_out col_offset parts ws ws_bytes stream
    "iex_linear_f16_splitk_gather": (c_int, [c_int, c_int, c_int, c_ptr, c_ptr, ctypes.POINTER(c_ptr), c_int,
                                             c_int, c_ll, c_ll, c_int, c_ptr, c_size, c_ptr]),
    # signals world rank stream
    "iex_peer_barrier": (c_int, [ctypes.POINTER(c_ptr), c_int, c_int, c_ptr]),
    # signals world rank max_polls stream
    "iex_peer_barrier_bounded": (c_int, [ctypes.POINTER(c_ptr), c_int, c_int, ctypes.c_uint, c_ptr]),
    # m k dense value_bits relu row_offsets row_indices stream
    "iex_dense_to_csr_count": (c_int, [c_int, c_int, c_ptr, c_int, c_int, c_ptr, c_ptr, c_ptr]),
    # m k dense value_bits relu row_offsets values cols index_bits stream
    "iex_dense_to_csr_fill": (c_int, [c_int, c_int, c_ptr, c_int, c_int, c_ptr, c_ptr, c_ptr, c_int, c_ptr]),
    "iex_csr_to_dense_f16": (c_int, [c_int, c_int, c_ptr, c_ptr, c_int, c_ptr, c_ptr, c_ptr]),
    # m k nnz row_offsets cols index_bits row_indices require_ascending result stream
    "iex_csr_validate": (c_int, [c_int, c_int, c_int, c_ptr, c_ptr, c_int, c_ptr, c_int, c_ptr, c_ptr]),
    "iex_stream_is_capturing": (c_int, [c_ptr]),
    "iex_last_device_status": (c_int, [c_int]),
    # graph constructor (opaque handle first)
    "iex_graph_create": (c_ptr, []),
    "iex_graph_destroy": (c_int, [c_ptr]),
    "iex_graph_register_stream": (c_int, [c_ptr, c_ptr]),
    "iex_graph_add_event_record_node": (c_int, [c_ptr, c_ptr, c_ptr]),
    "iex_graph_add_stream_wait_event_node": (c_int, [c_ptr, c_ptr, c_ptr]),
    "iex_graph_join": (c_int, [c_ptr, ctypes.POINTER(c_ptr), c_int, c_ptr]),
    "iex_graph_capture_begin": (c_int, [c_ptr, c_ptr]),
    "iex_graph_capture_end": (c_int, [c_ptr, c_ptr]),
    "iex_graph_instantiate": (c_int, [c_ptr]),
    "iex_graph_launch": (c_int, [c_ptr, c_ptr]),
    "iex_graph_exec_destroy": (c_int, [c_ptr]),
    "iex_graph_node_count": (c_int, [c_ptr, ctypes.POINTER(c_ll), ctypes.POINTER(c_ll)]),
    "iex_graph_dump": (c_int, [c_ptr, ctypes.c_char_p]),
    "iex_graph_add_child": (c_int, [c_ptr, c_ptr]),
    "iex_graph_combine": (c_ptr, [ctypes.POINTER(c_ptr), c_int]),
}


class IexError(RuntimeError):
    """A C-ABI entry point returned a non-zero status."""

    def __init__(self, name: str, status: int, text: str):
        super().__init__(f"{name} failed with status {status}: {text}")
        self.status = status


def _load() -> ctypes.CDLL:
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: the CUDA library has not been built. "
            "Run `python intrasm_engine_b200/build.py` (needs nvcc). "
            "There is no CPU or PyTorch fallback for these operators.")
    lib = ctypes.CDLL(LIB_PATH)
    for name, (restype, argtypes) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError here = header and library disagree
        fn.restype = restype
        fn.argtypes = argtypes
    return lib


lib = _load()


def error_string(status: int) -> str:
    return lib.iex_error_string(int(status)).decode()


def call(name: str, *args) -> None:
    """Call a status-returning entry point and raise ``IexError`` on failure."""
    status = getattr(lib, name)(*args)
    if status != 0:
        raise IexError(name, status, error_string(status))
