"""intrasm_engine_b200 — B200 (sm_100a) implementation of intrasm_engine's hot path.

Importing the package loads ``libiex_b200.so`` (raising if it was not built — there is no
CPU or PyTorch fallback) and registers the ``torch.ops.iex_ops`` operators with the
reference's schemas (intrasm_engine/pytorch/csrc/extensions/sputnik_kernels.cpp:189-193).
Unlike the reference's package init (intrasm_engine/__init__.py:17-85) it creates no
streams, changes no global precision flags and loads no host-specific CUDA runtime.
"""
from . import _lib  # noqa: F401  (raises ImportError when the CUDA library is missing)
from . import ops  # noqa: F401  (registers torch.ops.iex_ops.*)

__version__ = "0.1.0"
