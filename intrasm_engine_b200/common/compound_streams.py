"""``CompoundStream`` — one CUDA stream as the graph constructor and the operators see it.

The reference wraps a single ``cudaStream_t`` in three library views (pycuda, torch and
cupy, intrasm_engine/common/compound_streams.py:7-58) because its dense branch runs
through CUTLASS-Python and Triton.  Here every kernel takes the raw stream handle through
the C ABI, so the torch view is the only one needed; the attribute layout
(``.torch_stream.stream.cuda_stream``, ``.device``, context-manager use) is kept so that code
written against the reference keeps working.
"""
from __future__ import annotations

import torch


class CompoundStream:
    def __init__(self, torch_stream: "torch.cuda.StreamContext | torch.cuda.Stream"):
        if isinstance(torch_stream, torch.cuda.Stream):
            torch_stream = torch.cuda.stream(torch_stream)
        self.torch_stream = torch_stream
        self.device = torch_stream.stream.device

    @property
    def cuda_stream(self) -> int:
        """The ``cudaStream_t`` value, as the C ABI takes it."""
        return self.torch_stream.stream.cuda_stream

    def __enter__(self):
        self.torch_stream.__enter__()
        return self

    def __exit__(self, *args):
        self.torch_stream.__exit__(*args)


class _CurrentStreams(dict):
    """``device -> CompoundStream`` of the stream that is current on first use.

    The reference creates one stream per GPU at import time and makes it current
    (intrasm_engine/__init__.py:17-51); here the entry is made lazily from whatever stream
    is current, and nothing global is changed.
    """

    def __missing__(self, device):
        device = torch.device(device)
        if device.index is None:
            device = torch.device("cuda", torch.cuda.current_device())
        cur = torch.cuda.current_stream(device)
        if cur == torch.cuda.default_stream(device):
            # Captures need a non-default stream (cudaStreamBeginCapture refuses the legacy one).
            cur = torch.cuda.Stream(device=device)
        self[device] = CompoundStream(cur)
        return self[device]


current_stream = _CurrentStreams()
