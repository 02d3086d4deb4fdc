"""``TorchCUDAGraphConstructor`` — multi-stream capture into one CUDA graph.

Same entry points as intrasm_engine/pytorch/cpp_extensions/cuda_graph_constructor.py:12-147
(``get_primary_stream``, ``register_new_stream(s)``, ``add_event_record_node``,
``add_stream_wait_event_node``, ``capture_library_call_begin/end``, ``join``,
``instantiate_graph_exec``, ``execute_graph``, ``synchronize``, ``destroy_graph_exec``,
``print_graph``, context-manager use), on top of the ``iex_graph_*`` C ABI instead of a
pybind class.  ``CUDAGraphCaptureNotifier`` does the PyTorch bookkeeping that the
reference does in C++ (pybind.cu:163-333): while a foreign capture is active, tensor
allocations of the capturing thread go to a private pool of the caching allocator, so the
memory the captured kernels write stays reserved for replays.
"""
from __future__ import annotations

import ctypes

import torch

from ... import _lib
from ...common.compound_streams import CompoundStream, current_stream


class CUDAGraphCaptureNotifier:
    """Allocator bookkeeping around a capture that PyTorch did not start itself.

    ``capture_begin(pool)`` routes this thread's allocations on the current device to a
    private pool (a fresh one, or ``pool`` to share), ``capture_end`` stops that, ``pool()``
    returns the pool id.  The reference also snapshots the default generator's Philox
    state for replay (pybind.cu:183-196, :269-285); none of the kernels behind this library
    draws random numbers, so ``replay`` has nothing to restore.
    """

    def __init__(self):
        self._pool = None
        self._device = None
        self._active = False

    def capture_begin(self, pool=None):
        if self._active:
            raise RuntimeError("capture_begin called twice without capture_end")
        stream = torch.cuda.current_stream()
        if stream == torch.cuda.default_stream():
            raise RuntimeError("CUDA graphs must be captured on a non-default stream")
        self._device = torch.cuda.current_device()
        if pool is not None:
            self._pool = pool
        elif self._pool is None:
            self._pool = torch.cuda.graph_pool_handle()
        torch._C._cuda_beginAllocateCurrentThreadToPool(self._device, self._pool)
        self._active = True

    def assert_capture_has_begun(self):
        if not self._active or not torch.cuda.is_current_stream_capturing():
            raise RuntimeError("the current stream is not capturing")

    def capture_end(self):
        if not self._active:
            raise RuntimeError("capture_end without capture_begin")
        torch._C._cuda_endAllocateToPool(self._device, self._pool)
        self._active = False

    def replay(self):
        return None

    def pool(self):
        return self._pool


class TorchCUDAGraphConstructor:
    """One CUDA graph built from library calls on several registered streams."""

    def __init__(self, device=None):
        if device is None:
            device = torch.device("cuda", torch.cuda.current_device())
        self.device = torch.device(device)
        self.registeredStreams: list[CompoundStream] = [current_stream[self.device]]
        self.notifier = CUDAGraphCaptureNotifier()
        self._handle = _lib.lib.iex_graph_create()
        if not self._handle:
            raise RuntimeError("iex_graph_create failed")
        _lib.call("iex_graph_register_stream", self._handle, self.registeredStreams[0].cuda_stream)
        self._capturing_stream = None

    # -- the native handle, for add_child / combine ------------------------------------
    @property
    def constructor(self):
        return self

    def __del__(self):
        handle, self._handle = getattr(self, "_handle", None), None
        if handle:
            _lib.lib.iex_graph_destroy(handle)

    # -- streams -------------------------------------------------------------------------
    def get_primary_stream(self) -> CompoundStream:
        """The first stream: where the other streams join and where the graph is launched."""
        return self.registeredStreams[0]

    def register_new_stream(self) -> CompoundStream:
        stream = CompoundStream(torch.cuda.Stream(device=self.device))
        self.registeredStreams.append(stream)
        _lib.call("iex_graph_register_stream", self._handle, stream.cuda_stream)
        return stream

    def register_new_streams(self, num_streams: int) -> list[CompoundStream]:
        return [self.register_new_stream() for _ in range(num_streams)]

    def assert_current_stream_registered(self):
        cur = torch.cuda.current_stream(self.device).cuda_stream
        if cur not in {s.cuda_stream for s in self.registeredStreams}:
            raise AssertionError("Current stream is not registered.")

    # -- explicit nodes ------------------------------------------------------------------
    @staticmethod
    def _event_handle(event: torch.cuda.Event) -> int:
        if event.cuda_event == 0:
            raise AssertionError(
                "Event uninitialized: PyTorch creates the CUDA event lazily; call event.record() "
                "once before handing it to the graph constructor.")
        return event.cuda_event

    @staticmethod
    def _stream_handle(stream) -> int:
        if isinstance(stream, CompoundStream):
            return stream.cuda_stream
        if isinstance(stream, torch.cuda.Stream):
            return stream.cuda_stream
        return stream.stream.cuda_stream  # torch.cuda.StreamContext

    def add_event_record_node(self, event: torch.cuda.Event, torch_stream):
        _lib.call("iex_graph_add_event_record_node", self._handle, self._event_handle(event),
                  self._stream_handle(torch_stream))

    def add_stream_wait_event_node(self, torch_stream, event: torch.cuda.Event):
        _lib.call("iex_graph_add_stream_wait_event_node", self._handle,
                  self._stream_handle(torch_stream), self._event_handle(event))

    def join(self, streams: list, dest_stream):
        arr = (ctypes.c_void_p * len(streams))(*[self._stream_handle(s) for s in streams])
        _lib.call("iex_graph_join", self._handle, arr, len(streams), self._stream_handle(dest_stream))

    # -- capture of library calls --------------------------------------------------------
    def capture_library_call_begin(self):
        self.assert_current_stream_registered()
        self.notifier.capture_begin(None)
        self._capturing_stream = torch.cuda.current_stream(self.device).cuda_stream
        try:
            _lib.call("iex_graph_capture_begin", self._handle, self._capturing_stream)
        except Exception:
            self.notifier.capture_end()
            self._capturing_stream = None
            raise
        self.notifier.assert_capture_has_begun()

    def capture_library_call_end(self):
        stream, self._capturing_stream = self._capturing_stream, None
        try:
            _lib.call("iex_graph_capture_end", self._handle, stream)
        finally:
            self.notifier.capture_end()

    def __enter__(self):
        """``with stream: with constructor: <library calls>`` records the calls."""
        self.capture_library_call_begin()
        return self

    def __exit__(self, *args):
        self.capture_library_call_end()

    # -- execution -----------------------------------------------------------------------
    def instantiate_graph_exec(self):
        _lib.call("iex_graph_instantiate", self._handle)

    def execute_graph(self):
        self.notifier.replay()
        _lib.call("iex_graph_launch", self._handle, self.registeredStreams[0].cuda_stream)

    def synchronize(self):
        torch.cuda.synchronize(device=self.device)

    def destroy_graph_exec(self):
        _lib.call("iex_graph_exec_destroy", self._handle)

    # -- inspection / composition --------------------------------------------------------
    def node_count(self) -> tuple[int, int]:
        n, e = ctypes.c_longlong(0), ctypes.c_longlong(0)
        _lib.call("iex_graph_node_count", self._handle, ctypes.byref(n), ctypes.byref(e))
        return n.value, e.value

    def print_graph(self):
        n, e = self.node_count()
        print(f"CUDA graph: {n} nodes, {e} edges, {len(self.registeredStreams)} registered streams")

    def dump_graph(self, path: str):
        _lib.call("iex_graph_dump", self._handle, str(path).encode())

    def add_graph_as_child_node(self, other: "TorchCUDAGraphConstructor"):
        _lib.call("iex_graph_add_child", self._handle, other._handle)


def combine_graphs(constructors: list[TorchCUDAGraphConstructor]) -> TorchCUDAGraphConstructor:
    """A constructor whose graph runs the given graphs side by side under one root."""
    out = TorchCUDAGraphConstructor(constructors[0].device if constructors else None)
    for c in constructors:
        out.add_graph_as_child_node(c)
    return out
