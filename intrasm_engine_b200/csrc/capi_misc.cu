// Entry points that are not kernels: status text, version, compiled architecture.
#include "common.cuh"

extern "C" const char* iex_error_string(int status) {
  switch (status) {
    case IEX_OK: return "success";
    case IEX_ERR_BAD_ARG: return "iex: bad argument (null pointer, negative size or batch out of range)";
    case IEX_ERR_UNSUPPORTED: return "iex: shape not supported by this kernel family";
    case IEX_ERR_TOO_LARGE: return "iex: size exceeds a fixed-size resource of this entry point";
    case IEX_ERR_DRIVER: return "iex: CUDA driver entry point failed (tensor-map encode)";
    case IEX_ERR_TIMEOUT: return "iex: a bounded device-side wait gave up";
    case IEX_ERR_BAD_CSR: return "iex: malformed CSR argument";
    default: break;
  }
  if (status > 0) return cudaGetErrorString(static_cast<cudaError_t>(status));
  return "iex: unknown status";
}

extern "C" int iex_version(void) { return 100; }

extern "C" int iex_compiled_sm(void) {
#if defined(IEX_TARGET_SM)
  return IEX_TARGET_SM;
#else
  return 100;
#endif
}

extern "C" int iex_stream_is_capturing(void* stream) {
  cudaStreamCaptureStatus st = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(static_cast<cudaStream_t>(stream), &st) != cudaSuccess) {
    cudaGetLastError();  // a failed query must not poison the next launch check
    return 0;
  }
  return st != cudaStreamCaptureStatusNone ? 1 : 0;
}
