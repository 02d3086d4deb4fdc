// Shared device/host helpers for the sm_100a kernels of the SpMM / SDDMM / fused path.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/iex_b200.h"

namespace iex {

constexpr int kNumSMs = 148;  // B200: 2 dies x 74 SMs

// Launchers return the cudaError_t of the launch as a positive int (the reference's
// launchers return cudaGetLastError(), sputnik_spmm.cu.inc:359) or a negative IEX_ERR_*.
inline int launch_status() { return static_cast<int>(cudaGetLastError()); }

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Programmatic dependent launch.  A kernel launched through launch_overlapped() may be set up
// on the SMs (its blocks scheduled, their prologues run) while the kernel before it in the
// stream is still finishing; it calls grid_dependency_wait() before its first access to
// global memory, which returns once that kernel has completed and its writes are visible, so
// the stream's ordering is unchanged.  What is saved is the launch latency and the drain of
// the previous grid, a few microseconds per launch -- most of the time of the small launches
// on this path.  grid_launch_dependents() tells the scheduler that the kernels after this one
// may start their set-up.
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename... KArgs, typename... Args>
inline int launch_overlapped(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                             Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  const cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
  return static_cast<int>(e != cudaSuccess ? e : cudaGetLastError());
}

__device__ __forceinline__ float2 ffma2(float2 a, float2 b, float2 c) {
  return __ffma2_rn(a, b, c);  // packed fp32x2 FMA (sm_100): two exact fmaf() per issue slot
}

__device__ __forceinline__ float to_float(float v) { return v; }
__device__ __forceinline__ float to_float(__half v) { return __half2float(v); }

// Index widths: int32, or 16-bit as in the reference's fp16 kernel (short2 column
// indices, sputnik_kernels.cpp:179-181).  16-bit indices are read as unsigned.
__device__ __forceinline__ int to_index(int v) { return v; }
__device__ __forceinline__ int to_index(uint16_t v) { return static_cast<int>(v); }

}  // namespace iex
