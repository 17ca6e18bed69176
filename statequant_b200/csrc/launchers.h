// Launchers of the staged decode-step kernels (one translation unit per recurrence kind, so that they compile in
// parallel) and of the fold kernel.  Return 0: launched; 1: the kernel does not take this shape (the caller falls back);
// < 0: -(1000 + cudaError_t).
#pragma once
#include <atomic>
#include <cuda_runtime.h>
#include "delta_step.cuh"

namespace sqb {
// cudaFuncAttributeMaxDynamicSharedMemorySize is a per-device setting of a kernel: remember, per device, the largest
// size already set, so that the attribute call is made only when a launch needs more on the device it runs on.
struct SmemLimit {
  std::atomic<int> set[64];
  template <class K>
  cudaError_t ensure(K kern, int bytes) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    const bool cached = dev >= 0 && dev < 64;
    if (cached && bytes <= set[dev].load(std::memory_order_relaxed)) return cudaSuccess;
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (e == cudaSuccess && cached) set[dev].store(bytes, std::memory_order_relaxed);
    return e;
  }
};
struct GgaArgs;
// the GGA step with the tile in registers (gga_reg.cuh): 0, 1 = shape not taken, -1000 - cudaError
int launch_gga_reg(const GgaArgs& a, long long ctas, cudaStream_t stream);
int launch_staged_gdn(const StepArgs& a, int bits, bool axk, cudaStream_t stream);
int launch_staged_m2(const StepArgs& a, int bits, bool axk, cudaStream_t stream);
int launch_staged_kda(const StepArgs& a, int bits, bool axk, cudaStream_t stream);
// the tensor-core kernels (step_mma.cuh); mode 0: the step alone (the fold launch follows), 3: the step with the fold
// of a slot's m-th token inside
int launch_mma_gdn(const StepArgs& a, int bits, int mode, cudaStream_t stream);
int launch_mma_m2(const StepArgs& a, int bits, int mode, cudaStream_t stream);
int launch_mma_kda(const StepArgs& a, int bits, int mode, cudaStream_t stream);
// the fold launch that follows a staged step (that kernel only appends on a slot's m-th token)
int launch_fold(int kind, const StepArgs& a, int bits, bool axk, cudaStream_t stream);
// the fold kernel in its read-out mode: out fp32 [rows, HV, d_v, d_k] = the state advanced across its pending buffer
int launch_read(int kind, const StepArgs& a, int bits, bool axk, float* out, cudaStream_t stream);
// pack canonical fp32 states X [rows, HV, d_v, d_k] into the slots and empty their buffers
int launch_write(int kind, const StepArgs& a, int bits, bool axk, const float* X, cudaStream_t stream);
}  // namespace sqb
