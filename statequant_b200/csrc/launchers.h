// Launchers of the staged decode-step kernels (one translation unit per recurrence kind, so that they compile in
// parallel) and of the fold kernel.  Return 0: launched; 1: the kernel does not take this shape (the caller falls back);
// < 0: -(1000 + cudaError_t).
#pragma once
#include <cuda_runtime.h>
#include "delta_step.cuh"

namespace sqb {
int launch_staged_gdn(const StepArgs& a, int bits, bool axk, cudaStream_t stream);
int launch_staged_m2(const StepArgs& a, int bits, bool axk, cudaStream_t stream);
int launch_staged_kda(const StepArgs& a, int bits, bool axk, cudaStream_t stream);
// the fold launch that follows a staged step (that kernel only appends on a slot's m-th token)
int launch_fold(int kind, const StepArgs& a, int bits, bool axk, cudaStream_t stream);
// the fold kernel in its read-out mode: out fp32 [rows, HV, d_v, d_k] = the state advanced across its pending buffer
int launch_read(int kind, const StepArgs& a, int bits, bool axk, float* out, cudaStream_t stream);
// pack canonical fp32 states X [rows, HV, d_v, d_k] into the slots and empty their buffers
int launch_write(int kind, const StepArgs& a, int bits, bool axk, const float* X, cudaStream_t stream);
}  // namespace sqb
