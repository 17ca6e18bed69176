// Host side of the persistent pipeline: stage / prologue-buffer counts that fit three CTAs per SM, grid size, launch
// (see launchers.h for the return convention).
#pragma once
#include <atomic>
#include "launchers.h"
#include "step_pipe.cuh"

namespace sqb {
inline bool al16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }
struct DeviceInfo { int sms = 0; int smem_sm = 0; };
inline const DeviceInfo& device_info() {
  static thread_local DeviceInfo info[64];
  int dev = 0;
  cudaGetDevice(&dev);
  DeviceInfo& d = info[dev & 63];
  if (!d.sms) {
    cudaDeviceGetAttribute(&d.sms, cudaDevAttrMultiProcessorCount, dev);
    cudaDeviceGetAttribute(&d.smem_sm, cudaDevAttrMaxSharedMemoryPerMultiprocessor, dev);
  }
  return d;
}

template <int KIND, int BITS, bool AXK, int LPR>
int launch_pipe_one(const StepArgs& a, cudaStream_t stream) {
  auto kern = step_pipe_kernel<KIND, BITS, AXK, LPR>;
  const int gqa = a.HV / a.HK;
  const int vsz = dt_size(a.dt_v);
  if (KIND == K_KDA && (!al16(a.GB) || a.sGB % 16)) return 1;
  const DeviceInfo& dev = device_info();
  if (!dev.sms) return 1;
  // three CTAs per SM; as many stages as fit beside two (or three) prologue buffers
  const int budget = dev.smem_sm / 3 - 1024;
  Smem3 plan;
  int nst = 0, npb = 0;
  const int tries[][2] = {{4, 3}, {3, 3}, {3, 2}, {2, 2}};
  for (auto& t : tries) {
    plan = smem3_plan(KIND, BITS, AXK, a.group, a.DK, a.DV, a.M, a.qbuf, t[0], t[1], gqa, vsz);
    if (plan.total <= budget) { nst = t[0]; npb = t[1]; break; }
  }
  if (!nst) return 1;                      // does not fit: the caller falls back
  static std::atomic<int> configured{0};
  if (plan.total > configured.load()) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, plan.total);
    if (e != cudaSuccess) return -1000 - static_cast<int>(e);
    configured.store(plan.total);
  }
  const long long tiles = static_cast<long long>(a.rows) * a.HK;
  if (tiles > 2147483647LL) return 1;
  PipeCfg cfg;
  cfg.nst = nst; cfg.npb = npb;
  cfg.ntiles = static_cast<int>(tiles);
  const long long resident = 3LL * dev.sms;
  cfg.grid = static_cast<int>(tiles < resident ? tiles : resident);
  const long long vrow = static_cast<long long>(gqa) * a.DV * vsz;
  cfg.v_bulk = al16(a.v) && a.sv % 16 == 0 && vrow % 16 == 0;
  kern<<<cfg.grid, NTP, plan.total, stream>>>(a, plan, cfg);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return -1000 - static_cast<int>(e);
  return 0;
}

template <int KIND>
int launch_pipe(const StepArgs& a, int bits, bool axk, cudaStream_t stream) {
  const bool d128 = a.DK == 128;
  if (bits == 4) {
    if (axk) return d128 ? launch_pipe_one<KIND, 4, true, 8>(a, stream) : launch_pipe_one<KIND, 4, true, 4>(a, stream);
    return d128 ? launch_pipe_one<KIND, 4, false, 8>(a, stream) : launch_pipe_one<KIND, 4, false, 4>(a, stream);
  }
  if (axk) return d128 ? launch_pipe_one<KIND, 8, true, 8>(a, stream) : launch_pipe_one<KIND, 8, true, 4>(a, stream);
  return d128 ? launch_pipe_one<KIND, 8, false, 8>(a, stream) : launch_pipe_one<KIND, 8, false, 4>(a, stream);
}

}  // namespace sqb
