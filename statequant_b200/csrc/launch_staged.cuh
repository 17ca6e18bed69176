// Host side of the staged kernel: shared-memory sizing and launch (see launchers.h for the return convention).
#pragma once
#include <atomic>
#include "launchers.h"
#include "step_tma.cuh"

// Stages are dropped until the CTA's shared memory fits under a cap: 32 000 bytes lets seven CTAs share an SM (the
// kernels for states scaled along k are built for seven or eight; at the usual shapes they then take 24 to 25 KB,
// which fits eight), the larger one is for the others.
#ifndef SQB_STAGE_CAP_K
#define SQB_STAGE_CAP_K 32000
#endif
#ifndef SQB_STAGE_CAP
#define SQB_STAGE_CAP (100 * 1024)
#endif

namespace sqb {
template <int KIND, int BITS, bool AXK, int LPR>
int launch_staged_one(const StepArgs& a, cudaStream_t stream) {
  auto kern = step_tma_kernel<KIND, BITS, AXK, LPR>;
  const int gqa = a.HV / a.HK;
  int nst = gqa < 2 ? gqa : (KIND == K_M2 && gqa >= 3 ? 3 : 2);
  Smem2 plan = smem2_plan(KIND, BITS, AXK, a.group, a.DK, a.DV, a.M, a.qbuf, nst, gqa);
  while (nst > 1 && plan.total > (AXK ? SQB_STAGE_CAP_K : SQB_STAGE_CAP)) {
    nst--;
    plan = smem2_plan(KIND, BITS, AXK, a.group, a.DK, a.DV, a.M, a.qbuf, nst, gqa);
  }
  if (plan.total > 220 * 1024) return 1;    // does not fit: the caller falls back to the generic kernel
  static SmemLimit limit;                   // per instantiation
  {
    cudaError_t e = limit.ensure(kern, plan.total);
    if (e != cudaSuccess) return -1000 - static_cast<int>(e);
  }
  const long long ctas = static_cast<long long>(a.rows) * a.HK;
  if (ctas > 2147483647LL) return 1;
  kern<<<static_cast<unsigned>(ctas), NT, plan.total, stream>>>(a, plan, nst);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return -1000 - static_cast<int>(e);
  return 0;
}

template <int KIND>
int launch_staged(const StepArgs& a, int bits, bool axk, cudaStream_t stream) {
  const bool d128 = a.DK == 128;
  if (bits == 4) {
    if (axk) return d128 ? launch_staged_one<KIND, 4, true, 8>(a, stream) : launch_staged_one<KIND, 4, true, 4>(a, stream);
    return d128 ? launch_staged_one<KIND, 4, false, 8>(a, stream) : launch_staged_one<KIND, 4, false, 4>(a, stream);
  }
  if (axk) return d128 ? launch_staged_one<KIND, 8, true, 8>(a, stream) : launch_staged_one<KIND, 8, true, 4>(a, stream);
  return d128 ? launch_staged_one<KIND, 8, false, 8>(a, stream) : launch_staged_one<KIND, 8, false, 4>(a, stream);
}


}  // namespace sqb
