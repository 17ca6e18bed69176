// Host side of the tensor-core decode-step kernels (step_mma.cuh): which shapes they take, shared-memory sizing,
// launch (see launchers.h for the return convention).
#pragma once
#include "launchers.h"
#include "step_mma.cuh"

namespace sqb {

// Shapes the tensor-core kernels take: 4 / 8-bit codes scaled along k in groups of 32, 64 or 128, d_k 128, d_v 64 or
// 128 (whole stages of 128 rows per key head), int8 buffer, q / k per key head, every per-head chunk and table
// stride a multiple of 16 bytes.
// Scaled along v: 4- or 8-bit codes in groups of 32 rows, Gated DeltaNet, buffer length 8 (the fold inside the step kernel
// is the tensor-pipe one).
inline bool mma_shape_ok(const StepArgs& a, int bits, bool axk, bool kda, int kind = K_GDN) {
  if ((bits != 4 && bits != 8) || a.DK != 128 || !a.qbuf) return false;
  if (a.DV != 64 && a.DV != 128) return false;
  if (!axk) {
    if (a.group != 32 || kind != K_GDN || a.M != 8 || a.DV != 128) return false;
  } else if (a.group != 32 && a.group != 64 && a.group != 128) return false;
  if (!a.per_key_head && a.HV != a.HK) return false;
  const int gqa = a.HV / a.HK, hps = 128 / a.DV;
  if (gqa % hps) return false;
  if (a.M < 1 || a.M > 32 || (a.M & (a.M - 1))) return false;
  auto a16 = [](const void* p, long long s) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0 && s % 16 == 0; };
  if (!a16(a.S, a.sS) || !a16(a.SC, a.sSC) || !a16(a.UB, a.sUB) || !a16(a.KB, a.sKB)) return false;
  if (((long long)a.M * a.DV) % 16) return false;
  if (kda && (!a16(a.GB, a.sGB) || !a16(a.GCUR, a.sGC))) return false;
  return true;
}

// The fold inside the step kernel (mode 3): the formats whose fold runs on the tensor pipe carry no other fold in that
// kernel, and that one takes a buffer of 8; with another buffer length they run as step kernel + fold launch (mode 0).
inline bool mma_fold_inside(const StepArgs& a, int bits, int kind) {
  const int upg = a.axv ? 1 : a.group / 32;
  const bool tfmt = a.axv || (bits == 8 && upg == 1) || (bits == 4 && upg == 2);
  return !tfmt || fold_on_tensor_pipe(kind, bits, upg, a.M, a.axv != 0);
}

// stages resident per CTA and the plan; false if the CTA does not fit
// value heads a CTA takes (a.hpc set by the caller, if it is a divisor of the key head's value heads that fills whole
// stages; else the default below)
inline int mma_hpc(const StepArgs& a) {
  const int gqa = a.HV / a.HK, hps = 128 / a.DV;
  if (a.hpc > 0 && gqa % a.hpc == 0 && a.hpc % hps == 0) return a.hpc;
  // two stages per CTA where the key head has them (Qwen GDN: both value heads of the key head; Nemotron-H Mamba2: 4 of
  // the group's 16 heads, measured 113 us per layer-step against 158 us with all 16 and 133 us with 2)
  return gqa % (2 * hps) == 0 ? 2 * hps : gqa;
}

template <int KIND>
inline bool mma_plan(const StepArgs& a, int bits, int mode, SmemM& plan, int& nst) {
  const int gqa = mma_hpc(a), nsh = gqa / (128 / a.DV), upg = a.axv ? 1 : a.group / 32;
  nst = nsh < 4 ? nsh : 4;
  plan = smemm_plan(KIND, bits, upg, a.DV, a.M, nst, gqa, mode == 3, a.axv != 0);
  while (nst > 1 && plan.total > 96 * 1024) {
    nst--;
    plan = smemm_plan(KIND, bits, upg, a.DV, a.M, nst, gqa, mode == 3, a.axv != 0);
  }
  return plan.total <= 220 * 1024;
}

template <int KIND, int BITS, int UPG, int DV, int MODE, bool AXV, bool BIO>
int launch_mma_one_io(const StepArgs& a, cudaStream_t stream);

// bf16 activations and output take the kernel with those element types compiled in
template <int KIND, int BITS, int UPG, int DV, int MODE, bool AXV = false>
int launch_mma_one(const StepArgs& a, cudaStream_t stream) {
  if (a.dt_qk == DT_BF16 && a.dt_v == DT_BF16 && a.dt_out == DT_BF16)
    return launch_mma_one_io<KIND, BITS, UPG, DV, MODE, AXV, true>(a, stream);
  return launch_mma_one_io<KIND, BITS, UPG, DV, MODE, AXV, false>(a, stream);
}

template <int KIND, int BITS, int UPG, int DV, int MODE, bool AXV, bool BIO>
int launch_mma_one_io(const StepArgs& a, cudaStream_t stream) {
  auto kern = step_mma_kernel<KIND, BITS, UPG, DV, MODE, AXV, BIO>;
  SmemM plan;
  int nst;
  if (!mma_plan<KIND>(a, BITS, MODE, plan, nst)) return 1;
  static SmemLimit limit;                   // per instantiation
  {
    cudaError_t e = limit.ensure(kern, plan.total);
    if (e != cudaSuccess) return -1000 - static_cast<int>(e);
  }
  StepArgs b = a;
  b.hpc = mma_hpc(a);
  const long long ctas = static_cast<long long>(a.rows) * (a.HV / b.hpc);
  if (ctas > 2147483647LL) return 1;
  b.gqa_full = a.HV / a.HK;
  b.m_log2 = 0;
  while ((1 << b.m_log2) < a.M) b.m_log2++;
  if (a.HV / b.hpc > 65535) return 1;
  const dim3 grid(static_cast<unsigned>(a.rows), static_cast<unsigned>(a.HV / b.hpc));
  kern<<<grid, NT, plan.total, stream>>>(b, plan, nst);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return -1000 - static_cast<int>(e);
  return 0;
}

template <int KIND, int DV, int MODE>
int launch_mma_fmt(const StepArgs& a, int bits, cudaStream_t stream) {
  if (a.axv) {
    if constexpr (KIND == K_GDN && DV == 128)
      return bits == 4 ? launch_mma_one<KIND, 4, 1, DV, MODE, true>(a, stream) : launch_mma_one<KIND, 8, 1, DV, MODE, true>(a, stream);
    else return 1;
  }
  const int upg = a.group / 32;
  if (bits == 4) {
    if (upg == 1) return launch_mma_one<KIND, 4, 1, DV, MODE>(a, stream);
    if (upg == 2) return launch_mma_one<KIND, 4, 2, DV, MODE>(a, stream);
    return launch_mma_one<KIND, 4, 4, DV, MODE>(a, stream);
  }
  if (upg == 1) return launch_mma_one<KIND, 8, 1, DV, MODE>(a, stream);
  if (upg == 2) return launch_mma_one<KIND, 8, 2, DV, MODE>(a, stream);
  return launch_mma_one<KIND, 8, 4, DV, MODE>(a, stream);
}

// mode: 0 the step alone (the fold launch follows), 3 the step with the fold of the m-th token inside
template <int KIND, bool DV64>
int launch_mma(const StepArgs& a, int bits, int mode, cudaStream_t stream) {
  if (a.DV == 64) {
    if constexpr (DV64) {
      if (mode == 0) return launch_mma_fmt<KIND, 64, 0>(a, bits, stream);
      return launch_mma_fmt<KIND, 64, 3>(a, bits, stream);
    } else {
      return 1;
    }
  }
  if (mode == 0) return launch_mma_fmt<KIND, 128, 0>(a, bits, stream);
  return launch_mma_fmt<KIND, 128, 3>(a, bits, stream);
}

}  // namespace sqb
