// Host side of the fold launch (see fold_kernel.cuh and launchers.h for the return convention).
#include <atomic>
#include "launchers.h"
#include "fold_kernel.cuh"
#include "slot_io.cuh"

namespace sqb {
namespace {

template <bool VDEC, int BITS, bool AXK, int LPR>
int launch_fold_one(const StepArgs& a, cudaStream_t stream, float* out) {
  auto kern = fold_kernel<VDEC, BITS, AXK, LPR>;
  const SmemF plan = smemf_plan(VDEC, BITS, AXK, a.group, a.DK, a.DV, a.M, a.qbuf);
  if (plan.total > 220 * 1024) return 1;
  static SmemLimit limit;                   // per instantiation
  {
    cudaError_t e = limit.ensure(kern, plan.total);
    if (e != cudaSuccess) return -1000 - static_cast<int>(e);
  }
  static thread_local int sms[64];
  int dev = 0;
  cudaGetDevice(&dev);
  int& nsm = sms[dev & 63];
  if (!nsm) cudaDeviceGetAttribute(&nsm, cudaDevAttrMultiProcessorCount, dev);
  if (!nsm) return 1;
  FoldArgs f;
  f.S = a.S; f.SC = a.SC; f.KB = a.KB; f.KBS = a.KBS; f.UB = a.UB; f.UBS = a.UBS; f.GB = a.GB; f.GCUR = a.GCUR; f.NPTR = a.NPTR;
  f.sS = a.sS; f.sSC = a.sSC; f.sKB = a.sKB; f.sKBS = a.sKBS; f.sUB = a.sUB; f.sUBS = a.sUBS; f.sGB = a.sGB; f.sGC = a.sGC; f.sN = a.sN;
  f.idx = a.idx; f.group = a.group; f.qbuf = a.qbuf; f.M = a.M; f.HV = a.HV; f.HK = a.HK; f.DV = a.DV; f.rows = a.rows;
  f.status = a.status;
  f.out = out;
  f.tens = !VDEC && AXK && LPR == 8 && a.DV == 128 && a.M == 8 && a.qbuf &&
           ((BITS == 8 && a.group == 32) || (BITS == 4 && a.group == 64));
  const long long pairs = static_cast<long long>(a.rows) * a.HV;
  int per_sm = (220 * 1024) / (plan.total + 1024);
  if (per_sm > 4) per_sm = 4;
  if (per_sm < 1) per_sm = 1;
  long long grid = static_cast<long long>(nsm) * per_sm;
  if (grid > pairs) grid = pairs;
  kern<<<static_cast<unsigned>(grid), NT, plan.total, stream>>>(f, plan);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return -1000 - static_cast<int>(e);
  return 0;
}

template <bool VDEC>
int launch_fold_kind(const StepArgs& a, int bits, bool axk, cudaStream_t stream, float* out) {
  const bool d128 = a.DK == 128;
  if (bits == 4) {
    if (axk) return d128 ? launch_fold_one<VDEC, 4, true, 8>(a, stream, out) : launch_fold_one<VDEC, 4, true, 4>(a, stream, out);
    return d128 ? launch_fold_one<VDEC, 4, false, 8>(a, stream, out) : launch_fold_one<VDEC, 4, false, 4>(a, stream, out);
  }
  if (axk) return d128 ? launch_fold_one<VDEC, 8, true, 8>(a, stream, out) : launch_fold_one<VDEC, 8, true, 4>(a, stream, out);
  return d128 ? launch_fold_one<VDEC, 8, false, 8>(a, stream, out) : launch_fold_one<VDEC, 8, false, 4>(a, stream, out);
}

}  // namespace

int launch_fold(int kind, const StepArgs& a, int bits, bool axk, cudaStream_t stream) {
  return kind == K_KDA ? launch_fold_kind<true>(a, bits, axk, stream, nullptr) : launch_fold_kind<false>(a, bits, axk, stream, nullptr);
}

int launch_read(int kind, const StepArgs& a, int bits, bool axk, float* out, cudaStream_t stream) {
  return kind == K_KDA ? launch_fold_kind<true>(a, bits, axk, stream, out) : launch_fold_kind<false>(a, bits, axk, stream, out);
}

namespace {
template <int BITS, bool AXK, int LPR>
int launch_write_one(int kind, const StepArgs& a, const float* X, cudaStream_t stream) {
  WriteArgs w;
  w.S = a.S; w.SC = a.SC; w.GCUR = a.GCUR; w.NPTR = a.NPTR;
  w.sS = a.sS; w.sSC = a.sSC; w.sGC = a.sGC; w.sN = a.sN;
  w.idx = a.idx; w.X = X; w.group = a.group; w.HV = a.HV; w.DV = a.DV; w.rows = a.rows;
  w.nptr = a.HV > 4 ? a.HV : 4;
  w.gc_width = kind == K_KDA ? a.DK : 1;
  const long long ctas = static_cast<long long>(a.rows) * a.HV;
  if (ctas > 2147483647LL) return 1;
  slot_write_kernel<BITS, AXK, LPR><<<static_cast<unsigned>(ctas), NT, 0, stream>>>(w);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return -1000 - static_cast<int>(e);
  return 0;
}
}  // namespace

int launch_write(int kind, const StepArgs& a, int bits, bool axk, const float* X, cudaStream_t stream) {
  const bool d128 = a.DK == 128;
  if (bits == 4) {
    if (axk) return d128 ? launch_write_one<4, true, 8>(kind, a, X, stream) : launch_write_one<4, true, 4>(kind, a, X, stream);
    return d128 ? launch_write_one<4, false, 8>(kind, a, X, stream) : launch_write_one<4, false, 4>(kind, a, X, stream);
  }
  if (axk) return d128 ? launch_write_one<8, true, 8>(kind, a, X, stream) : launch_write_one<8, true, 4>(kind, a, X, stream);
  return d128 ? launch_write_one<8, false, 8>(kind, a, X, stream) : launch_write_one<8, false, 4>(kind, a, X, stream);
}

}  // namespace sqb
