#include "gga_reg.cuh"
#include "launchers.h"
namespace sqb {
// The register-tile GGA step over every (row, head) of the launch; heads it does not take return at once.
// Returns 0, 1 if the shape is not this kernel's, or -1000 - cudaError.
int launch_gga_reg(const GgaArgs& a, long long ctas, cudaStream_t stream) {
  if (a.DK != RD || a.DV != RD || a.M < 1 || a.M > 16 || a.qsz % 16 || a.qoff % 16) return 1;
  const GgaRegSmem plan = gga_reg_smem(a.M, a.qsz);
  static SmemLimit limit;
  cudaError_t e = limit.ensure(gga_step_reg_kernel, plan.total);
  if (e != cudaSuccess) return -1000 - static_cast<int>(e);
  if (ctas <= 0) return 0;
  gga_step_reg_kernel<<<static_cast<unsigned>(ctas), RNT, plan.total, stream>>>(a);
  e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -1000 - static_cast<int>(e);
}
}  // namespace sqb
