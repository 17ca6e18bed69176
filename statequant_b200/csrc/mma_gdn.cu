#include "launch_mma.cuh"
namespace sqb {
int launch_mma_gdn(const StepArgs& a, int bits, int mode, cudaStream_t stream) { return launch_mma<K_GDN, false>(a, bits, mode, stream); }
}  // namespace sqb

#ifdef SQB_TRACE
extern "C" int sqb_debug_trace(long long* host, int n) {
  return static_cast<int>(cudaMemcpyFromSymbol(host, sqb::g_mma_trace, sizeof(long long) * n));
}
#endif
