#include "launch_mma.cuh"
namespace sqb {
int launch_mma_m2(const StepArgs& a, int bits, int mode, cudaStream_t stream) { return launch_mma<K_M2, true>(a, bits, mode, stream); }
}  // namespace sqb
