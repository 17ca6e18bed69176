#include "launch_mma.cuh"
namespace sqb {
int launch_mma_kda(const StepArgs& a, int bits, int mode, cudaStream_t stream) { return launch_mma<K_KDA, false>(a, bits, mode, stream); }
}  // namespace sqb
