#include "launch_staged.cuh"
namespace sqb {
int launch_staged_kda(const StepArgs& a, int bits, bool axk, cudaStream_t stream) { return launch_staged<K_KDA>(a, bits, axk, stream); }
}  // namespace sqb
