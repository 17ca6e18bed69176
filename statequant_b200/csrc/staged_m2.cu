#include "launch_staged.cuh"
namespace sqb {
int launch_staged_m2(const StepArgs& a, int bits, bool axk, cudaStream_t stream) { return launch_staged<K_M2>(a, bits, axk, stream); }
}  // namespace sqb
