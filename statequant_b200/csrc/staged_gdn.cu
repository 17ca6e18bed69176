#include "launch_staged.cuh"
namespace sqb {
int launch_staged_gdn(const StepArgs& a, int bits, bool axk, cudaStream_t stream) { return launch_staged<K_GDN>(a, bits, axk, stream); }
}  // namespace sqb
