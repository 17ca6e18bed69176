#include "launch_pipe.cuh"
namespace sqb {
int launch_pipe_gdn(const StepArgs& a, int bits, bool axk, cudaStream_t stream) { return launch_pipe<K_GDN>(a, bits, axk, stream); }
}  // namespace sqb
