#include "launch_pipe.cuh"
namespace sqb {
int launch_pipe_m2(const StepArgs& a, int bits, bool axk, cudaStream_t stream) { return launch_pipe<K_M2>(a, bits, axk, stream); }
}  // namespace sqb
