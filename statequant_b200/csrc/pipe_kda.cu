#include "launch_pipe.cuh"
namespace sqb {
int launch_pipe_kda(const StepArgs& a, int bits, bool axk, cudaStream_t stream) { return launch_pipe<K_KDA>(a, bits, axk, stream); }
}  // namespace sqb
