// Explicit instantiation of the fused backward launcher (see bwd_launch.cuh).
#include "bwd_launch.cuh"
namespace splash {
template int launch_bwd_col<64, 64, true>(const SplashParams&, cudaStream_t);
}  // namespace splash
