// Explicit instantiations of the column-schedule backward launcher (see bwd_launch.cuh).
#include "bwd_launch.cuh"
namespace splash {
template int launch_bwd_col<128, 128, false>(const SplashParams&, cudaStream_t);
}  // namespace splash
