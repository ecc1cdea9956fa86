// Explicit instantiations of the forward launcher (see fwd_launch.cuh).
#include "fwd_launch.cuh"
namespace splash {
template int launch_fwd<128, 128, 64, 2>(const SplashParams&, cudaStream_t);
template int launch_fwd<128, 128, 128, 2>(const SplashParams&, cudaStream_t);
}  // namespace splash
