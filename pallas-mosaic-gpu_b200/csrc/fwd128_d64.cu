// Explicit instantiations of the forward launcher (see fwd_launch.cuh).
#include "fwd_launch.cuh"
namespace splash {
template int launch_fwd<64, 64, 64, 1>(const SplashParams&, cudaStream_t);
template int launch_fwd<64, 64, 128, 1>(const SplashParams&, cudaStream_t);
template int launch_fwd<64, 128, 64, 1>(const SplashParams&, cudaStream_t);
template int launch_fwd<64, 128, 128, 1>(const SplashParams&, cudaStream_t);
}  // namespace splash
