// Explicit instantiations of the forward launcher (see fwd_launch.cuh).
#include "fwd_launch.cuh"
namespace splash {
template int launch_fwd<256, 256, 64, 1>(const SplashParams&, cudaStream_t);
template int launch_fwd<256, 256, 128, 1>(const SplashParams&, cudaStream_t);
}  // namespace splash
