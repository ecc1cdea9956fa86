// Explicit instantiations of the row-schedule (dQ) backward launcher (see bwd_launch.cuh).
#include "bwd_launch.cuh"
namespace splash {
template int launch_bwd_row<64, 64, 64>(const SplashParams&, cudaStream_t);
template int launch_bwd_row<64, 64, 128>(const SplashParams&, cudaStream_t);
template size_t bwd_row_smem<64, 64, 64>(const SplashParams&);
template size_t bwd_row_smem<64, 64, 128>(const SplashParams&);
}  // namespace splash
