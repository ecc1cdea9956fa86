// Explicit instantiations of the split backward launchers for head_dim != head_dim_v
// (see bwd_launch.cuh): dK/dV over the column schedule and dQ over the row schedule.
#include "bwd_launch.cuh"
namespace splash {
template int launch_bwd_col<128, 64, false>(const SplashParams&, cudaStream_t);
template int launch_bwd_col<64, 128, false>(const SplashParams&, cudaStream_t);
template int launch_bwd_row<128, 64, 64>(const SplashParams&, cudaStream_t);
template int launch_bwd_row<128, 64, 128>(const SplashParams&, cudaStream_t);
template int launch_bwd_row<64, 128, 64>(const SplashParams&, cudaStream_t);
template int launch_bwd_row<64, 128, 128>(const SplashParams&, cudaStream_t);
template size_t bwd_row_smem<128, 64, 128>(const SplashParams&);
template size_t bwd_row_smem<64, 128, 128>(const SplashParams&);
}  // namespace splash
