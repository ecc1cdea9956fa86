// Declarations of the per-configuration launchers; each is explicitly instantiated
// in exactly one translation unit so the kernels compile in parallel.
#pragma once

#include <cuda_runtime.h>

#include "../../include/splash_sm100.h"

namespace splash {

template <int D, int DV, int BKV, int NT>
int launch_fwd(const SplashParams& p, cudaStream_t stream);

}  // namespace splash
