// Host-side launchers of the mixture-of-experts kernels (moe.cu).
#pragma once
#include <cuda_runtime.h>

namespace piper {
}  // namespace piper
