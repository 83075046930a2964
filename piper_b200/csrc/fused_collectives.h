// Host-side launchers of the kernels that fuse a collective with the compute
// next to it over NVLink peer memory (fused_collectives.cu).
#pragma once
#include <cuda_runtime.h>

namespace piper {
}  // namespace piper
