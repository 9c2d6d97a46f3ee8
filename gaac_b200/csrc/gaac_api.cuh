// Helpers shared by the C-ABI entry points.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include "../../include/gaac_b200.h"

namespace gaac {
inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
inline int launch_status() { return cudaGetLastError() == cudaSuccess ? GAAC_OK : GAAC_E_LAUNCH; }
}  // namespace gaac
