// Launcher of the CTA-pair GEMM kernels (gemm_pair.cu).
#pragma once
#include "gemm_common.cuh"

namespace b200k {

// maps: A, B (128-row boxes, 128-byte swizzle), scale factors of A and B (4-D atom maps; any
// valid map for the unscaled kinds).  `p.idesc` must describe a 256 x 256 MMA.
int launch_gemm_pair(int kind, int out_dtype, const CUtensorMap* maps, const GemmParams& p, int sms,
                     cudaStream_t stream);

}  // namespace b200k
