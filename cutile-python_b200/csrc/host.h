// Host-side helpers shared by the entry-point translation units: error
// reporting, tensor-map encoding through the driver entry point, and the
// per-device status word.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/b200k.h"

namespace b200k {

// Stores a printf-style message for b200k_last_error() and returns `code`.
int fail(int code, const char* fmt, ...);

// Address of the calling thread's current device's status word (device memory that
// lives in the library image; nothing is allocated).  nullptr on failure.
int* device_status_word();

int current_sm_count();

// Rank-3 tiled tensor map.  dims/strides in the driver's convention: dims[0] is the
// contiguous dimension; strides_bytes[i] is the byte stride of dims[i + 1].
bool encode_tmap_3d(CUtensorMap* out, CUtensorMapDataType dtype, const void* base,
                    uint64_t d0, uint64_t d1, uint64_t d2, uint64_t stride1_bytes,
                    uint64_t stride2_bytes, uint32_t box0, uint32_t box1, uint32_t box2,
                    CUtensorMapSwizzle swizzle);

bool encode_tmap_4d(CUtensorMap* out, CUtensorMapDataType dtype, const void* base,
                    uint64_t d0, uint64_t d1, uint64_t d2, uint64_t d3, uint64_t stride1_bytes,
                    uint64_t stride2_bytes, uint64_t stride3_bytes, uint32_t box0, uint32_t box1,
                    uint32_t box2, uint32_t box3, CUtensorMapSwizzle swizzle);

// Counters of the tensor-map cache behind encode_tmap_3d / encode_tmap_4d.
void tmap_cache_stats(uint64_t* hits, uint64_t* misses, uint64_t* entries);

inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

// Launches `kernel` with programmatic stream serialisation: it may become resident while
// the kernel before it in `stream` still runs, and must call pdl_wait() (common.cuh) before
// it touches anything that kernel writes or reads.  Saves the launch gap between the two
// halves of a two-kernel operation (about 2 us).
template <typename... Params, typename... Args>
cudaError_t launch_after_predecessor(void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem_bytes,
                                     cudaStream_t stream, Args... args) {
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem_bytes;
  cfg.stream = stream;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<Params>(args)...);
}

#define B200K_CHECK_LAUNCH(what)                                                        \
  do {                                                                                  \
    cudaError_t e__ = cudaGetLastError();                                               \
    if (e__ != cudaSuccess)                                                             \
      return ::b200k::fail(B200K_CUDA_ERROR, "%s: %s", what, cudaGetErrorString(e__));  \
  } while (0)

}  // namespace b200k
