// Block quantisers and the scale-factor relayout that sit either side of the
// block-scaled GEMM.  All three are HBM-bound byte shuffles: one pass over the input,
// 16-byte vector loads and stores, no shared-memory staging needed.
//
//   mxfp8_quantize : x (rows, K) f32|bf16|f16 -> e4m3 bytes + one ue8m0 scale per 32
//                    elements, bit-for-bit the result of the reference's
//                    block_quantize(x.float(), 32) (test/kernels/kernel_utils.py:38-80)
//   sf_swizzle     : logical (rows, K/block) scale bytes -> swizzle_32_4_4 atoms
//                    (test/kernels/kernel_utils.py:83-98)
//   nvfp4_quantize : x -> e2m1 pairs + one ue4m3 scale per 16 elements + one fp32
//                    per-tensor scale (the reference has no such quantiser; the rule is
//                    stated at b200k_nvfp4_quantize in include/b200k.h)
#include <cuda_fp8.h>
#include <cuda_fp4.h>

#include <mutex>

#include "common.cuh"
#include "host.h"
#include "mx_quant.cuh"

namespace b200k {
namespace {

template <typename T>
__device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }
__device__ __forceinline__ float2 to_f32x2(__nv_bfloat162 v) { return __bfloat1622float2(v); }
__device__ __forceinline__ float2 to_f32x2(__half2 v) { return __half22float2(v); }
template <typename P> __device__ __forceinline__ P to_packed2(float v);
template <> __device__ __forceinline__ __nv_bfloat162 to_packed2<__nv_bfloat162>(float v) { return __float2bfloat162_rn(v); }
template <> __device__ __forceinline__ __half2 to_packed2<__half2>(float v) { return __float2half2_rn(v); }

// Loads N consecutive elements (N * sizeof(T) a multiple of 16, address 16-byte aligned
// when `vec` is true) and widens them to fp32.
template <typename T, int N>
__device__ __forceinline__ void load_block(const T* src, float (&v)[N], bool vec, int valid) {
  if (vec && valid == N) {
    constexpr int kPer = 16 / sizeof(T);
    constexpr int kVecs = N / kPer;
    const uint4* s4 = reinterpret_cast<const uint4*>(src);
#pragma unroll
    for (int i = 0; i < kVecs; ++i) {
      uint4 q = s4[i];
      const T* e = reinterpret_cast<const T*>(&q);
#pragma unroll
      for (int j = 0; j < kPer; ++j) v[i * kPer + j] = to_f32<T>(e[j]);
    }
  } else {
#pragma unroll
    for (int i = 0; i < N; ++i) v[i] = i < valid ? to_f32<T>(src[i]) : 0.0f;
  }
}

template <typename T> struct Packed2;
template <> struct Packed2<__nv_bfloat16> { using type = __nv_bfloat162; };
template <> struct Packed2<__half> { using type = __half2; };

// max |x| over the elements [begin, end) of the row-major index space of an (rows, k) tensor
// with leading dimension ldx, strided over the block's threads.  NaNs are ignored, as fmaxf
// does.  Rows of whole 16-byte vectors on 16-byte boundaries take a vector path: 16-bit
// types stay packed (|x| and max on pairs), one 16-byte load per 8 elements.
template <typename T>
__device__ __forceinline__ float block_strided_absmax(const T* __restrict__ x, int64_t k, int64_t ldx,
                                                      int64_t begin, int64_t end, int64_t first,
                                                      int64_t stride) {
  constexpr int VE = 16 / sizeof(T);
  const bool vec = (reinterpret_cast<uintptr_t>(x) % 16 == 0) && ((ldx * sizeof(T)) % 16 == 0) &&
                   (k % VE == 0) && (begin % VE == 0);
  float m = 0.0f;
  if (vec) {
    const int64_t kv = k / VE;
    const int64_t v_end = end / VE;
    if constexpr (sizeof(T) == 2) {
      using P = typename Packed2<T>::type;
      P pm[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) pm[i] = to_packed2<P>(0.0f);
      int64_t v = begin / VE + first;
      if (ldx == k) {
        // contiguous tensor: a flat array, four independent 16-byte loads per trip
        const uint4* flat = reinterpret_cast<const uint4*>(x);
        for (; v + 3 * stride < v_end; v += 4 * stride) {
          uint4 raw[4];
#pragma unroll
          for (int u = 0; u < 4; ++u) raw[u] = flat[v + u * stride];
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const P* pr = reinterpret_cast<const P*>(&raw[u]);
#pragma unroll
            for (int i = 0; i < 4; ++i) pm[i] = __hmax2(pm[i], __habs2(pr[i]));
          }
        }
      }
      for (; v < v_end; v += stride) {
        const int64_t row = v / kv;
        const uint4 raw = *reinterpret_cast<const uint4*>(x + row * ldx + (v - row * kv) * VE);
        const P* pr = reinterpret_cast<const P*>(&raw);
#pragma unroll
        for (int i = 0; i < 4; ++i) pm[i] = __hmax2(pm[i], __habs2(pr[i]));
      }
      const float2 a = to_f32x2(__hmax2(__hmax2(pm[0], pm[1]), __hmax2(pm[2], pm[3])));
      m = fmaxf(a.x, a.y);
    } else {
      for (int64_t v = begin / VE + first; v < v_end; v += stride) {
        const int64_t row = v / kv;
        const float4 f = *reinterpret_cast<const float4*>(x + row * ldx + (v - row * kv) * VE);
        m = fmaxf(m, fmaxf(fmaxf(fabsf(f.x), fabsf(f.y)), fmaxf(fabsf(f.z), fabsf(f.w))));
      }
    }
    begin = v_end * VE;   // scalar tail of a range that does not end on a vector
  }
  for (int64_t idx = begin + first; idx < end; idx += stride) {
    const int64_t row = idx / k;
    m = fmaxf(m, fabsf(to_f32<T>(x[row * ldx + (idx - row * k)])));
  }
  return m;
}

// One full, 16-byte-aligned block of 16-bit elements: the maximum is taken on packed pairs
// (NaN-propagating), the products are formed in fp32 and converted two at a time.  Returns
// the scale byte; writes the 32 quantised bytes.
template <typename T>
__device__ __forceinline__ uint8_t quantize_block_packed(const T* src, uint8_t* dst, int fmt_e5m2) {
  using P = typename Packed2<T>::type;
  uint4 raw[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) raw[i] = reinterpret_cast<const uint4*>(src)[i];
  const P* pairs = reinterpret_cast<const P*>(raw);
  P m = __habs2(pairs[0]);
#pragma unroll
  for (int i = 1; i < 16; ++i) m = __hmax2_nan(m, __habs2(pairs[i]));
  const float2 mf = to_f32x2(m);
  const bool has_nan = (mf.x != mf.x) || (mf.y != mf.y);
  float inv_scale;
  const uint8_t sf_byte = block_scale(fmaxf(mf.x, mf.y), has_nan, &inv_scale);
  uint32_t out[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    float2 lo = to_f32x2(pairs[2 * i]), hi = to_f32x2(pairs[2 * i + 1]);
    lo.x *= inv_scale; lo.y *= inv_scale; hi.x *= inv_scale; hi.y *= inv_scale;
    const __nv_fp8_interpretation_t fmt = fmt_e5m2 ? __NV_E5M2 : __NV_E4M3;
    const uint32_t a = __nv_cvt_float2_to_fp8x2(lo, __NV_SATFINITE, fmt);
    const uint32_t b = __nv_cvt_float2_to_fp8x2(hi, __NV_SATFINITE, fmt);
    out[i] = a | (b << 16);
  }
  reinterpret_cast<uint4*>(dst)[0] = make_uint4(out[0], out[1], out[2], out[3]);
  reinterpret_cast<uint4*>(dst)[1] = make_uint4(out[4], out[5], out[6], out[7]);
  return sf_byte;
}

template <typename T>
__global__ void __launch_bounds__(256)
mxfp8_quantize_kernel(const T* __restrict__ x, int64_t rows, int64_t k, int64_t ldx,
                      uint8_t* __restrict__ q, int64_t ldq, uint8_t* __restrict__ sf_logical,
                      uint8_t* __restrict__ sf_swizzled, int64_t k_atoms, int fmt_e5m2,
                      const int* __restrict__ gather_index, int gather_div, int64_t src_rows,
                      const int* __restrict__ live_blocks, int tile_m) {
  const int64_t kblocks = (k + 31) >> 5;
  if (live_blocks != nullptr) {
    const int64_t live = static_cast<int64_t>(*live_blocks) * tile_m;
    rows = live < rows ? live : rows;
  }
  const int64_t total = rows * kblocks;
  const bool vec_in = (reinterpret_cast<uintptr_t>(x) % 16 == 0) && ((ldx * sizeof(T)) % 16 == 0);
  const bool vec_out = (reinterpret_cast<uintptr_t>(q) % 16 == 0) && (ldq % 16 == 0);
  for (int64_t idx = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    int64_t row, kb;
    if (total < (1ll << 31)) {   // 32-bit division is several times cheaper than the 64-bit one
      const uint32_t r32 = static_cast<uint32_t>(idx) / static_cast<uint32_t>(kblocks);
      row = r32;
      kb = static_cast<uint32_t>(idx) - r32 * static_cast<uint32_t>(kblocks);
    } else {
      row = idx / kblocks;
      kb = idx - row * kblocks;
    }
    const int valid = static_cast<int>(k - kb * 32 < 32 ? k - kb * 32 : 32);
    float v[32];
    int64_t src_row = row;
    if (gather_index != nullptr) {
      const int g = gather_index[row];
      src_row = (g >= 0 && g / gather_div < src_rows) ? g / gather_div : -1;
    }
    if constexpr (sizeof(T) == 2) {
      if (vec_in && vec_out && valid == 32 && src_row >= 0) {
        const uint8_t sf_byte = quantize_block_packed<T>(x + src_row * ldx + kb * 32,
                                                         q + row * ldq + kb * 32, fmt_e5m2);
        if (sf_logical != nullptr) sf_logical[row * kblocks + kb] = sf_byte;
        if (sf_swizzled != nullptr) sf_swizzled[swizzled_sf_offset(row, kb, k_atoms)] = sf_byte;
        continue;
      }
    }
    if (src_row >= 0) {
      load_block<T, 32>(x + src_row * ldx + kb * 32, v, vec_in, valid);
    } else {
#pragma unroll
      for (int i = 0; i < 32; ++i) v[i] = 0.0f;
    }
    float amax = 0.0f;
    bool has_nan = false;
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      amax = fmaxf(amax, fabsf(v[i]));
      has_nan |= (v[i] != v[i]);
    }
    float inv_scale;
    const uint8_t sf_byte = block_scale(amax, has_nan, &inv_scale);
    uint32_t packed[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      uint32_t w = 0;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float y = v[4 * i + j] * inv_scale;
        const uint8_t b = fmt_e5m2 ? __nv_cvt_float_to_fp8(y, __NV_SATFINITE, __NV_E5M2)
                                   : __nv_cvt_float_to_fp8(y, __NV_SATFINITE, __NV_E4M3);
        w |= static_cast<uint32_t>(b) << (8 * j);
      }
      packed[i] = w;
    }
    uint8_t* dst = q + row * ldq + kb * 32;
    if (vec_out && valid == 32) {
      reinterpret_cast<uint4*>(dst)[0] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
      reinterpret_cast<uint4*>(dst)[1] = make_uint4(packed[4], packed[5], packed[6], packed[7]);
    } else {
      for (int i = 0; i < valid; ++i) dst[i] = (packed[i >> 2] >> (8 * (i & 3))) & 0xff;
    }
    if (sf_logical != nullptr) sf_logical[row * kblocks + kb] = sf_byte;
    if (sf_swizzled != nullptr) sf_swizzled[swizzled_sf_offset(row, kb, k_atoms)] = sf_byte;
  }
}

// One thread per 16 output bytes of the swizzled tensor (one row of an atom).
__global__ void __launch_bounds__(256)
sf_swizzle_kernel(const uint8_t* __restrict__ src, int64_t rows, int64_t kblocks, int64_t ld,
                  uint8_t* __restrict__ dst, int64_t row_tiles, int64_t k_atoms, int fill,
                  const int32_t* __restrict__ live_tiles, int live_tile_rows) {
  // only the first *live_tiles * live_tile_rows rows are in use (a device-side count)
  if (live_tiles != nullptr) {
    const int64_t live = (static_cast<int64_t>(*live_tiles) * live_tile_rows + 127) / 128;
    if (live < row_tiles) row_tiles = live;
  }
  const int64_t total = row_tiles * k_atoms * 32;
  for (int64_t idx = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t r32 = idx & 31;
    const int64_t atom = idx >> 5;
    const int64_t ka = atom % k_atoms;
    const int64_t rt = atom / k_atoms;
    uint32_t w[4];
#pragma unroll
    for (int m2 = 0; m2 < 4; ++m2) {
      const int64_t row = rt * 128 + m2 * 32 + r32;
      uint32_t word = 0;
#pragma unroll
      for (int k1 = 0; k1 < 4; ++k1) {
        const int64_t kb = ka * 4 + k1;
        uint32_t b = (row < rows && kb < kblocks) ? src[row * ld + kb] : static_cast<uint32_t>(fill);
        word |= b << (8 * k1);
      }
      w[m2] = word;
    }
    reinterpret_cast<uint4*>(dst)[idx] = make_uint4(w[0], w[1], w[2], w[3]);
  }
}

// ---- NVFP4 ----------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256)
absmax_kernel(const T* __restrict__ x, int64_t rows, int64_t k, int64_t ldx,
              uint32_t* __restrict__ amax_bits) {
  pdl_launch_dependents();   // the quantising kernel may be set up now; it waits for this grid
  float m = block_strided_absmax<T>(x, k, ldx, 0, rows * k,
                                    blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x,
                                    static_cast<int64_t>(gridDim.x) * blockDim.x);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  __shared__ float part[8];
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = m;
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int i = 1; i < 8; ++i) m = fmaxf(m, part[i]);
    // non-negative floats order like their bit patterns
    atomicMax(amax_bits, __float_as_uint(m));
  }
}

// BPT = blocks per thread.  2 (K a multiple of 32, 16-byte-aligned rows in and out): 64 or
// 128 bytes in flight per thread, one 16-byte store of codes and one 2-byte store of
// scales.  1: any shape.
template <typename T, int BPT>
__global__ void __launch_bounds__(256)
nvfp4_quantize_kernel(const T* __restrict__ x, int64_t rows, int64_t k, int64_t ldx,
                      uint8_t* __restrict__ q, int64_t ldq_bytes, uint8_t* __restrict__ sf_logical,
                      uint8_t* __restrict__ sf_swizzled, int64_t k_atoms,
                      const uint32_t* __restrict__ amax_bits, float* __restrict__ tensor_scale) {
  pdl_wait();   // the maximum comes from the kernel launched just before
  float s_t;
  if (amax_bits != nullptr) {
    const float amax_t = __uint_as_float(*amax_bits);
    s_t = __fdiv_rn(amax_t, 2688.0f);  // 448 * 6
    if (blockIdx.x == 0 && threadIdx.x == 0 && tensor_scale != nullptr) *tensor_scale = s_t;
  } else {
    s_t = *tensor_scale;               // given by the caller: nothing to find, nothing to write
  }
  const float six_st = __fmul_rn(6.0f, s_t);
  const int64_t kblocks = (k + 15) >> 4;
  const int64_t per_row = kblocks / BPT;          // BPT == 2 only with an even block count
  const int64_t total = rows * per_row;
  const bool vec_in = (reinterpret_cast<uintptr_t>(x) % 16 == 0) && ((ldx * sizeof(T)) % 16 == 0);
  for (int64_t idx = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    int64_t row, item;
    if (total < (1ll << 31)) {
      const uint32_t r32 = static_cast<uint32_t>(idx) / static_cast<uint32_t>(per_row);
      row = r32;
      item = static_cast<uint32_t>(idx) - r32 * static_cast<uint32_t>(per_row);
    } else {
      row = idx / per_row;
      item = idx - row * per_row;
    }
    const int64_t kb = item * BPT;
    if constexpr (BPT == 2) {
      float v[2][16];
      load_block<T, 16>(x + row * ldx + kb * 16, v[0], true, 16);
      load_block<T, 16>(x + row * ldx + kb * 16 + 16, v[1], true, 16);
      uint32_t w[4];
      const uint8_t s0 = nvfp4_block(v[0], six_st, s_t, &w[0], &w[1]);
      const uint8_t s1 = nvfp4_block(v[1], six_st, s_t, &w[2], &w[3]);
      *reinterpret_cast<uint4*>(q + row * ldq_bytes + kb * 8) = make_uint4(w[0], w[1], w[2], w[3]);
      const uint16_t pair = static_cast<uint16_t>(s0) | (static_cast<uint16_t>(s1) << 8);
      // kb is even: the two scale bytes are neighbours in both layouts
      if (sf_logical != nullptr) *reinterpret_cast<uint16_t*>(sf_logical + row * kblocks + kb) = pair;
      if (sf_swizzled != nullptr)
        *reinterpret_cast<uint16_t*>(sf_swizzled + swizzled_sf_offset(row, kb, k_atoms)) = pair;
    } else {
      const int valid = static_cast<int>(k - kb * 16 < 16 ? k - kb * 16 : 16);
      float v[16];
      load_block<T, 16>(x + row * ldx + kb * 16, v, vec_in, valid);
      uint32_t lo, hi;
      const uint8_t sf_byte = nvfp4_block(v, six_st, s_t, &lo, &hi);
      uint8_t* dst = q + row * ldq_bytes + kb * 8;
      if (valid == 16 && (reinterpret_cast<uintptr_t>(dst) % 8 == 0)) {
        *reinterpret_cast<uint2*>(dst) = make_uint2(lo, hi);
      } else {
        for (int i = 0; i < (valid + 1) / 2; ++i)
          dst[i] = ((i < 4 ? lo >> (8 * i) : hi >> (8 * (i - 4))) & 0xff);
      }
      if (sf_logical != nullptr) sf_logical[row * kblocks + kb] = sf_byte;
      if (sf_swizzled != nullptr) sf_swizzled[swizzled_sf_offset(row, kb, k_atoms)] = sf_byte;
    }
  }
}

// ---- scratch that lives in the library image (for b200k_nvfp4_quantize_noalloc) ----
// One partial |x| maximum per slab of kNoAllocSlabElems elements.  64 KB per GPU that
// loads the library, held until the process exits.
constexpr int kNoAllocSlots = 16384;
constexpr int64_t kNoAllocSlabElems = 65536;
static __device__ __align__(256) uint32_t g_noalloc_amax[kNoAllocSlots];

// Block b reduces elements [b * slab, (b + 1) * slab) of the row-major index space and
// overwrites slot b: every slot a call reads is written by that call first.
template <typename T>
__global__ void __launch_bounds__(256)
absmax_slab_kernel(const T* __restrict__ x, int64_t rows, int64_t k, int64_t ldx,
                   uint32_t* __restrict__ slots) {
  const int64_t total = rows * k;
  const int64_t begin = static_cast<int64_t>(blockIdx.x) * kNoAllocSlabElems;
  const int64_t end = begin + kNoAllocSlabElems < total ? begin + kNoAllocSlabElems : total;
  float m = block_strided_absmax<T>(x, k, ldx, begin, end, threadIdx.x, blockDim.x);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  __shared__ float part[8];
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = m;
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int i = 1; i < 8; ++i) m = fmaxf(m, part[i]);
    slots[blockIdx.x] = __float_as_uint(m);
  }
}

// Single block: folds slots [0, n) into slot 0.
__global__ void __launch_bounds__(256) fold_slots_kernel(uint32_t* __restrict__ slots, int n) {
  uint32_t m = 0;  // non-negative floats order like their bit patterns
  for (int i = threadIdx.x; i < n; i += blockDim.x) m = max(m, slots[i]);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = max(m, __shfl_xor_sync(0xffffffffu, m, o));
  __shared__ uint32_t part[8];
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = m;
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int i = 1; i < 8; ++i) m = max(m, part[i]);
    slots[0] = m;
  }
}

// Device address of g_noalloc_amax per device.  In host code the array's name is only a
// handle for the runtime, so the address a kernel can use is asked for once per device,
// with that device current.
uint32_t* noalloc_slots() {
  static uint32_t* addr[64] = {};
  static std::mutex mu;
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
    fail(B200K_CUDA_ERROR, "no current CUDA device");
    return nullptr;
  }
  std::lock_guard<std::mutex> lock(mu);
  if (addr[dev] == nullptr) {
    uint32_t* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_noalloc_amax);
    if (e != cudaSuccess || p == nullptr) {
      fail(B200K_CUDA_ERROR, "cudaGetSymbolAddress(scratch): %s", cudaGetErrorString(e));
      return nullptr;
    }
    addr[dev] = p;
  }
  return addr[dev];
}

int grid_for(int64_t work_items, int threads) {
  int sms = current_sm_count();
  if (sms <= 0) sms = 148;
  int64_t blocks = ceil_div(work_items, threads);
  int64_t cap = static_cast<int64_t>(sms) * 8;
  return static_cast<int>(blocks < cap ? (blocks > 0 ? blocks : 1) : cap);
}

}  // namespace
}  // namespace b200k

using namespace b200k;

extern "C" int b200k_mxfp8_quantize(const b200k_quantize_args* a, b200k_stream stream_) {
  if (a == nullptr) return fail(B200K_INVALID_ARG, "null args");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (a->rows < 0 || a->k < 0) return fail(B200K_INVALID_ARG, "negative dimension");
  if (a->rows == 0 || a->k == 0) return B200K_OK;
  if (!a->x || !a->q) return fail(B200K_INVALID_ARG, "null pointer");
  if (a->q_dtype != B200K_E4M3 && a->q_dtype != B200K_E5M2)
    return fail(B200K_INVALID_ARG, "q_dtype must be e4m3 or e5m2");
  if (a->sf_swizzled && (reinterpret_cast<uintptr_t>(a->sf_swizzled) % 16))
    return fail(B200K_UNSUPPORTED, "swizzled scale tensor must be 16-byte aligned");
  const int64_t kblocks = ceil_div(a->k, 32);
  if (a->sf_swizzled && a->sf_k_atoms < ceil_div(kblocks, 4))
    return fail(B200K_INVALID_ARG, "sf_k_atoms too small");
  const int e5m2 = a->q_dtype == B200K_E5M2;
  uint8_t* q = static_cast<uint8_t*>(a->q);
  uint8_t* sl = static_cast<uint8_t*>(a->sf_logical);
  uint8_t* ss = static_cast<uint8_t*>(a->sf_swizzled);
  const int gdiv = a->gather_divisor > 0 ? a->gather_divisor : 1;
  const int grid = grid_for(a->rows * kblocks, 256);
#define B200K_MXFP8_CASE(T)                                                                       \
  mxfp8_quantize_kernel<T><<<grid, 256, 0, stream>>>(                                             \
      static_cast<const T*>(a->x), a->rows, a->k, a->ldx, q, a->ldq, sl, ss, a->sf_k_atoms, e5m2, \
      a->gather_index, gdiv, a->src_rows, a->live_blocks, a->tile_m)
  switch (a->x_dtype) {
    case B200K_F32: B200K_MXFP8_CASE(float); break;
    case B200K_BF16: B200K_MXFP8_CASE(__nv_bfloat16); break;
    case B200K_F16: B200K_MXFP8_CASE(__half); break;
    default:
      return fail(B200K_INVALID_ARG, "x_dtype must be f32, bf16 or f16");
  }
#undef B200K_MXFP8_CASE
  B200K_CHECK_LAUNCH("mxfp8_quantize launch");
  return B200K_OK;
}

extern "C" int b200k_sf_swizzle(const void* sf, int64_t rows, int64_t kblocks, int64_t ld,
                                void* out, int64_t k_atoms, int32_t fill, const int32_t* live_tiles,
                                int32_t live_tile_rows, b200k_stream stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (rows < 0 || kblocks < 0) return fail(B200K_INVALID_ARG, "negative dimension");
  if (rows == 0 || kblocks == 0) return B200K_OK;
  if (!sf || !out) return fail(B200K_INVALID_ARG, "null pointer");
  if (reinterpret_cast<uintptr_t>(out) % 16) return fail(B200K_UNSUPPORTED, "output must be 16-byte aligned");
  if (k_atoms < ceil_div(kblocks, 4)) return fail(B200K_INVALID_ARG, "k_atoms too small");
  const int64_t row_tiles = ceil_div(rows, 128);
  const int grid = grid_for(row_tiles * k_atoms * 32, 256);
  sf_swizzle_kernel<<<grid, 256, 0, stream>>>(static_cast<const uint8_t*>(sf), rows, kblocks, ld,
                                              static_cast<uint8_t*>(out), row_tiles, k_atoms, fill,
                                              live_tiles, live_tile_rows);
  B200K_CHECK_LAUNCH("sf_swizzle launch");
  return B200K_OK;
}

// Two blocks per thread when every access of the fast path is aligned.
template <typename T>
void launch_nvfp4_quantize(const b200k_quantize_args* a, const uint32_t* amax, cudaStream_t stream) {
  uint8_t* q = static_cast<uint8_t*>(a->q);
  uint8_t* sl = static_cast<uint8_t*>(a->sf_logical);
  uint8_t* ss = static_cast<uint8_t*>(a->sf_swizzled);
  const T* x = static_cast<const T*>(a->x);
  const int64_t kblocks = ceil_div(a->k, 16);
  const bool pairs = (a->k % 32 == 0) && (reinterpret_cast<uintptr_t>(x) % 16 == 0) &&
                     ((a->ldx * sizeof(T)) % 16 == 0) && (reinterpret_cast<uintptr_t>(q) % 16 == 0) &&
                     (a->ldq % 16 == 0) && (reinterpret_cast<uintptr_t>(sl) % 2 == 0) &&
                     (reinterpret_cast<uintptr_t>(ss) % 2 == 0);
  // (errors of these launches surface through the caller's cudaGetLastError check)
  if (pairs) {
    launch_after_predecessor(nvfp4_quantize_kernel<T, 2>, dim3(grid_for(a->rows * kblocks / 2, 256)), dim3(256), 0,
                             stream, x, a->rows, a->k, a->ldx, q, a->ldq, sl, ss, a->sf_k_atoms, amax,
                             a->tensor_scale);
  } else {
    launch_after_predecessor(nvfp4_quantize_kernel<T, 1>, dim3(grid_for(a->rows * kblocks, 256)), dim3(256), 0,
                             stream, x, a->rows, a->k, a->ldx, q, a->ldq, sl, ss, a->sf_k_atoms, amax,
                             a->tensor_scale);
  }
}

extern "C" int b200k_nvfp4_quantize(const b200k_quantize_args* a, b200k_stream stream_) {
  if (a == nullptr) return fail(B200K_INVALID_ARG, "null args");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (a->rows < 0 || a->k < 0) return fail(B200K_INVALID_ARG, "negative dimension");
  if (a->rows == 0 || a->k == 0) return B200K_OK;
  if (!a->x || !a->q || (!a->scratch && !a->tensor_scale_given))
    return fail(B200K_INVALID_ARG, "null pointer");
  if (a->tensor_scale_given && !a->tensor_scale)
    return fail(B200K_INVALID_ARG, "tensor_scale_given without tensor_scale");
  if (a->k % 2) return fail(B200K_UNSUPPORTED, "K must be even (two e2m1 values per byte)");
  const int64_t kblocks = ceil_div(a->k, 16);
  if (a->sf_swizzled && a->sf_k_atoms < ceil_div(kblocks, 4))
    return fail(B200K_INVALID_ARG, "sf_k_atoms too small");
  if (a->tensor_scale_given) {   // one pass: the scale is the caller's
    switch (a->x_dtype) {
      case B200K_F32: launch_nvfp4_quantize<float>(a, nullptr, stream); break;
      case B200K_BF16: launch_nvfp4_quantize<__nv_bfloat16>(a, nullptr, stream); break;
      case B200K_F16: launch_nvfp4_quantize<__half>(a, nullptr, stream); break;
      default: return fail(B200K_INVALID_ARG, "x_dtype must be f32, bf16 or f16");
    }
    B200K_CHECK_LAUNCH("nvfp4_quantize launch");
    return B200K_OK;
  }
  uint32_t* amax = static_cast<uint32_t*>(a->scratch);
  cudaError_t e = cudaMemsetAsync(amax, 0, sizeof(uint32_t), stream);
  if (e != cudaSuccess) return fail(B200K_CUDA_ERROR, "memset: %s", cudaGetErrorString(e));
  const int grid_r = grid_for(a->rows * a->k / 16, 256);
#define B200K_NVFP4_CASE(T)                                                                       \
  absmax_kernel<T><<<grid_r, 256, 0, stream>>>(static_cast<const T*>(a->x), a->rows, a->k, a->ldx, \
                                               amax);                                             \
  launch_nvfp4_quantize<T>(a, amax, stream)
  switch (a->x_dtype) {
    case B200K_F32: B200K_NVFP4_CASE(float); break;
    case B200K_BF16: B200K_NVFP4_CASE(__nv_bfloat16); break;
    case B200K_F16: B200K_NVFP4_CASE(__half); break;
    default: return fail(B200K_INVALID_ARG, "x_dtype must be f32, bf16 or f16");
  }
#undef B200K_NVFP4_CASE
  B200K_CHECK_LAUNCH("nvfp4_quantize launch");
  return B200K_OK;
}

extern "C" int b200k_nvfp4_quantize_noalloc(const b200k_quantize_args* a, b200k_stream stream_) {
  if (a == nullptr) return fail(B200K_INVALID_ARG, "null args");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (a->rows < 0 || a->k < 0) return fail(B200K_INVALID_ARG, "negative dimension");
  if (a->rows == 0 || a->k == 0) return B200K_OK;
  if (!a->x || !a->q) return fail(B200K_INVALID_ARG, "null pointer");
  if (a->k % 2) return fail(B200K_UNSUPPORTED, "K must be even (two e2m1 values per byte)");
  const int64_t kblocks = ceil_div(a->k, 16);
  if (a->sf_swizzled && a->sf_k_atoms < ceil_div(kblocks, 4))
    return fail(B200K_INVALID_ARG, "sf_k_atoms too small");
  if (a->tensor_scale_given) {
    // The scale is the caller's: there is no maximum to find, so the built-in scratch is
    // not touched and the size limit does not apply.  Same launch as b200k_nvfp4_quantize.
    if (!a->tensor_scale) return fail(B200K_INVALID_ARG, "tensor_scale_given without tensor_scale");
    switch (a->x_dtype) {
      case B200K_F32: launch_nvfp4_quantize<float>(a, nullptr, stream); break;
      case B200K_BF16: launch_nvfp4_quantize<__nv_bfloat16>(a, nullptr, stream); break;
      case B200K_F16: launch_nvfp4_quantize<__half>(a, nullptr, stream); break;
      default: return fail(B200K_INVALID_ARG, "x_dtype must be f32, bf16 or f16");
    }
    B200K_CHECK_LAUNCH("nvfp4_quantize_noalloc launch");
    return B200K_OK;
  }
  const int64_t slabs = ceil_div(a->rows * a->k, kNoAllocSlabElems);
  if (slabs > kNoAllocSlots)
    return fail(B200K_UNSUPPORTED,
                "tensor of %lld elements exceeds the built-in scratch of this entry point "
                "(%lld elements at most); use b200k_nvfp4_quantize with caller scratch",
                (long long)(a->rows * a->k), (long long)(kNoAllocSlots * kNoAllocSlabElems));
  uint32_t* slots = noalloc_slots();
  if (slots == nullptr) return B200K_CUDA_ERROR;
#define B200K_NVFP4_NOALLOC_CASE(T)                                                               \
  absmax_slab_kernel<T><<<static_cast<int>(slabs), 256, 0, stream>>>(                             \
      static_cast<const T*>(a->x), a->rows, a->k, a->ldx, slots);                                 \
  fold_slots_kernel<<<1, 256, 0, stream>>>(slots, static_cast<int>(slabs));                       \
  launch_nvfp4_quantize<T>(a, slots, stream)
  switch (a->x_dtype) {
    case B200K_F32: B200K_NVFP4_NOALLOC_CASE(float); break;
    case B200K_BF16: B200K_NVFP4_NOALLOC_CASE(__nv_bfloat16); break;
    case B200K_F16: B200K_NVFP4_NOALLOC_CASE(__half); break;
    default: return fail(B200K_INVALID_ARG, "x_dtype must be f32, bf16 or f16");
  }
#undef B200K_NVFP4_NOALLOC_CASE
  B200K_CHECK_LAUNCH("nvfp4_quantize_noalloc launch");
  return B200K_OK;
}
