// Pieces shared by the GEMM kernels: launch parameters, per-kind traits, the grouped tile
// raster and the row-chunk store of the epilogue.
#pragma once
#include "common.cuh"
#include "host.h"

namespace b200k {

constexpr int kBM = 128;
constexpr int kStages = 4;
constexpr int kGroupM = 8;
constexpr int kNumThreads = 192;
constexpr int kTmemCols = 512;

enum OutType : int { kOutF16 = 0, kOutBF16 = 1, kOutF32 = 2,
                     kOutMX8 = 3, /* e4m3 + swizzled ue8m0 scale per 32 columns (CTA-pair kernel) */
                     kOutNVF4 = 4 /* packed e2m1 + swizzled ue4m3 scale per 16 columns (CTA-pair kernel) */ };

struct GemmParams {
  void* c;
  int m, n, k;          // k in elements
  int batch;
  int64_t ldc;          // elements
  int64_t stride_c;     // elements
  int tiles_m, tiles_n;
  int k_iters;
  int k_tail_mmas;      // MMAs of the last k iteration (1..4)
  int pair_bn;          // CTA-pair kernel: tile width 256 (also when 0) or 128 (unscaled kinds)
  int b_mn;             // CTA-pair kernel: B stored (K, N), N contiguous
  int coalesce_store;   // store the tile through shared memory (set by the launchers from store_mode)
  int store_mode;       // host side only: 1 = direct stores, 0 or 2 = staged
  int split_k;          // > 1: `batch` counts (batch, split) pairs, each split owns k_per_split k-steps
  int k_per_split;
  uint32_t idesc;
  float alpha;
  const float* alpha_a;
  const float* alpha_b;
  // scale factors (swizzled atoms of 512 bytes)
  const uint8_t* sfa;
  const uint8_t* sfb;
  int sf_k_atoms;
  int sfb_row_tiles;    // 128-row tiles present in sfb (reads are clamped to it)
  int sfb_group_tiles;  // 128-row tiles of sfb per group (grouped CTA-pair kernel)
  int64_t stride_sfa, stride_sfb;
  // grouped mode
  const int* tile_group;
  const int* num_row_tiles;
  const int* row_map;
  const float* row_scale;
  int64_t c_rows;
  int epilogue;
  uint8_t* c_sf;        // kOutMX8 / kOutNVF4: swizzled scales of the output
  int c_sf_k_atoms;
  const float* c_scale; // kOutNVF4: the output's per-tensor scale (device scalar)
  int* status;
  // CTA-pair kernel: time budget of every pipeline wait, and the test hook of
  // b200k_gemm_config.withhold_arrival (1 = the arrival that opens a tile to the second MMA
  // issuer is never made, so that issuer's wait runs out of its budget)
  uint64_t wait_budget_ns;
  int withhold_arrival;
  int programmatic_launch;   // host side only: launch with programmatic stream serialisation
  int group_m;               // CTA-pair kernel: row tiles per raster band
  // CTA-pair kernel, grouped: output rows scattered over up to 16 buffers (peer-mapped or
  // local); row_map values are then buffer * c_peer_rows + row
  int skip_tile0;      // CTA-pair kernel, plain problems: 256-row tiles [skip_tile0, skip_tile0 +
  int skip_tiles;      // skip_tiles) of A and C take no part in the product
  int num_c_peers;
  int64_t c_peer_rows;
  void* c_peers[16];
};

template <int KIND>
struct KindTraits;
template <> struct KindTraits<kKindF16>  { static constexpr int kElemBits = 16; static constexpr bool kScaled = false; };
template <> struct KindTraits<kKindTF32> { static constexpr int kElemBits = 32; static constexpr bool kScaled = false; };
template <> struct KindTraits<kKindF8>   { static constexpr int kElemBits = 8;  static constexpr bool kScaled = false; };
template <> struct KindTraits<kKindMXF8> { static constexpr int kElemBits = 8;  static constexpr bool kScaled = true;
                                           static constexpr int kSfBlock = 32; };
template <> struct KindTraits<kKindNVF4> { static constexpr int kElemBits = 4;  static constexpr bool kScaled = true;
                                           static constexpr int kSfBlock = 16; };

template <int KIND, int BN, bool B_MN>
struct GemmCfg {
  using T = KindTraits<KIND>;
  static constexpr int kBKElems = 128 * 8 / T::kElemBits;  // K elements per stage
  static constexpr int kMmaK = kBKElems / 4;               // 32 bytes of K per MMA
  static constexpr int kABytes = kBM * 128;
  static constexpr int kBBytes = BN * 128;
  // MN-major B: boxes of (128 bytes of N) x (kBKElems rows of K)
  static constexpr int kBBoxN = 128 * 8 / T::kElemBits;    // N elements per 128-byte row
  static constexpr int kBBoxBytes = kBKElems * 128;
  static constexpr int kBBoxes = B_MN ? BN / kBBoxN : BN / 128;
  static constexpr bool kScaled = T::kScaled;
  static constexpr int kSfaAtoms = kScaled ? (KIND == kKindNVF4 ? 4 : 1) : 0;  // per stage
  static constexpr int kSfbAtoms = kSfaAtoms * (BN / 128);
  static constexpr int kSfBytes = (kSfaAtoms + kSfbAtoms) * 512;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kNumAcc = kScaled ? 1 : (BN <= 256 ? 512 / 256 : 1);
  static constexpr int kAccStride = 256;
  static constexpr int kSfTmemBase = 256;
  static constexpr int kSfaCols = kSfaAtoms * 4;
  static constexpr int kSfbCols = kSfbAtoms * 4;
  // epilogue staging (32 rows x 128 bytes per warp) where shared memory has room for it
  static constexpr int kStagingBytes = (KIND == kKindNVF4) ? 0 : 4 * 4096;
  static constexpr int kSmemBytes =
      1024 /*alignment slack*/ + kStages * (kStageBytes + kSfBytes) + 256 /*barriers*/ + kStagingBytes;
  static_assert(!kScaled || kSfTmemBase + kStages * (kSfaCols + kSfbCols) <= kTmemCols,
                "scale factors do not fit in tensor memory");
  static_assert(!(B_MN && KIND == kKindNVF4), "fp4 operands are K-major only");
};

// x * sigmoid(x) with the fast exponential and reciprocal (two special-function ops): the
// result is rounded to 16 bits or quantised right after, and an IEEE division per element
// made the SwiGLU epilogue longer than the mainloop of a 32-k-step tile.
__device__ __forceinline__ float silu(float x) { return __fdividef(x, 1.0f + __expf(-x)); }

struct TileCoord {
  int batch, pid_m, pid_n;
};

// Grouped raster order: consecutive tile ids walk `group_m` row tiles before moving to
// the next column tile, which keeps a band of A and one B tile hot in L2 (the reference's
// GROUP_SIZE_M = 8, test/kernels/matmul.py:13-23; here the band height is a launch parameter,
// chosen from the operand sizes: see pick_group_m).
__device__ __forceinline__ TileCoord tile_coord(int tile, int tiles_m, int tiles_n, int group_m = kGroupM) {
  int per_batch = tiles_m * tiles_n;
  TileCoord c;
  c.batch = tile / per_batch;
  int t = tile - c.batch * per_batch;
  int group_tiles = group_m * tiles_n;
  int group = t / group_tiles;
  int first_m = group * group_m;
  int rows = min(group_m, tiles_m - first_m);
  int in_group = t - group * group_tiles;
  c.pid_m = first_m + in_group % rows;
  c.pid_n = in_group / rows;
  return c;
}

// Band height of the raster for the CTA-pair kernel: as many 256-row tiles of A as fit a
// quarter of the L2 (with their scale factors), at least the reference's 8.  Every band
// re-reads B once, so a taller band cuts B's traffic from DRAM: NVFP4 8192 x 28672 x 8192
// holds all of A (36 MB) and reads B once instead of four times.
inline int pick_group_m(int64_t m, int64_t a_row_bytes, int forced) {
  if (forced > 0) return forced;
  const int64_t tile_bytes = 256 * a_row_bytes;
  const int64_t budget = 40ll << 20;
  int64_t g = tile_bytes > 0 ? budget / tile_bytes : kGroupM;
  if (g < kGroupM) g = kGroupM;
  const int64_t tiles_m = (m + 255) / 256;
  if (g >= tiles_m) return static_cast<int>(tiles_m > 0 ? tiles_m : 1);
  const int64_t bands = (tiles_m + g - 1) / g;      // bands of equal height
  g = (tiles_m + bands - 1) / bands;
  return static_cast<int>(g);
}

template <int OUT>
__device__ __forceinline__ void store_row_chunk(void* c_row, int col0, int n_limit,
                                                const float (&v)[32], bool vec_ok) {
  // 32 consecutive output columns of one row, starting at col0.
  if constexpr (OUT == kOutF32) {
    float* dst = static_cast<float*>(c_row) + col0;
    if (vec_ok && col0 + 32 <= n_limit) {
#pragma unroll
      for (int i = 0; i < 8; ++i)
        reinterpret_cast<float4*>(dst)[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
    } else {
#pragma unroll
      for (int i = 0; i < 32; ++i)
        if (col0 + i < n_limit) dst[i] = v[i];
    }
  } else {
    uint16_t* dst = static_cast<uint16_t*>(c_row) + col0;
    if (vec_ok && col0 + 32 <= n_limit) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        uint4 q;
        if constexpr (OUT == kOutBF16) {
          q.x = pack_bf16x2(v[8 * i + 0], v[8 * i + 1]);
          q.y = pack_bf16x2(v[8 * i + 2], v[8 * i + 3]);
          q.z = pack_bf16x2(v[8 * i + 4], v[8 * i + 5]);
          q.w = pack_bf16x2(v[8 * i + 6], v[8 * i + 7]);
        } else {
          q.x = pack_f16x2(v[8 * i + 0], v[8 * i + 1]);
          q.y = pack_f16x2(v[8 * i + 2], v[8 * i + 3]);
          q.z = pack_f16x2(v[8 * i + 4], v[8 * i + 5]);
          q.w = pack_f16x2(v[8 * i + 6], v[8 * i + 7]);
        }
        reinterpret_cast<uint4*>(dst)[i] = q;
      }
    } else {
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        if (col0 + i < n_limit) {
          if constexpr (OUT == kOutBF16) {
            __nv_bfloat16 h = __float2bfloat16_rn(v[i]);
            dst[i] = *reinterpret_cast<uint16_t*>(&h);
          } else {
            __half h = __float2half_rn(v[i]);
            dst[i] = *reinterpret_cast<uint16_t*>(&h);
          }
        }
      }
    }
  }
}

}  // namespace b200k
