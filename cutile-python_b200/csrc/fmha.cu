// Flash-attention forward for sm_100a: S = Q K^T and O += P V on tcgen05 with S, P and O
// in tensor memory, online softmax in the exp2 domain.
//
// One CTA owns one 128-row query tile of one (batch, head) and walks its key/value
// tiles of 128 rows; two CTAs share an SM (96 KB of shared memory and 256 TMEM columns
// each), so one CTA's softmax overlaps the other's MMAs.
//
//   warp 0      TMA producer (one lane): Q once, then K_j and V_j
//   warp 1      MMA issuer (one lane): S_j = Q K_j^T, then O += P_j V_j
//   warps 2..5  softmax: one query row per thread (TMEM lane), P written back to TMEM
//               as 16-bit pairs over S, O rescaled in TMEM only when the row maximum
//               grew by more than 2^8 (exact: the deferred factor cancels in O / l)
//
// Semantics follow fmha_kernel (reference: test/kernels/attention.py:20-128): scores
// scaled by qk_scale * log2(e), causal mask with query positions offset by input_pos,
// out-of-range keys masked, fp32 running max / sum, P rounded to the input type before
// P V, output = accumulator / sum rounded to the input type, grouped-query heads by
// integer division.
#include <stdlib.h>

#include "common.cuh"
#include "fmha_decode.h"
#include "host.h"

namespace b200k {

constexpr int kFmhaBM = 128;
constexpr int kFmhaBN = 128;
constexpr int kFmhaThreads = 192;
constexpr int kFmhaTmemCols = 256;
constexpr float kRescaleThreshold = 8.0f;  // log2 units

struct FmhaParams {
  void* out;
  int64_t o_stride_b, o_stride_h, o_stride_s;  // elements
  int batch, heads_q, heads_kv, group;
  int sq, sk;
  int q_tiles;
  float scale_log2;
  int causal;
  int input_pos;
  int* status;
};

__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float r;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
}

// Every kFmhaPolyEvery-th pair of scores takes its exp2 on the FMA pipe (a degree-3
// polynomial after splitting off the integer part) instead of the special-function unit,
// which is the busiest pipe of the softmax.  Relative error 7.5e-5, far below the rounding
// of P to 16 bits.  0 disables the polynomial path.
#ifndef B200K_FMHA_POLY
#define B200K_FMHA_POLY 4
#endif
constexpr int kFmhaPolyEvery = B200K_FMHA_POLY;

__device__ __forceinline__ float2 exp2_poly_pair(float2 x) {
  const float2 magic = make_float2(12582912.0f, 12582912.0f);       // 1.5 * 2^23
  const float2 neg_magic = make_float2(-12582912.0f, -12582912.0f);
  x.x = fmaxf(x.x, -125.0f);
  x.y = fmaxf(x.y, -125.0f);
  const float2 t = __fadd2_rn(x, magic);            // integer part lands in the low mantissa bits
  const float2 i = __fadd2_rn(t, neg_magic);
  const float2 f = __fadd2_rn(x, make_float2(-i.x, -i.y));   // in [-0.5, 0.5]
  float2 p = __ffma2_rn(make_float2(0.05517164617776871f, 0.05517164617776871f), f,
                        make_float2(0.2426111251115799f, 0.2426111251115799f));
  p = __ffma2_rn(p, f, make_float2(0.6932609677314758f, 0.6932609677314758f));
  p = __ffma2_rn(p, f, make_float2(0.9999280571937561f, 0.9999280571937561f));
  float2 r;
  r.x = __int_as_float(__float_as_int(p.x) + (__float_as_int(t.x) << 23));
  r.y = __int_as_float(__float_as_int(p.y) + (__float_as_int(t.y) << 23));
  return r;
}

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// One softmax warp group (4 warps, one query row per thread) working on the 128-row query
// tile that starts at row q0 of (batch b, head h): for each of its n_kv key tiles it reads S
// from tensor memory, updates the running maximum / sum, writes P back over S as 16-bit
// pairs, rescales O when needed, and finally writes O / l.
template <int D, bool BF16>
__device__ __forceinline__ void softmax_tile(const FmhaParams& p, int warp, int lane, int b, int h,
                                             int q0, int n_kv, uint32_t tmem_s, uint32_t tmem_o,
                                             uint32_t s_full, uint32_t p_half, uint32_t p_full,
                                             uint32_t pv_done, volatile int* abort_flag) {
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    const uint32_t lane_addr = uint32_t(quarter * 32) << 16;
    const int q_pos = p.input_pos + q0 + row;
    float m_used = -INFINITY;
    float l = 0.0f;
    bool ok = true;
    for (int j = 0; j < n_kv; ++j) {
      const uint32_t ph = j & 1;
      if (!mbar_wait(s_full, ph, abort_flag)) {
        report_status(p.status, 31, j);
        *abort_flag = 1;
        ok = false;
        break;
      }
      tc_fence_after_sync();
      float s[128];
      {
        uint32_t r[128];
        tmem_ld_32x32b_x128(tmem_s + lane_addr, r);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 128; ++i) s[i] = __uint_as_float(r[i]);
      }
      const int key0 = j * kFmhaBN;
      const bool need_mask = (key0 + kFmhaBN > p.sk) || (p.causal && key0 + kFmhaBN - 1 > p.input_pos + q0);
      if (need_mask) {
        const int limit = p.causal ? min(p.sk - 1, q_pos) : p.sk - 1;  // last visible key
#pragma unroll
        for (int i = 0; i < 128; ++i)
          if (key0 + i > limit) s[i] = -INFINITY;
      }
      // three-input max, eight independent chains of 16 scores
      float mx8[8];
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        float m = fmax3(s[16 * c], s[16 * c + 1], s[16 * c + 2]);
#pragma unroll
        for (int i = 3; i < 15; i += 2) m = fmax3(m, s[16 * c + i], s[16 * c + i + 1]);
        mx8[c] = fmaxf(m, s[16 * c + 15]);
      }
      const float mx = fmax3(fmax3(mx8[0], mx8[1], mx8[2]), fmax3(mx8[3], mx8[4], mx8[5]),
                             fmaxf(mx8[6], mx8[7]));
      const float m_new = fmaxf(m_used, mx * p.scale_log2);
      // Deferred rescale: keep the stale maximum while the true one is less than 2^8
      // above it.  A row whose maximum is still -inf has seen no key yet.
      bool grow = (m_new - m_used > kRescaleThreshold) || (m_used == -INFINITY && m_new > -INFINITY);
      const bool any_grow = __any_sync(0xffffffffu, grow);
      float alpha = 1.0f;
      if (grow) {
        alpha = (m_used == -INFINITY) ? 0.0f : fast_exp2(m_used - m_new);
        m_used = m_new;
      }
      if (any_grow && j > 0) {
        // S_FULL of tile j was committed after P V of tile j-1, so O is quiescent here
        l *= alpha;
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          uint32_t r[32];
          tmem_ld_32x32b_x32(tmem_o + lane_addr + c * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
          tmem_st_32x32b_x32(tmem_o + lane_addr + c * 32, r);
        }
      }
      const float neg_m = (m_used == -INFINITY) ? 0.0f : -m_used;
      // packed fp32 pairs: one FFMA2 scales and shifts two scores, one FADD2 adds two
      // probabilities into the running sums
      const float2 scale2 = make_float2(p.scale_log2, p.scale_log2);
      const float2 negm2 = make_float2(neg_m, neg_m);
      float2 sum2[4] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f), make_float2(0.f, 0.f),
                        make_float2(0.f, 0.f)};
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t pk[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const float2 x = __ffma2_rn(make_float2(s[c * 64 + 2 * i], s[c * 64 + 2 * i + 1]), scale2, negm2);
          const bool poly = kFmhaPolyEvery > 0 && (i % (kFmhaPolyEvery > 0 ? kFmhaPolyEvery : 1)) == kFmhaPolyEvery - 1;
          const float2 e = poly ? exp2_poly_pair(x) : make_float2(fast_exp2(x.x), fast_exp2(x.y));
          sum2[i & 3] = __fadd2_rn(sum2[i & 3], e);
          pk[i] = BF16 ? pack_bf16x2(e.x, e.y) : pack_f16x2(e.x, e.y);
        }
        tmem_st_32x32b_x32(tmem_s + lane_addr + c * 32, pk);
        if (c == 0 && p_half != 0) {
          // the first 64 keys of P are enough for the first half of P V
          tmem_st_wait();
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(p_half);
        }
      }
      l += ((sum2[0].x + sum2[0].y) + (sum2[1].x + sum2[1].y)) +
           ((sum2[2].x + sum2[2].y) + (sum2[3].x + sum2[3].y));
      tmem_st_wait();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full);
    }
    // epilogue: O / l
    if (ok && n_kv > 0) {
      if (!mbar_wait(pv_done, (n_kv - 1) & 1, abort_flag)) {
        report_status(p.status, 32, 0);
        *abort_flag = 1;
        ok = false;
      }
    }
    tc_fence_after_sync();
    const bool row_ok = (q0 + row) < p.sq;
    uint16_t* o_row = static_cast<uint16_t*>(p.out) + b * p.o_stride_b + h * p.o_stride_h +
                      static_cast<int64_t>(q0 + row) * p.o_stride_s;
    const bool vec_ok = (reinterpret_cast<uintptr_t>(p.out) % 16 == 0) && (p.o_stride_b % 8 == 0) &&
                        (p.o_stride_h % 8 == 0) && (p.o_stride_s % 8 == 0);
    const float inv_l = (l > 0.0f) ? __fdividef(1.0f, l) : 0.0f;
#pragma unroll
    for (int c = 0; c < D / 32; ++c) {
      uint32_t r[32];
      if (ok && n_kv > 0) {
        tmem_ld_32x32b_x32(tmem_o + lane_addr + c * 32, r);
        tmem_ld_wait();
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) r[i] = 0;
      }
      if (row_ok) {
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const float a = __uint_as_float(r[2 * i]) * inv_l;
          const float c2 = __uint_as_float(r[2 * i + 1]) * inv_l;
          pk[i] = BF16 ? pack_bf16x2(a, c2) : pack_f16x2(a, c2);
        }
        if (vec_ok) {
#pragma unroll
          for (int i = 0; i < 4; ++i)
            reinterpret_cast<uint4*>(o_row + c * 32)[i] = make_uint4(pk[4 * i], pk[4 * i + 1], pk[4 * i + 2], pk[4 * i + 3]);
        } else {
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            o_row[c * 32 + 2 * i] = static_cast<uint16_t>(pk[i] & 0xffff);
            o_row[c * 32 + 2 * i + 1] = static_cast<uint16_t>(pk[i] >> 16);
          }
        }
      }
    }
}

template <int D, bool BF16>
__global__ void __launch_bounds__(kFmhaThreads, 2)
fmha_fwd_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                const __grid_constant__ CUtensorMap tmap_v, const FmhaParams p) {
  constexpr int kBoxes = D / 64;            // 64-element (128-byte) slices of the head dim
  constexpr int kTileBytes = 128 * D * 2;   // Q, K or V tile
  constexpr int kBoxBytes = 128 * 128;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t q_smem = base;
  const uint32_t k_smem = base + kTileBytes;
  const uint32_t v_smem = base + 2 * kTileBytes;
  uint8_t* tail = smem + 3 * kTileBytes;
  const uint32_t bar0 = smem_u32(tail);
  // barriers: q_full, k_full, k_empty, v_full, v_empty, s_full, p_full, pv_done
  enum { Q_FULL = 0, K_FULL, K_EMPTY, V_FULL, V_EMPTY, S_FULL, P_FULL, PV_DONE, NUM_BARS };
  auto bar = [&](int i) { return bar0 + 8u * i; };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tail + 8 * NUM_BARS);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tail + 8 * NUM_BARS + 8);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  // tile assignment: (batch, head) major, query tiles from the last (most keys under a
  // causal mask) to the first
  const int bh = blockIdx.x / p.q_tiles;
  const int qt = p.q_tiles - 1 - (blockIdx.x - bh * p.q_tiles);
  const int b = bh / p.heads_q;
  const int h = bh - b * p.heads_q;
  const int h_kv = h / p.group;
  const int q0 = qt * kFmhaBM;

  int n_kv = (p.sk + kFmhaBN - 1) / kFmhaBN;
  if (p.causal) {
    const int last_key = p.input_pos + q0 + kFmhaBM - 1;  // largest visible key index
    n_kv = min(n_kv, max(0, last_key / kFmhaBN + 1));
  }

  if (threadIdx.x == 0) {
    for (int i = 0; i < NUM_BARS; ++i) mbar_init(bar(i), i == P_FULL ? 4 : 1);
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmap_q);
    tma_prefetch_desc(&tmap_k);
    tma_prefetch_desc(&tmap_v);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), kFmhaTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_s = tmem_base;          // S: 128 columns; P aliases its first 64
  const uint32_t tmem_o = tmem_base + 128;    // O: D columns

  constexpr uint32_t kFmt = BF16 ? kFmtBF16 : kFmtF16;

  if (warp == 0) {
    // warp-uniform loop (addresses and coordinates stay in uniform registers), one elected
    // lane issues
    if (n_kv > 0) {
      const bool elected = elect_one();
      if (elected) {
        mbar_arrive_expect_tx(bar(Q_FULL), kTileBytes);
#pragma unroll
        for (int i = 0; i < kBoxes; ++i)
          tma_load_4d(q_smem + i * kBoxBytes, &tmap_q, bar(Q_FULL), i * 64, q0, h, b);
      }
      for (int j = 0; j < n_kv; ++j) {
        const uint32_t ph = j & 1;
        if (!mbar_wait(bar(K_EMPTY), ph ^ 1, abort_flag)) {
          report_status(p.status, 11, j);
          *abort_flag = 1;
          break;
        }
        if (elected) {
          mbar_arrive_expect_tx(bar(K_FULL), kTileBytes);
#pragma unroll
          for (int i = 0; i < kBoxes; ++i)
            tma_load_4d(k_smem + i * kBoxBytes, &tmap_k, bar(K_FULL), i * 64, j * kFmhaBN, h_kv, b);
        }
        if (!mbar_wait(bar(V_EMPTY), ph ^ 1, abort_flag)) {
          report_status(p.status, 12, j);
          *abort_flag = 1;
          break;
        }
        if (elected) {
          mbar_arrive_expect_tx(bar(V_FULL), kTileBytes);
#pragma unroll
          for (int i = 0; i < kBoxes; ++i)
            tma_load_4d(v_smem + i * kBoxBytes, &tmap_v, bar(V_FULL), i * 64, j * kFmhaBN, h_kv, b);
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (n_kv > 0) {
      const bool elected = elect_one();
      constexpr uint32_t idesc_qk = make_idesc(kFmt, kFmt, false, false, kFmhaBM, kFmhaBN);
      constexpr uint32_t idesc_pv = make_idesc(kFmt, kFmt, false, true, kFmhaBM, D);
      bool ok = mbar_wait(bar(Q_FULL), 0, abort_flag);
      if (!ok) {
        report_status(p.status, 20, 0);
        *abort_flag = 1;
      }
      for (int j = 0; j < n_kv && ok; ++j) {
        const uint32_t ph = j & 1;
        if (!mbar_wait(bar(K_FULL), ph, abort_flag)) {
          report_status(p.status, 21, j);
          *abort_flag = 1;
          break;
        }
        tc_fence_after_sync();
        // S = Q K^T: both operands K-major, 16 elements (32 bytes) of the head dim per MMA
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (kk / 4) * kBoxBytes;
          const uint64_t qd = make_smem_desc(q_smem + off, 16, 1024, kSwizzle128B) + 2 * (kk % 4);
          const uint64_t kd = make_smem_desc(k_smem + off, 16, 1024, kSwizzle128B) + 2 * (kk % 4);
          if (elected) umma<kKindF16>(tmem_s, qd, kd, idesc_qk, kk > 0 ? 1u : 0u);
        }
        if (elected) {
          tc_commit(bar(K_EMPTY));
          tc_commit(bar(S_FULL));
        }
        if (!mbar_wait(bar(P_FULL), ph, abort_flag)) {
          report_status(p.status, 22, j);
          *abort_flag = 1;
          break;
        }
        if (!mbar_wait(bar(V_FULL), ph, abort_flag)) {
          report_status(p.status, 23, j);
          *abort_flag = 1;
          break;
        }
        tc_fence_after_sync();
        // O += P V: P from tensor memory (8 columns of 16-bit pairs per MMA), V is
        // (keys, D) with D contiguous = MN-major B: 16 key rows of 128 bytes per MMA,
        // the 64-element slices of D one tile apart
#pragma unroll
        for (int kk = 0; kk < kFmhaBN / 16; ++kk) {
          const uint64_t vd = make_smem_desc(v_smem + kk * 2048, kBoxBytes, 1024, kSwizzle128B);
          if (elected) umma_f16_ts(tmem_o, tmem_s + kk * 8, vd, idesc_pv, (j > 0 || kk > 0) ? 1u : 0u);
        }
        if (elected) {
          tc_commit(bar(V_EMPTY));
          tc_commit(bar(PV_DONE));
        }
      }
    }
    __syncwarp();
  } else {
    softmax_tile<D, BF16>(p, warp, lane, b, h, q0, n_kv, tmem_s, tmem_o, bar(S_FULL), 0u, bar(P_FULL),
                          bar(PV_DONE), abort_flag);
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, kFmhaTmemCols);
  }
}

// ---------------------------------------------------------------------------
// Two query tiles per CTA (head dim 128): one CTA per SM owns 256 query rows.  Warp group A
// (warps 2-5) does the softmax of rows [q0, q0 + 128), warp group B (warps 6-9) of rows
// [q0 + 128, q0 + 256); the single MMA thread interleaves their matrix products
//     P V (A, j)   S (A, j + 1)   P V (B, j)   S (B, j + 1)
// so that while one group is in its softmax the tensor core works for the other.  K and V
// tiles are double-buffered and shared by both query tiles.
// TMEM: S_A [0,128)  S_B [128,256)  O_A [256,384)  O_B [384,512); P aliases S.
// ---------------------------------------------------------------------------
constexpr int kFmha2Threads = 320;   // TMA warp, MMA warp, 2 x 4 softmax warps

template <bool BF16>
__global__ void __launch_bounds__(kFmha2Threads, 1)
fmha_fwd_pair_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                     const __grid_constant__ CUtensorMap tmap_v, const FmhaParams p) {
  constexpr int D = 128;
  constexpr int kTileBytes = 128 * D * 2;
  constexpr int kBoxBytes = 128 * 128;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t q_smem = base;                          // Q_A, Q_B
  const uint32_t k_smem = base + 2 * kTileBytes;         // K[2]
  const uint32_t v_smem = base + 4 * kTileBytes;         // V[2]
  uint8_t* tail = smem + 6 * kTileBytes;
  const uint32_t bar0 = smem_u32(tail);
  enum { Q_FULL = 0, K_FULL = 1, K_EMPTY = 3, V_FULL = 5, V_EMPTY = 7, S_FULL = 9, P_FULL = 11,
         PV_DONE = 13, P_HALF = 15, NUM_BARS = 17 };
  auto bar = [&](int i) { return bar0 + 8u * i; };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tail + 8 * NUM_BARS);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tail + 8 * NUM_BARS + 8);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  const int q_pairs = (p.sq + 255) / 256;
  const int bh = blockIdx.x / q_pairs;
  const int qp = q_pairs - 1 - (blockIdx.x - bh * q_pairs);   // heaviest (causal) tiles first
  const int b = bh / p.heads_q;
  const int h = bh - b * p.heads_q;
  const int h_kv = h / p.group;
  const int q0 = qp * 256;

  // key tiles per query tile
  const int kv_all = (p.sk + kFmhaBN - 1) / kFmhaBN;
  int n_x[2];
#pragma unroll
  for (int x = 0; x < 2; ++x) {
    const int qx = q0 + x * 128;
    int n = kv_all;
    if (p.causal) n = min(n, (p.input_pos + qx + kFmhaBM - 1) / kFmhaBN + 1);
    if (qx >= p.sq) n = 0;
    n_x[x] = n;
  }
  const int n_kv = max(n_x[0], n_x[1]);

  if (threadIdx.x == 0) {
    for (int i = 0; i < NUM_BARS; ++i)
      mbar_init(bar(i), (i == P_FULL || i == P_FULL + 1 || i == P_HALF || i == P_HALF + 1) ? 4 : 1);
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmap_q);
    tma_prefetch_desc(&tmap_k);
    tma_prefetch_desc(&tmap_v);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  constexpr uint32_t kFmt = BF16 ? kFmtBF16 : kFmtF16;

  if (warp == 0) {
    if (n_kv > 0) {
      const bool elected = elect_one();
      if (elected) {
        mbar_arrive_expect_tx(bar(Q_FULL), 2 * kTileBytes);
#pragma unroll
        for (int x = 0; x < 2; ++x)
#pragma unroll
          for (int i = 0; i < 2; ++i)
            tma_load_4d(q_smem + x * kTileBytes + i * kBoxBytes, &tmap_q, bar(Q_FULL), i * 64, q0 + x * 128, h, b);
      }
      for (int j = 0; j < n_kv; ++j) {
        const int st = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (!mbar_wait(bar(K_EMPTY + st), ph ^ 1, abort_flag)) {
          report_status(p.status, 61, j);
          *abort_flag = 1;
          break;
        }
        if (elected) {
          mbar_arrive_expect_tx(bar(K_FULL + st), kTileBytes);
#pragma unroll
          for (int i = 0; i < 2; ++i)
            tma_load_4d(k_smem + st * kTileBytes + i * kBoxBytes, &tmap_k, bar(K_FULL + st), i * 64,
                        j * kFmhaBN, h_kv, b);
        }
        if (!mbar_wait(bar(V_EMPTY + st), ph ^ 1, abort_flag)) {
          report_status(p.status, 62, j);
          *abort_flag = 1;
          break;
        }
        if (elected) {
          mbar_arrive_expect_tx(bar(V_FULL + st), kTileBytes);
#pragma unroll
          for (int i = 0; i < 2; ++i)
            tma_load_4d(v_smem + st * kTileBytes + i * kBoxBytes, &tmap_v, bar(V_FULL + st), i * 64,
                        j * kFmhaBN, h_kv, b);
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (n_kv > 0) {
      const bool elected = elect_one();
      constexpr uint32_t idesc_qk = make_idesc(kFmt, kFmt, false, false, kFmhaBM, kFmhaBN);
      constexpr uint32_t idesc_pv = make_idesc(kFmt, kFmt, false, true, kFmhaBM, D);
      // S_x = Q_x K^T for key tile j (stage st): 8 MMAs of K = 16
      auto issue_s = [&](int x, int st) {
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (kk / 4) * kBoxBytes;
          const uint64_t qd = make_smem_desc(q_smem + x * kTileBytes + off, 16, 1024, kSwizzle128B) + 2 * (kk % 4);
          const uint64_t kd = make_smem_desc(k_smem + st * kTileBytes + off, 16, 1024, kSwizzle128B) + 2 * (kk % 4);
          if (elected) umma<kKindF16>(tmem_base + x * 128, qd, kd, idesc_qk, kk > 0 ? 1u : 0u);
        }
        if (elected) tc_commit(bar(S_FULL + x));
      };
      // O_x += P_x V for key tile j: P from TMEM, V MN-major
      // `half` 0: keys 0..63 of the tile, 1: keys 64..127 (and the completion signal)
      auto issue_pv = [&](int x, int st, bool first, int half) {
#pragma unroll
        for (int k4 = 0; k4 < kFmhaBN / 32; ++k4) {
          const int kk = half * (kFmhaBN / 32) + k4;
          const uint64_t vd = make_smem_desc(v_smem + st * kTileBytes + kk * 2048, kBoxBytes, 1024, kSwizzle128B);
          if (elected)
            umma_f16_ts(tmem_base + 256 + x * 128, tmem_base + x * 128 + kk * 8, vd, idesc_pv,
                        (!first || kk > 0) ? 1u : 0u);
        }
        if (half == 1 && elected) tc_commit(bar(PV_DONE + x));
      };
      bool ok = mbar_wait(bar(Q_FULL), 0, abort_flag);
      if (ok) ok = mbar_wait(bar(K_FULL), 0, abort_flag);
      if (!ok) {
        report_status(p.status, 70, 0);
        *abort_flag = 1;
      } else {
        tc_fence_after_sync();
        if (n_x[0] > 0) issue_s(0, 0);
        if (n_x[1] > 0) issue_s(1, 0);
        if (elected) tc_commit(bar(K_EMPTY));
      }
      for (int j = 0; j < n_kv && ok; ++j) {
        const int st = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        const bool more = j + 1 < n_kv;
        const int st1 = (j + 1) & 1;
        const uint32_t ph1 = ((j + 1) >> 1) & 1;
        if (!mbar_wait(bar(V_FULL + st), ph, abort_flag)) {
          report_status(p.status, 71, j);
          *abort_flag = 1;
          break;
        }
        if (more && !mbar_wait(bar(K_FULL + st1), ph1, abort_flag)) {
          report_status(p.status, 72, j);
          *abort_flag = 1;
          break;
        }
#pragma unroll
        for (int x = 0; x < 2; ++x) {
          if (j < n_x[x]) {
            if (!mbar_wait(bar(P_HALF + x), j & 1, abort_flag)) {
              report_status(p.status, 75 + x, j);
              *abort_flag = 1;
              ok = false;
              break;
            }
            tc_fence_after_sync();
            issue_pv(x, st, j == 0, 0);
            if (!mbar_wait(bar(P_FULL + x), j & 1, abort_flag)) {
              report_status(p.status, 73 + x, j);
              *abort_flag = 1;
              ok = false;
              break;
            }
            tc_fence_after_sync();
            issue_pv(x, st, j == 0, 1);
          }
          if (more && j + 1 < n_x[x]) issue_s(x, st1);
        }
        if (!ok) break;
        if (elected) {
          tc_commit(bar(V_EMPTY + st));
          if (more) tc_commit(bar(K_EMPTY + st1));
        }
      }
    }
    __syncwarp();
  } else {
    const int x = (warp - 2) >> 2;           // warp group: query tile A (warps 2-5) or B (6-9)
    softmax_tile<D, BF16>(p, warp, lane, b, h, q0 + x * 128, n_x[x], tmem_base + x * 128,
                          tmem_base + 256 + x * 128, bar(S_FULL + x), bar(P_HALF + x), bar(P_FULL + x),
                          bar(PV_DONE + x), abort_flag);
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
}

namespace {

template <int D, bool BF16>
int launch_fmha(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
                const FmhaParams& p, int grid, cudaStream_t stream) {
  constexpr int kSmem = 1024 + 3 * 128 * D * 2 + 128;
  auto kernel = fmha_fwd_kernel<D, BF16>;
  static bool configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem);
    if (e != cudaSuccess)
      return fail(B200K_CUDA_ERROR, "cudaFuncSetAttribute(%d): %s", kSmem, cudaGetErrorString(e));
    configured[dev] = true;
  }
  kernel<<<grid, kFmhaThreads, kSmem, stream>>>(tq, tk, tv, p);
  B200K_CHECK_LAUNCH("fmha launch");
  return B200K_OK;
}

template <bool BF16>
int launch_fmha_pair(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
                     const FmhaParams& p, int grid, cudaStream_t stream) {
  constexpr int kSmem = 1024 + 6 * 128 * 128 * 2 + 256;
  auto kernel = fmha_fwd_pair_kernel<BF16>;
  static bool configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem);
    if (e != cudaSuccess)
      return fail(B200K_CUDA_ERROR, "cudaFuncSetAttribute(%d): %s", kSmem, cudaGetErrorString(e));
    configured[dev] = true;
  }
  kernel<<<grid, kFmha2Threads, kSmem, stream>>>(tq, tk, tv, p);
  B200K_CHECK_LAUNCH("fmha (two-tile) launch");
  return B200K_OK;
}

}  // namespace
}  // namespace b200k

using namespace b200k;

extern "C" int b200k_fmha_fwd(const b200k_fmha_args* a, b200k_stream stream_) {
  if (a == nullptr) return fail(B200K_INVALID_ARG, "null args");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (a->batch < 0 || a->heads_q < 0 || a->heads_kv <= 0 || a->seq_q < 0 || a->seq_kv < 0)
    return fail(B200K_INVALID_ARG, "negative dimension");
  if (a->batch == 0 || a->heads_q == 0 || a->seq_q == 0) return B200K_OK;
  if (!a->q || !a->k || !a->v || !a->out) return fail(B200K_INVALID_ARG, "null pointer");
  if (a->seq_kv == 0) return fail(B200K_UNSUPPORTED, "attention over zero keys is undefined");
  if (a->head_dim != 64 && a->head_dim != 128)
    return fail(B200K_UNSUPPORTED, "head_dim must be 64 or 128 (got %d)", a->head_dim);
  if (a->dtype != B200K_F16 && a->dtype != B200K_BF16)
    return fail(B200K_INVALID_ARG, "dtype must be f16 or bf16");
  if (a->query_group_size <= 0 || a->heads_kv * a->query_group_size != a->heads_q)
    return fail(B200K_INVALID_ARG, "heads_kv * query_group_size must equal heads_q");
  if (a->input_pos < 0) return fail(B200K_INVALID_ARG, "input_pos must be >= 0");
  const int64_t strides[] = {a->q_stride_b, a->q_stride_h, a->q_stride_s, a->k_stride_b, a->k_stride_h,
                             a->k_stride_s, a->v_stride_b, a->v_stride_h, a->v_stride_s};
  for (int64_t s : strides)
    if ((s * 2) % 16 != 0)
      return fail(B200K_UNSUPPORTED, "Q/K/V strides must be multiples of 16 bytes");
  if ((reinterpret_cast<uintptr_t>(a->q) | reinterpret_cast<uintptr_t>(a->k) |
       reinterpret_cast<uintptr_t>(a->v)) & 15)
    return fail(B200K_UNSUPPORTED, "Q/K/V must be 16-byte aligned");

  // a few query rows per KV head: stream K / V once over many CTAs instead of padding a
  // 128-row tensor-core tile
  if (a->workspace != nullptr && fmha_decode_applies(a) &&
      (reinterpret_cast<uintptr_t>(a->workspace) & 15) == 0) {
    const int sms = current_sm_count();
    if (sms > 0 && a->workspace_bytes >= fmha_decode_workspace_bytes(a, sms) &&
        (a->o_stride_b | a->o_stride_h | a->o_stride_s) >= 0)
      return launch_fmha_decode(a, sms, stream);
  }

  const CUtensorMapDataType dt =
      a->dtype == B200K_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  CUtensorMap tq, tk, tv;
  const int d = a->head_dim;
  if (!encode_tmap_4d(&tq, dt, a->q, d, a->seq_q, a->heads_q, a->batch, a->q_stride_s * 2,
                      a->q_stride_h * 2, a->q_stride_b * 2, 64, 128, 1, 1, CU_TENSOR_MAP_SWIZZLE_128B))
    return B200K_INVALID_ARG;
  if (!encode_tmap_4d(&tk, dt, a->k, d, a->seq_kv, a->heads_kv, a->batch, a->k_stride_s * 2,
                      a->k_stride_h * 2, a->k_stride_b * 2, 64, 128, 1, 1, CU_TENSOR_MAP_SWIZZLE_128B))
    return B200K_INVALID_ARG;
  if (!encode_tmap_4d(&tv, dt, a->v, d, a->seq_kv, a->heads_kv, a->batch, a->v_stride_s * 2,
                      a->v_stride_h * 2, a->v_stride_b * 2, 64, 128, 1, 1, CU_TENSOR_MAP_SWIZZLE_128B))
    return B200K_INVALID_ARG;

  FmhaParams p = {};
  p.out = a->out;
  p.o_stride_b = a->o_stride_b;
  p.o_stride_h = a->o_stride_h;
  p.o_stride_s = a->o_stride_s;
  p.batch = static_cast<int>(a->batch);
  p.heads_q = static_cast<int>(a->heads_q);
  p.heads_kv = static_cast<int>(a->heads_kv);
  p.group = a->query_group_size;
  p.sq = static_cast<int>(a->seq_q);
  p.sk = static_cast<int>(a->seq_kv);
  p.q_tiles = static_cast<int>(ceil_div(a->seq_q, kFmhaBM));
  p.scale_log2 = a->qk_scale * 1.4426950408889634f;
  p.causal = a->causal;
  p.input_pos = static_cast<int>(a->input_pos);
  p.status = device_status_word();
  const int64_t grid64 = static_cast<int64_t>(p.q_tiles) * a->batch * a->heads_q;
  if (grid64 > INT32_MAX) return fail(B200K_UNSUPPORTED, "too many tiles");
  const int grid = static_cast<int>(grid64);
  const bool bf16 = a->dtype == B200K_BF16;
  // head dim 128 and more than one query tile: two query tiles per CTA (B200K_FMHA_ONE_TILE=1
  // forces the one-tile kernel)
  const char* one_tile = getenv("B200K_FMHA_ONE_TILE");
  if (d == 128 && a->seq_q > 128 && !(one_tile != nullptr && one_tile[0] == '1')) {
    const int64_t g2 = ceil_div(a->seq_q, 256) * a->batch * a->heads_q;
    if (g2 > INT32_MAX) return fail(B200K_UNSUPPORTED, "too many tiles");
    return bf16 ? launch_fmha_pair<true>(tq, tk, tv, p, static_cast<int>(g2), stream)
                : launch_fmha_pair<false>(tq, tk, tv, p, static_cast<int>(g2), stream);
  }
  if (d == 128)
    return bf16 ? launch_fmha<128, true>(tq, tk, tv, p, grid, stream)
                : launch_fmha<128, false>(tq, tk, tv, p, grid, stream);
  return bf16 ? launch_fmha<64, true>(tq, tk, tv, p, grid, stream)
              : launch_fmha<64, false>(tq, tk, tv, p, grid, stream);
}

extern "C" int64_t b200k_fmha_workspace_bytes(const b200k_fmha_args* a) {
  if (a == nullptr || a->batch <= 0 || a->heads_kv <= 0 || a->seq_q <= 0 || a->seq_kv <= 0 ||
      a->query_group_size <= 0 || (a->head_dim != 64 && a->head_dim != 128))
    return 0;
  const int sms = current_sm_count();
  if (sms <= 0) return 0;
  return fmha_decode_workspace_bytes(a, sms);
}
