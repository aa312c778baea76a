// Attention forward for a handful of query rows per key/value head (decode steps, short
// query chunks, grouped-query heads that share one KV head): HBM-bound.  The keys of one
// (batch, KV head) are split over several CTAs ("flash decoding"): every CTA streams its
// chunk of K and V once, straight from global memory into MMA fragments (no shared-memory
// staging, no TMA), keeps an online softmax per query row and leaves an unnormalised partial
// (max, sum, accumulator); the partials are merged over distributed shared memory by the
// CTAs of a cluster, or by a second kernel.
//
// Same semantics as the tensor-core kernels in fmha.cu (reference:
// test/kernels/attention.py:20-128): scores in the exp2 domain, causal mask with query
// positions offset by input_pos, grouped-query heads by integer division, P rounded to the
// input type before P V.
#include "fmha_decode.h"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cstdlib>
#include <type_traits>

namespace b200k {
namespace {

constexpr int kDecThreads = 128;
constexpr int kDecWarps = kDecThreads / 32;

struct DecodeParams {
  const void* q;
  const void* k;
  const void* v;
  void* out;
  float* ws;
  int64_t q_stride_b, q_stride_h, q_stride_s;
  int64_t k_stride_b, k_stride_h, k_stride_s;
  int64_t v_stride_b, v_stride_h, v_stride_s;
  int64_t o_stride_b, o_stride_h, o_stride_s;
  int heads_kv, group, sq, sk;
  int rows;        // sq * group query rows share one KV head
  int splits;
  int chunk;       // keys per split, a multiple of 64
  float scale_log2;
  int causal;
  int input_pos;
};

template <typename T> __device__ __forceinline__ float to_float(T v);
template <> __device__ __forceinline__ float to_float<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ __half from_float<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float decode_exp2(float x) {   // exp2(-inf) = 0
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// ---- tensor-core fragments (legacy mma.sync m16n8k16: the work is HBM-bound, the point is
// the instruction count - one MMA replaces 8 x 16 x 16 fused multiply-adds spread over a
// warp's CUDA cores, conversions and shuffles included) -------------------------------------
template <typename T> struct Frag;
template <> struct Frag<__half> {
  static __device__ __forceinline__ void mma(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                             uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
                 "{%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  }
  static __device__ __forceinline__ uint32_t pack(float lo, float hi) {
    const __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&h);
  }
};
template <> struct Frag<__nv_bfloat16> {
  static __device__ __forceinline__ void mma(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                             uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
                 "{%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  }
  static __device__ __forceinline__ uint32_t pack(float lo, float hi) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&h);
  }
};
// 8 x 8 transpose of 16-bit elements inside a warp: lane (g, t) gives row g, columns 2t, 2t+1
// and receives the same of the transposed matrix.
__device__ __forceinline__ uint32_t transpose_8x8_b16(uint32_t x) {
  uint32_t y;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(y) : "r"(x));
  return y;
}
__device__ __forceinline__ uint32_t comp(const uint4& v, int i) {
  return i == 0 ? v.x : (i == 1 ? v.y : (i == 2 ? v.z : v.w));
}

constexpr int kDecRows = kFmhaDecodeMaxRows;   // 8 = the N of the MMAs

// The CTA-wide partial softmax state of the keys [c0, c1) of one (batch, KV head) for up to
// eight query rows: on return cta_ml[r] = running maximum, cta_ml[8 + r] = running sum and
// cta_acc[r * D + d] = unnormalised output, in shared memory, visible to the whole CTA.
//
// A warp takes 16 keys per step, lane = (g, t) = (lane / 4, lane % 4):
//   S^T (16 keys x 8 rows) = K (16 keys x D) . Q^T       A = K rows g, g + 8; B = Q row g
//   O^T (D x 8 rows)      += V^T (D x 16 keys) . P^T     A = V^T, B = P^T
// Both contractions only sum over their K index, so the order of the head dimension inside a
// k-step (first product) and of the output dimensions (second) is free: lanes read K, Q and V
// rows as 16-byte vectors and use their 32-bit components directly as fragments, no shuffles,
// no shared memory.  The S^T accumulator gives lane (g, t) the scores of keys g, g + 8 for the
// rows 2t, 2t + 1 - the same two rows whose O^T columns the lane holds, so the online-softmax
// rescale needs no exchange; P^T becomes the B operand of the second product through two
// 8 x 8 register transposes.  P is rounded to the input type before P V, as in the
// tensor-core prefill kernels.
template <typename T, int D, int WARPS>
__device__ __forceinline__ void decode_cta_partial(const DecodeParams& p, int b, int hkv, int c0, int c1,
                                                   float* cta_ml, float* cta_acc) {
  constexpr int R = kDecRows;
  constexpr int KV = D / 32;        // 16-byte vectors of a K (or Q) row per lane: dims [(t + 4 i) * 8, + 8)
  constexpr int VV = D / 64;        // 16-byte vectors of a V row per lane: dims [(g + 8 i) * 8, + 8)
  constexpr int NB = 2;             // 16-key blocks per step: 2 x 8 KB of rows in flight per warp
  constexpr int KPB = 16 * NB;      // keys per warp and step
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const T* kbase = static_cast<const T*>(p.k) + b * p.k_stride_b + hkv * p.k_stride_h;
  const T* vbase = static_cast<const T*>(p.v) + b * p.v_stride_b + hkv * p.v_stride_h;
  const int64_t kstep = p.k_stride_s / 8, vstep = p.v_stride_s / 8;   // rows in 16-byte units
  const uint4* k16 = reinterpret_cast<const uint4*>(kbase) + t;
  const uint4* v16 = reinterpret_cast<const uint4*>(vbase) + g;

  uint4 kreg[NB][2][KV];   // per block: keys blk + g, blk + g + 8
  uint4 vreg[NB][4][VV];   // per block: keys blk + 2t, 2t + 1, 2t + 8, 2t + 9
  // rows past the end of the chunk repeat its last key; they are masked below
  auto load_k = [&](int base) {
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) {
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const uint4* row = k16 + static_cast<int64_t>(min(base + 16 * nb + g + 8 * j, c1 - 1)) * kstep;
#pragma unroll
        for (int i = 0; i < KV; ++i) kreg[nb][j][i] = __ldg(row + 4 * i);
      }
    }
  };
  auto load_v = [&](int base) {
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int key = base + 16 * nb + 2 * t + (j & 1) + 8 * (j >> 1);
        const uint4* row = v16 + static_cast<int64_t>(min(key, c1 - 1)) * vstep;
#pragma unroll
        for (int i = 0; i < VV; ++i) vreg[nb][j][i] = __ldg(row + 8 * i);
      }
    }
  };
  int base = c0 + warp * KPB;
  if (base < c1) {   // in flight before anything else is fetched
    load_k(base);
    load_v(base);
  }

  // this lane's query row g (row r = grp * sq + s: head hkv * group + grp, query s), raw
  uint4 qreg[KV];
  {
    const bool real = g < p.rows;
    const int grp = real ? g / p.sq : 0, s_i = real ? g % p.sq : 0;
    const T* qrow = static_cast<const T*>(p.q) + b * p.q_stride_b +
                    static_cast<int64_t>(hkv * p.group + grp) * p.q_stride_h + s_i * p.q_stride_s;
#pragma unroll
    for (int i = 0; i < KV; ++i) {
      qreg[i] = make_uint4(0u, 0u, 0u, 0u);
      if (real) {
        // the query row need not be 16-byte aligned: element loads, once per CTA and lane
        const T* src = qrow + (t + 4 * i) * 8;
        uint32_t w[4];
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const uint16_t lo = *reinterpret_cast<const uint16_t*>(src + 2 * c);
          const uint16_t hi = *reinterpret_cast<const uint16_t*>(src + 2 * c + 1);
          w[c] = static_cast<uint32_t>(lo) | (static_cast<uint32_t>(hi) << 16);
        }
        qreg[i] = make_uint4(w[0], w[1], w[2], w[3]);
      }
    }
  }

  // rows 2t, 2t + 1 of this lane: softmax state and the last key each may see
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  int row_pos[2];
#pragma unroll
  for (int c = 0; c < 2; ++c) row_pos[c] = p.input_pos + ((2 * t + c) % p.sq);
  float acc[VV * 4][4];   // m-tile (i, jj): dims (g + 8 i) * 8 + 2 jj (+ 1) x rows 2t, 2t + 1
#pragma unroll
  for (int m = 0; m < VV * 4; ++m) {
#pragma unroll
    for (int c = 0; c < 4; ++c) acc[m][c] = 0.f;
  }
  // every key of the chunk visible to every row: always so for a decode step
  const bool unmasked = !p.causal || c1 - 1 <= p.input_pos;

  while (base < c1) {
    // S^T per block: sc[.][0], [1] = key blk + g x rows 2t, 2t + 1; sc[.][2], [3] = key blk + g + 8
    float sc[NB][4];
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) {
#pragma unroll
      for (int c = 0; c < 4; ++c) sc[nb][c] = 0.f;
#pragma unroll
      for (int i = 0; i < KV; ++i) {
#pragma unroll
        for (int h = 0; h < 2; ++h)
          Frag<T>::mma(sc[nb], comp(kreg[nb][0][i], 2 * h), comp(kreg[nb][1][i], 2 * h),
                       comp(kreg[nb][0][i], 2 * h + 1), comp(kreg[nb][1][i], 2 * h + 1), comp(qreg[i], 2 * h),
                       comp(qreg[i], 2 * h + 1));
      }
    }
    const int next = base + WARPS * KPB;
    if (next < c1) load_k(next);   // the K registers are free: next keys behind the softmax and P V
    const bool mask = !unmasked || base + KPB > c1;
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) {
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        sc[nb][c] *= p.scale_log2;
        if (mask) {
          const int key = base + 16 * nb + g + 8 * (c >> 1);
          if (key >= c1 || (p.causal && key > row_pos[c & 1])) sc[nb][c] = -INFINITY;
        }
      }
    }
    // row maxima over the step's keys: 2 NB in this lane, the rest in the lanes of equal t
    float m_new[2], corr[2];
    bool grew = false;
#pragma unroll
    for (int c = 0; c < 2; ++c) {
      float m = fmaxf(sc[0][c], sc[0][c + 2]);
#pragma unroll
      for (int nb = 1; nb < NB; ++nb) m = fmaxf(m, fmaxf(sc[nb][c], sc[nb][c + 2]));
      m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 4));
      m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 8));
      m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 16));
      m_new[c] = fmaxf(m_run[c], m);
      grew = grew || (m_new[c] > m_run[c]);
      corr[c] = decode_exp2(m_run[c] - m_new[c]);   // exp2(-inf - x) = 0 on the first block
      if (m_new[c] == -INFINITY) corr[c] = 1.f;      // every key so far masked: nothing to rescale
      m_run[c] = m_new[c];
    }
    if (__any_sync(0xffffffffu, grew)) {
#pragma unroll
      for (int c = 0; c < 2; ++c) l_run[c] *= corr[c];
#pragma unroll
      for (int m = 0; m < VV * 4; ++m) {
        acc[m][0] *= corr[0];
        acc[m][1] *= corr[1];
        acc[m][2] *= corr[0];
        acc[m][3] *= corr[1];
      }
    }
    const float mref[2] = {m_new[0] == -INFINITY ? 0.f : m_new[0], m_new[1] == -INFINITY ? 0.f : m_new[1]};
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) {
      float pw[4];
#pragma unroll
      for (int c = 0; c < 4; ++c) pw[c] = decode_exp2(sc[nb][c] - mref[c & 1]);   // masked: exp2(-inf) = 0
      // the sums use the rounded weights, like the prefill kernels
      const uint32_t p_lo = Frag<T>::pack(pw[0], pw[1]), p_hi = Frag<T>::pack(pw[2], pw[3]);
      const T* e = reinterpret_cast<const T*>(&p_lo);
      const T* f = reinterpret_cast<const T*>(&p_hi);
      l_run[0] += to_float<T>(e[0]) + to_float<T>(f[0]);
      l_run[1] += to_float<T>(e[1]) + to_float<T>(f[1]);
      const uint32_t b0 = transpose_8x8_b16(p_lo), b1 = transpose_8x8_b16(p_hi);
#pragma unroll
      for (int i = 0; i < VV; ++i) {
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) {
          const uint32_t w0 = comp(vreg[nb][0][i], jj), w1 = comp(vreg[nb][1][i], jj);
          const uint32_t w2 = comp(vreg[nb][2][i], jj), w3 = comp(vreg[nb][3][i], jj);
          Frag<T>::mma(acc[i * 4 + jj], __byte_perm(w0, w1, 0x5410), __byte_perm(w0, w1, 0x7632),
                       __byte_perm(w2, w3, 0x5410), __byte_perm(w2, w3, 0x7632), b0, b1);
        }
      }
    }
    base = next;
    if (base < c1) load_v(base);
  }

  // row sums over the lanes of equal t
#pragma unroll
  for (int c = 0; c < 2; ++c) {
    l_run[c] += __shfl_xor_sync(0xffffffffu, l_run[c], 4);
    l_run[c] += __shfl_xor_sync(0xffffffffu, l_run[c], 8);
    l_run[c] += __shfl_xor_sync(0xffffffffu, l_run[c], 16);
  }

  // merge the warps
  __shared__ float sm_m[WARPS][R], sm_l[WARPS][R];
  __shared__ float sm_acc[WARPS][R][D];
  if (g == 0) {
#pragma unroll
    for (int c = 0; c < 2; ++c) {
      sm_m[warp][2 * t + c] = m_run[c];
      sm_l[warp][2 * t + c] = l_run[c];
    }
  }
#pragma unroll
  for (int i = 0; i < VV; ++i) {
#pragma unroll
    for (int jj = 0; jj < 4; ++jj) {
      const int d = (g + 8 * i) * 8 + 2 * jj;
      const float* a = acc[i * 4 + jj];
      sm_acc[warp][2 * t][d] = a[0];
      sm_acc[warp][2 * t + 1][d] = a[1];
      sm_acc[warp][2 * t][d + 1] = a[2];
      sm_acc[warp][2 * t + 1][d + 1] = a[3];
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < p.rows * D; idx += WARPS * 32) {
    const int r = idx / D, d = idx % D;
    float m = -INFINITY;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) m = fmaxf(m, sm_m[w][r]);
    float l = 0.f, o = 0.f;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) {
      const float f = (sm_m[w][r] == -INFINITY) ? 0.f : exp2f(sm_m[w][r] - m);
      l += sm_l[w][r] * f;
      o += sm_acc[w][r][d] * f;
    }
    if (d == 0) {
      cta_ml[r] = m;
      cta_ml[R + r] = l;
    }
    cta_acc[r * D + d] = o;
  }
  __syncthreads();
}

// Split-KV, two kernels: grid (splits, batch * heads_kv); every CTA writes its partial
// [max, sum, acc[D]] per row to scratch memory.
template <typename T, int D>
__global__ void __launch_bounds__(kDecThreads, 2)
fmha_decode_kernel(const DecodeParams p) {
  constexpr int R = kDecRows;
  __shared__ float cta_ml[2 * R];
  __shared__ float cta_acc[R * D];
  pdl_launch_dependents();   // the merge kernel may be set up now; it waits for this grid
  const int split = blockIdx.x;
  const int b = blockIdx.y / p.heads_kv, hkv = blockIdx.y % p.heads_kv;
  const int c0 = split * p.chunk;
  decode_cta_partial<T, D, kDecWarps>(p, b, hkv, c0, min(p.sk, c0 + p.chunk), cta_ml, cta_acc);
  for (int idx = threadIdx.x; idx < p.rows * D; idx += kDecThreads) {
    const int r = idx / D, d = idx % D;
    float* dst = p.ws + ((static_cast<int64_t>(blockIdx.y) * p.rows + r) * p.splits + split) * (D + 2);
    if (d == 0) {
      dst[0] = cta_ml[r];
      dst[1] = cta_ml[R + r];
    }
    dst[2 + d] = cta_acc[idx];
  }
}

// Split-KV, one kernel: the CTAs of a cluster (1, 2, 4 or 8, chosen at launch) share one
// (batch, KV head); after its chunk every CTA leaves its partial in shared memory, and each
// CTA merges D / cluster-size output columns of all rows by reading the partials over
// distributed shared memory.
constexpr int kMaxClusterSplits = 8;
constexpr int kClusterThreads = 128;

template <typename T, int D>
__global__ void __launch_bounds__(kClusterThreads, 2)
fmha_decode_cluster_kernel(const DecodeParams p) {
  constexpr int R = kDecRows;
  __shared__ float cta_ml[2 * R];
  __shared__ float cta_acc[R * D];
  const int split = static_cast<int>(cluster_ctarank());
  const int cs = p.splits;   // == the cluster size of this launch
  const int b = blockIdx.y / p.heads_kv, hkv = blockIdx.y % p.heads_kv;
  const int c0 = split * p.chunk;
  decode_cta_partial<T, D, kClusterThreads / 32>(p, b, hkv, c0, min(p.sk, c0 + p.chunk), cta_ml, cta_acc);
  cluster_sync_all();   // every partial of the cluster is in place
  const int cols = D / cs;
  const uint32_t ml_addr = smem_u32(cta_ml), acc_addr = smem_u32(cta_acc);
  for (int idx = threadIdx.x; idx < p.rows * cols; idx += kClusterThreads) {
    const int r = idx / cols, d = split * cols + idx % cols;
    float ms[kMaxClusterSplits];
    float m = -INFINITY;
#pragma unroll
    for (int c = 0; c < kMaxClusterSplits; ++c) {
      ms[c] = -INFINITY;
      if (c < cs) {
        ms[c] = ld_shared_cluster_f32(map_to_cta(ml_addr + 4u * r, c));
        m = fmaxf(m, ms[c]);
      }
    }
    float l = 0.f, o = 0.f;
#pragma unroll
    for (int c = 0; c < kMaxClusterSplits; ++c) {
      if (c < cs) {
        const float f = (ms[c] == -INFINITY) ? 0.f : exp2f(ms[c] - m);
        l += ld_shared_cluster_f32(map_to_cta(ml_addr + 4u * (R + r), c)) * f;
        o += ld_shared_cluster_f32(map_to_cta(acc_addr + 4u * (r * D + d), c)) * f;
      }
    }
    const int g = r / p.sq, sidx = r % p.sq;
    T* orow = static_cast<T*>(p.out) + b * p.o_stride_b + static_cast<int64_t>(hkv * p.group + g) * p.o_stride_h +
              sidx * p.o_stride_s;
    orow[d] = from_float<T>(l > 0.f ? __fdividef(o, l) : 0.f);
  }
  cluster_sync_all();   // nobody leaves while its shared memory may still be read
}

// grid (batch * heads_kv * rows), D threads: merges the splits and normalises.
constexpr int kMaxMergeSplits = 256;

template <typename T, int D>
__global__ void __launch_bounds__(D)
fmha_decode_merge_kernel(const DecodeParams p) {
  const int r = blockIdx.x % p.rows;
  const int bh = blockIdx.x / p.rows;
  const int b = bh / p.heads_kv, hkv = bh % p.heads_kv;
  const int d = threadIdx.x;
  const float* src = p.ws + static_cast<int64_t>(blockIdx.x) * p.splits * (D + 2);
  // one round trip for all maxima and sums, one (unrolled) for the accumulators
  __shared__ float sm_m[kMaxMergeSplits], sm_f[kMaxMergeSplits];
  __shared__ float sm_l;
  pdl_wait();   // the partial results come from the kernel launched just before
  for (int s = d; s < p.splits; s += D) {
    sm_m[s] = src[s * (D + 2)];
    sm_f[s] = src[s * (D + 2) + 1];
  }
  __syncthreads();
  float m = -INFINITY;
  for (int s = 0; s < p.splits; ++s) m = fmaxf(m, sm_m[s]);
  __syncthreads();
  if (d == 0) {
    float l = 0.f;
    for (int s = 0; s < p.splits; ++s) {
      const float f = (sm_m[s] == -INFINITY) ? 0.f : exp2f(sm_m[s] - m);
      l += sm_f[s] * f;
      sm_f[s] = f;
    }
    sm_l = l;
  }
  __syncthreads();
  float o = 0.f;
#pragma unroll 8
  for (int s = 0; s < p.splits; ++s) o = fmaf(src[s * (D + 2) + 2 + d], sm_f[s], o);
  const float l = sm_l;
  const int g = r / p.sq, sidx = r % p.sq;
  T* orow = static_cast<T*>(p.out) + b * p.o_stride_b + static_cast<int64_t>(hkv * p.group + g) * p.o_stride_h +
            sidx * p.o_stride_s;
  orow[d] = from_float<T>(l > 0.f ? __fdividef(o, l) : 0.f);
}

struct DecodePlan {
  int splits, chunk;
  bool cluster;    // one kernel, `splits` CTAs per (batch, KV head) merged over DSMEM
};

DecodePlan plan_decode(int64_t batch, int64_t heads_kv, int64_t sk, int sms) {
  const int64_t groups = batch * heads_kv;
  DecodePlan plan;
  int forced = 0;   // B200K_DECODE_PLAN=1|2|4|8 (cluster size) or s (two kernels): measurements
  bool force_two = false;
  if (const char* e = getenv("B200K_DECODE_PLAN")) {
    if (e[0] == 's') force_two = true;
    else forced = atoi(e);
    // only the cluster sizes the kernel has (powers of two up to kMaxClusterSplits): anything
    // else is ignored, since D / cluster columns per CTA must divide evenly
    if (forced != 1 && forced != 2 && forced != 4 && forced != 8) forced = 0;
  }
  // One kernel, no scratch: the smallest cluster that gives every SM a CTA of four warps.
  // More CTAs than that only add rounds of launch, warp merge and cluster barriers.
  if (!force_two && (forced > 0 || groups * kMaxClusterSplits * 4 >= sms)) {
    int cs = 1;
    while (cs < kMaxClusterSplits && groups * cs < sms) cs *= 2;
    // at least two steps per warp (256 keys per CTA): q (1,32,1,128) against 1024 keys took
    // 16.4 us in clusters of eight and 14.4 us in clusters of four
    while (cs > 1 && ceil_div(sk, cs) < 256) cs /= 2;
    if (forced > 0) cs = forced;
    plan.cluster = true;
    plan.splits = cs;
    plan.chunk = static_cast<int>(ceil_div(ceil_div(sk, cs), 16) * 16);
    return plan;
  }
  plan.cluster = false;
  // light CTAs (64 - 128 keys each), about four per SM, so that most of K and V is
  // requested in the first round trip
  int64_t want = ceil_div(4 * static_cast<int64_t>(sms), groups);
  int64_t max_splits = ceil_div(sk, 64);
  if (max_splits > kMaxMergeSplits) max_splits = kMaxMergeSplits;
  if (want > max_splits) want = max_splits;
  if (want < 1) want = 1;
  plan.chunk = static_cast<int>(ceil_div(ceil_div(sk, want), 64) * 64);
  plan.splits = static_cast<int>(ceil_div(sk, plan.chunk));
  return plan;
}

template <typename T, int D>
int launch_decode(const DecodeParams& p, bool cluster, int64_t batch, cudaStream_t stream) {
  const dim3 grid(p.splits, static_cast<unsigned>(batch * p.heads_kv));
  if (cluster) {
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = static_cast<unsigned>(p.splits);
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(kClusterThreads);
    cfg.stream = stream;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const cudaError_t e = cudaLaunchKernelEx(&cfg, fmha_decode_cluster_kernel<T, D>, p);
    if (e != cudaSuccess)
      return fail(B200K_CUDA_ERROR, "fmha decode (cluster of %d) launch: %s", p.splits, cudaGetErrorString(e));
    return B200K_OK;
  }
  fmha_decode_kernel<T, D><<<grid, kDecThreads, 0, stream>>>(p);
  B200K_CHECK_LAUNCH("fmha decode launch");
  const cudaError_t e = launch_after_predecessor(fmha_decode_merge_kernel<T, D>,
                                                 dim3(static_cast<unsigned>(batch * p.heads_kv * p.rows)), dim3(D), 0,
                                                 stream, p);
  if (e != cudaSuccess) return fail(B200K_CUDA_ERROR, "fmha decode merge launch: %s", cudaGetErrorString(e));
  return B200K_OK;
}

int64_t visible_keys(const b200k_fmha_args* a) {
  // keys no query row can see under the causal mask are never read
  int64_t sk = a->seq_kv;
  if (a->causal && a->input_pos + a->seq_q < sk) sk = a->input_pos + a->seq_q;
  return sk;
}

}  // namespace

bool fmha_decode_applies(const b200k_fmha_args* a) {
  // K and V rows are read with 16-byte loads
  const auto rows16 = [](const void* base, int64_t sb, int64_t sh, int64_t ss) {
    return (reinterpret_cast<uintptr_t>(base) & 15) == 0 && sb % 8 == 0 && sh % 8 == 0 && ss % 8 == 0;
  };
  return a->seq_q * a->query_group_size <= kFmhaDecodeMaxRows && a->batch * a->heads_kv <= 65535 &&
         rows16(a->k, a->k_stride_b, a->k_stride_h, a->k_stride_s) &&
         rows16(a->v, a->v_stride_b, a->v_stride_h, a->v_stride_s);
}

int64_t fmha_decode_workspace_bytes(const b200k_fmha_args* a, int sms) {
  if (!fmha_decode_applies(a)) return 0;
  const DecodePlan plan = plan_decode(a->batch, a->heads_kv, visible_keys(a), sms);
  // the cluster path needs no scratch; a token amount keeps "0 = path does not apply"
  if (plan.cluster) return 16;
  return a->batch * a->heads_kv * a->seq_q * a->query_group_size * plan.splits * (a->head_dim + 2) * 4;
}

int launch_fmha_decode(const b200k_fmha_args* a, int sms, cudaStream_t stream) {
  DecodeParams p = {};
  p.q = a->q; p.k = a->k; p.v = a->v; p.out = a->out;
  p.ws = static_cast<float*>(a->workspace);
  p.q_stride_b = a->q_stride_b; p.q_stride_h = a->q_stride_h; p.q_stride_s = a->q_stride_s;
  p.k_stride_b = a->k_stride_b; p.k_stride_h = a->k_stride_h; p.k_stride_s = a->k_stride_s;
  p.v_stride_b = a->v_stride_b; p.v_stride_h = a->v_stride_h; p.v_stride_s = a->v_stride_s;
  p.o_stride_b = a->o_stride_b; p.o_stride_h = a->o_stride_h; p.o_stride_s = a->o_stride_s;
  p.heads_kv = static_cast<int>(a->heads_kv);
  p.group = a->query_group_size;
  p.sq = static_cast<int>(a->seq_q);
  const int64_t sk = visible_keys(a);
  p.sk = static_cast<int>(sk);
  p.rows = p.sq * p.group;
  const DecodePlan plan = plan_decode(a->batch, a->heads_kv, sk, sms);
  p.splits = plan.splits;
  p.chunk = plan.chunk;
  p.scale_log2 = a->qk_scale * 1.4426950408889634f;
  p.causal = a->causal;
  p.input_pos = static_cast<int>(a->input_pos);
  const bool bf16 = a->dtype == B200K_BF16;
  if (a->head_dim == 128)
    return bf16 ? launch_decode<__nv_bfloat16, 128>(p, plan.cluster, a->batch, stream)
                : launch_decode<__half, 128>(p, plan.cluster, a->batch, stream);
  return bf16 ? launch_decode<__nv_bfloat16, 64>(p, plan.cluster, a->batch, stream)
              : launch_decode<__half, 64>(p, plan.cluster, a->batch, stream);
}

}  // namespace b200k
