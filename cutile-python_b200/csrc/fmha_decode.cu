// Attention forward for a handful of query rows per key/value head (decode steps, short
// query chunks, grouped-query heads that share one KV head): HBM-bound, so no tensor
// cores.  The keys of one (batch, KV head) are split over several CTAs ("flash
// decoding"): every CTA streams its chunk of K and V once, keeps an online softmax per
// query row and writes an unnormalised partial (max, sum, accumulator) to scratch memory;
// a second kernel merges the partials.
//
// Same semantics as the tensor-core kernels in fmha.cu (reference:
// test/kernels/attention.py:20-128): scores in the exp2 domain, causal mask with query
// positions offset by input_pos, grouped-query heads by integer division.  P stays in
// fp32 here (the tensor-core path rounds it to the input type before P V).
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

// Eight 16-bit elements (one 16-byte load) widened to fp32.
template <typename T>
__device__ __forceinline__ void widen8(const uint4& raw, float* dst) {
  const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
  for (int i = 0; i < 8; ++i) dst[i] = to_float<T>(e[i]);
}

// How a warp is laid over keys and head dimension.  L lanes share one key: lane `sub` of a
// group holds the elements [v * 8 L + 8 sub, + 8) for v < VEC of that key's row (16-byte
// loads; the L lanes of a group read whole 128-byte lines).  A warp therefore takes G = 32 / L
// keys per step, a dot product needs log2(L) shuffle steps - shared by the G keys - instead of
// five per key, and every group keeps its own online-softmax state (maximum, sum, its slice
// of the accumulator), merged once at the end: nothing crosses groups in the loop.
template <int D, int R>
struct DecodeLayout {
  static constexpr int L = (D == 128 && R > 4) ? 16 : 8;   // eight rows: halve the accumulator slice
  static constexpr int G = 32 / L;
  static constexpr int EPL = D / L;        // 16 or 8 elements per lane
  static constexpr int VEC = EPL / 8;      // 16-byte loads per row and lane
  // steps per batch: 16 keys (2 x 4 KB of rows) in flight per warp; 32 keys for one or two
  // rows, whose accumulators leave the registers for it
  static constexpr int KS = (R <= 2 ? 32 : 16) / G;
};

// The CTA-wide partial softmax state of the keys [c0, c1) of one (batch, KV head) for up to R
// query rows: on return cta_ml[r] = running maximum, cta_ml[R + r] = running sum and
// cta_acc[r * D + d] = unnormalised output, in shared memory, visible to the whole CTA.
// q_smem: R * D floats of scratch (the pre-scaled query rows).
template <typename T, int D, int R, int WARPS>
__device__ __forceinline__ void decode_cta_partial(const DecodeParams& p, int b, int hkv, int c0, int c1,
                                                   float* cta_ml, float* cta_acc, float* q_smem) {
  using Lay = DecodeLayout<D, R>;
  constexpr int L = Lay::L, G = Lay::G, EPL = Lay::EPL, VEC = Lay::VEC, KS = Lay::KS;
  constexpr int KPB = KS * G;   // keys per warp and batch
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int grp = lane / L, sub = lane % L;
  const T* kbase = static_cast<const T*>(p.k) + b * p.k_stride_b + hkv * p.k_stride_h;
  const T* vbase = static_cast<const T*>(p.v) + b * p.v_stride_b + hkv * p.v_stride_h;

  // K / V rows in 16-byte units; this lane's first element of the key `grp` of step 0
  const int64_t kstep = p.k_stride_s / 8, vstep = p.v_stride_s / 8;
  const uint4* k16 = reinterpret_cast<const uint4*>(kbase) + sub;
  const uint4* v16 = reinterpret_cast<const uint4*>(vbase) + sub;

  uint4 kreg[KS][VEC], vreg[KS][VEC];
  // FULL: the whole batch lies inside [c0, c1) (one multiply per batch, adds per step);
  // otherwise rows past the end repeat the last key of the chunk and are masked below
  auto load_rows = [&](const uint4* base16, int64_t step16, int base, bool full, uint4 (&reg)[KS][VEC]) {
    if (full) {
      const uint4* row = base16 + static_cast<int64_t>(base + grp) * step16;
#pragma unroll
      for (int st = 0; st < KS; ++st) {
#pragma unroll
        for (int v = 0; v < VEC; ++v) reg[st][v] = __ldg(row + v * L);
        row += G * step16;
      }
    } else {
#pragma unroll
      for (int st = 0; st < KS; ++st) {
        const uint4* row = base16 + static_cast<int64_t>(min(base + st * G + grp, c1 - 1)) * step16;
#pragma unroll
        for (int v = 0; v < VEC; ++v) reg[st][v] = __ldg(row + v * L);
      }
    }
  };
  int base = c0 + warp * KPB;
  if (base < c1) {   // in flight before anything else is fetched
    load_rows(k16, kstep, base, base + KPB <= c1, kreg);
    load_rows(v16, vstep, base, base + KPB <= c1, vreg);
  }

  // Query rows of this KV head, pre-scaled, to shared memory; row r = g * sq + s (head
  // hkv * group + g, query s).  Layout [row][v][half][sub][4]: the eight (sixteen) lanes of a
  // group read consecutive 16-byte pieces, so a 128-bit load has no bank conflicts.
  for (int idx = threadIdx.x; idx < R * D; idx += WARPS * 32) {
    const int r = idx / D, d = idx % D;
    float qf = 0.f;
    if (r < p.rows) {
      const int g = r / p.sq, sq_i = r % p.sq;
      const T* qrow = static_cast<const T*>(p.q) + b * p.q_stride_b +
                      static_cast<int64_t>(hkv * p.group + g) * p.q_stride_h + sq_i * p.q_stride_s;
      qf = to_float<T>(qrow[d]) * p.scale_log2;
    }
    const int v = d / (8 * L), lane_sub = (d / 8) % L, j = d % 8;
    q_smem[r * D + ((v * 2 + j / 4) * L + lane_sub) * 4 + (j % 4)] = qf;
  }
  __syncthreads();

  float m_run[R], l_run[R], acc[R][EPL];
  int row_pos[R];   // last key a row may see under the causal mask
#pragma unroll
  for (int r = 0; r < R; ++r) {
    m_run[r] = -INFINITY;
    l_run[r] = 0.f;
    row_pos[r] = p.input_pos + (r % p.sq);
#pragma unroll
    for (int e = 0; e < EPL; ++e) acc[r][e] = 0.f;
  }
  // every key of the chunk visible to every row (always so for a decode step), all R rows real
  const bool plain = (!p.causal || c1 - 1 <= p.input_pos) && p.rows == R;

  // One batch: PLAIN = no masks and no row predicates.
  auto batch = [&](auto plain_tag, bool full) {
    constexpr bool PLAIN = decltype(plain_tag)::value;
    // scores of this group's key in every step, for every row (two partial sums per dot
    // product: half the dependent chain)
    float sc[R][KS];
#pragma unroll
    for (int st = 0; st < KS; ++st) {
      float kf[EPL];
#pragma unroll
      for (int v = 0; v < VEC; ++v) widen8<T>(kreg[st][v], kf + v * 8);
#pragma unroll
      for (int r = 0; r < R; ++r) {
        float p0 = 0.f, p1 = 0.f;
        if (PLAIN || r < p.rows) {
#pragma unroll
          for (int v = 0; v < VEC; ++v) {
            const float4 q0 = *reinterpret_cast<const float4*>(q_smem + r * D + ((v * 2 + 0) * L + sub) * 4);
            const float4 q1 = *reinterpret_cast<const float4*>(q_smem + r * D + ((v * 2 + 1) * L + sub) * 4);
            p0 = fmaf(q0.x, kf[v * 8 + 0], p0);
            p1 = fmaf(q1.x, kf[v * 8 + 4], p1);
            p0 = fmaf(q0.y, kf[v * 8 + 1], p0);
            p1 = fmaf(q1.y, kf[v * 8 + 5], p1);
            p0 = fmaf(q0.z, kf[v * 8 + 2], p0);
            p1 = fmaf(q1.z, kf[v * 8 + 6], p1);
            p0 = fmaf(q0.w, kf[v * 8 + 3], p0);
            p1 = fmaf(q1.w, kf[v * 8 + 7], p1);
          }
        }
        sc[r][st] = p0 + p1;
      }
    }
    const int next = base + WARPS * KPB;
    // the K registers are free: next batch's keys are fetched behind the P V below
    if (next < c1) load_rows(k16, kstep, next, next + KPB <= c1, kreg);
#pragma unroll
    for (int o = L / 2; o > 0; o >>= 1) {
#pragma unroll
      for (int r = 0; r < R; ++r) {
#pragma unroll
        for (int st = 0; st < KS; ++st) sc[r][st] += __shfl_xor_sync(0xffffffffu, sc[r][st], o);
      }
    }
    // online softmax of this group's KS keys, per row
#pragma unroll
    for (int r = 0; r < R; ++r) {
      if (PLAIN || r < p.rows) {
        float m_new = m_run[r];
#pragma unroll
        for (int st = 0; st < KS; ++st) {
          if (!PLAIN || !full) {
            const int key = base + st * G + grp;
            if (key >= c1 || (!PLAIN && p.causal && key > row_pos[r])) sc[r][st] = -INFINITY;
          }
          m_new = fmaxf(m_new, sc[r][st]);
        }
        if (m_new > m_run[r]) {   // also the first block: exp2(-inf) = 0
          const float corr = decode_exp2(m_run[r] - m_new);
          l_run[r] *= corr;
#pragma unroll
          for (int e = 0; e < EPL; ++e) acc[r][e] *= corr;
          m_run[r] = m_new;
        }
#pragma unroll
        for (int st = 0; st < KS; ++st) {
          // a masked key (or every key so far masked, m_new = -inf) weighs 0, not exp2(nan)
          float w = decode_exp2(sc[r][st] - m_new);
          if ((!PLAIN || !full) && sc[r][st] == -INFINITY) w = 0.f;
          sc[r][st] = w;
          l_run[r] += w;
        }
      }
    }
#pragma unroll
    for (int st = 0; st < KS; ++st) {
      float vf[EPL];
#pragma unroll
      for (int v = 0; v < VEC; ++v) widen8<T>(vreg[st][v], vf + v * 8);
#pragma unroll
      for (int r = 0; r < R; ++r) {
        if (PLAIN || r < p.rows) {
#pragma unroll
          for (int e = 0; e < EPL; ++e) acc[r][e] = fmaf(sc[r][st], vf[e], acc[r][e]);
        }
      }
    }
    base = next;
    if (base < c1) load_rows(v16, vstep, base, base + KPB <= c1, vreg);
  };

  while (base < c1) {
    const bool full = base + KPB <= c1;
    if (plain) batch(std::true_type{}, full);
    else batch(std::false_type{}, full);
  }

  // merge the G groups of the warp (same rule as between warps and between CTAs)
#pragma unroll
  for (int r = 0; r < R; ++r) {
    float m_all = m_run[r];
#pragma unroll
    for (int o = L; o < 32; o <<= 1) m_all = fmaxf(m_all, __shfl_xor_sync(0xffffffffu, m_all, o));
    const float f = (m_run[r] == -INFINITY) ? 0.f : exp2f(m_run[r] - m_all);
    float l = l_run[r] * f;
#pragma unroll
    for (int o = L; o < 32; o <<= 1) l += __shfl_xor_sync(0xffffffffu, l, o);
#pragma unroll
    for (int e = 0; e < EPL; ++e) {
      float a = acc[r][e] * f;
#pragma unroll
      for (int o = L; o < 32; o <<= 1) a += __shfl_xor_sync(0xffffffffu, a, o);
      acc[r][e] = a;
    }
    m_run[r] = m_all;
    l_run[r] = l;
  }

  // merge the warps
  __shared__ float sm_m[WARPS][R], sm_l[WARPS][R];
  __shared__ float sm_acc[WARPS][R][D];
#pragma unroll
  for (int r = 0; r < R; ++r) {
    if (lane == 0) {
      sm_m[warp][r] = m_run[r];
      sm_l[warp][r] = l_run[r];
    }
    if (grp == 0) {
#pragma unroll
      for (int e = 0; e < EPL; ++e) sm_acc[warp][r][(e / 8) * 8 * L + sub * 8 + (e % 8)] = acc[r][e];
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
// [max, sum, acc[D]] per row to scratch memory.  R = compile-time bound on the query rows.
template <typename T, int D, int R>
__global__ void __launch_bounds__(kDecThreads, 2)
fmha_decode_kernel(const DecodeParams p) {
  __shared__ float cta_ml[2 * R];
  __shared__ float cta_acc[R * D];
  __shared__ __align__(16) float q_smem[R * D];
  pdl_launch_dependents();   // the merge kernel may be set up now; it waits for this grid
  const int split = blockIdx.x;
  const int b = blockIdx.y / p.heads_kv, hkv = blockIdx.y % p.heads_kv;
  const int c0 = split * p.chunk;
  decode_cta_partial<T, D, R, kDecWarps>(p, b, hkv, c0, min(p.sk, c0 + p.chunk), cta_ml, cta_acc, q_smem);
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

template <typename T, int D, int R>
__global__ void __launch_bounds__(kClusterThreads, 2)
fmha_decode_cluster_kernel(const DecodeParams p) {
  __shared__ float cta_ml[2 * R];
  __shared__ float cta_acc[R * D];
  __shared__ __align__(16) float q_smem[R * D];
  const int split = static_cast<int>(cluster_ctarank());
  const int cs = p.splits;   // == the cluster size of this launch
  const int b = blockIdx.y / p.heads_kv, hkv = blockIdx.y % p.heads_kv;
  const int c0 = split * p.chunk;
  decode_cta_partial<T, D, R, kClusterThreads / 32>(p, b, hkv, c0, min(p.sk, c0 + p.chunk), cta_ml, cta_acc,
                                                    q_smem);
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
  }
  // One kernel, no scratch: the smallest cluster that gives every SM a CTA of four warps.
  // More CTAs than that only add rounds of launch, warp merge and cluster barriers.
  if (!force_two && (forced > 0 || groups * kMaxClusterSplits * 2 >= sms)) {
    int cs = 1;
    while (cs < kMaxClusterSplits && groups * cs < sms) cs *= 2;
    while (cs > 1 && ceil_div(sk, cs) < 64) cs /= 2;   // at least 64 keys per CTA
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
    cudaError_t e;
    if (p.rows <= 1) e = cudaLaunchKernelEx(&cfg, fmha_decode_cluster_kernel<T, D, 1>, p);
    else if (p.rows <= 2) e = cudaLaunchKernelEx(&cfg, fmha_decode_cluster_kernel<T, D, 2>, p);
    else if (p.rows <= 4) e = cudaLaunchKernelEx(&cfg, fmha_decode_cluster_kernel<T, D, 4>, p);
    else e = cudaLaunchKernelEx(&cfg, fmha_decode_cluster_kernel<T, D, 8>, p);
    if (e != cudaSuccess)
      return fail(B200K_CUDA_ERROR, "fmha decode (cluster of %d) launch: %s", p.splits, cudaGetErrorString(e));
    return B200K_OK;
  }
  if (p.rows <= 1) fmha_decode_kernel<T, D, 1><<<grid, kDecThreads, 0, stream>>>(p);
  else if (p.rows <= 2) fmha_decode_kernel<T, D, 2><<<grid, kDecThreads, 0, stream>>>(p);
  else if (p.rows <= 4) fmha_decode_kernel<T, D, 4><<<grid, kDecThreads, 0, stream>>>(p);
  else fmha_decode_kernel<T, D, 8><<<grid, kDecThreads, 0, stream>>>(p);
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
