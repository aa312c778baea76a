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

// EPL consecutive elements of a row, lane-contiguous (8 or 4 bytes per lane: a warp reads one
// whole row of 256 or 128 bytes per instruction).  Rows wait in registers as loaded (raw
// 16-bit pairs) and are widened where they are used: half the registers per row in flight.
template <int EPL> struct RawRow;
template <> struct RawRow<4> { uint2 v; };
template <> struct RawRow<2> { uint32_t v; };

template <typename T, int EPL>
__device__ __forceinline__ RawRow<EPL> load_raw(const T* row, int lane) {
  RawRow<EPL> r;
  if constexpr (EPL == 4) r.v = __ldg(reinterpret_cast<const uint2*>(row + lane * 4));
  else r.v = __ldg(reinterpret_cast<const uint32_t*>(row + lane * 2));
  return r;
}

template <typename T, int EPL>
__device__ __forceinline__ void widen(const RawRow<EPL>& raw, float (&dst)[EPL]) {
  const T* e = reinterpret_cast<const T*>(&raw.v);
#pragma unroll
  for (int i = 0; i < EPL; ++i) dst[i] = to_float<T>(e[i]);
}

template <typename T, int EPL>
__device__ __forceinline__ void load_row(const T* row, int lane, float (&dst)[EPL]) {
  widen<T, EPL>(load_raw<T, EPL>(row, lane), dst);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// The CTA-wide partial softmax state of the keys [c0, c1) of one (batch, KV head) for up to R
// query rows: on return cta_ml[r] = running maximum, cta_ml[R + r] = running sum and
// cta_acc[r * D + d] = unnormalised output, in shared memory, visible to the whole CTA.
template <typename T, int D, int R, int WARPS>
__device__ __forceinline__ void decode_cta_partial(const DecodeParams& p, int b, int hkv, int c0, int c1,
                                                   float* cta_ml, float* cta_acc) {
  constexpr int EPL = D / 32;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const T* kbase = static_cast<const T*>(p.k) + b * p.k_stride_b + hkv * p.k_stride_h;
  const T* vbase = static_cast<const T*>(p.v) + b * p.v_stride_b + hkv * p.v_stride_h;

  float m_run[R], l_run[R], acc[R][EPL];
#pragma unroll
  for (int r = 0; r < R; ++r) {
    m_run[r] = -INFINITY;
    l_run[r] = 0.f;
#pragma unroll
    for (int e = 0; e < EPL; ++e) acc[r][e] = 0.f;
  }

  // Keys are taken KB at a time: the K and V rows of a batch are all requested before any
  // arithmetic, so a warp keeps 2 * KB rows (4 - 8 KB) in flight and four CTAs fit an SM; that is what hides the
  // HBM latency when the whole problem is a few megabytes.
  constexpr int KB = (R <= 2) ? 16 : 8;
  RawRow<EPL> kreg[KB], vreg[KB];
  auto load_batch = [&](int base) {
    const int last = min(KB, c1 - base) - 1;   // rows past the end repeat the last one, masked below
#pragma unroll
    for (int j = 0; j < KB; ++j)
      kreg[j] = load_raw<T, EPL>(kbase + static_cast<int64_t>(base + min(j, last)) * p.k_stride_s, lane);
#pragma unroll
    for (int j = 0; j < KB; ++j)
      vreg[j] = load_raw<T, EPL>(vbase + static_cast<int64_t>(base + min(j, last)) * p.v_stride_s, lane);
  };
  int base = c0 + warp * KB;
  if (base < c1) load_batch(base);   // in flight before anything else is fetched

  // query rows of this KV head, pre-scaled; row r = g * sq + s  (head hkv * group + g, query s)
  float qv[R][EPL];
#pragma unroll
  for (int r = 0; r < R; ++r) {
    if (r < p.rows) {
      const int g = r / p.sq, s = r % p.sq;
      const T* qrow = static_cast<const T*>(p.q) + b * p.q_stride_b +
                      static_cast<int64_t>(hkv * p.group + g) * p.q_stride_h + s * p.q_stride_s;
      load_row<T, EPL>(qrow, lane, qv[r]);
#pragma unroll
      for (int e = 0; e < EPL; ++e) qv[r][e] *= p.scale_log2;
    } else {
#pragma unroll
      for (int e = 0; e < EPL; ++e) qv[r][e] = 0.f;
    }
  }

  while (base < c1) {
    const int nk = min(KB, c1 - base);
    // scores: lane j ends up with the score of key base + j for every row
    float s_mine[R];
#pragma unroll
    for (int r = 0; r < R; ++r) s_mine[r] = -INFINITY;
#pragma unroll
    for (int j = 0; j < KB; ++j) {
      float kf[EPL];
      widen<T, EPL>(kreg[j], kf);
#pragma unroll
      for (int r = 0; r < R; ++r) {
        if (r < p.rows) {
          float part = 0.f;
#pragma unroll
          for (int e = 0; e < EPL; ++e) part = fmaf(qv[r][e], kf[e], part);
          part = warp_sum(part);
          if (lane == j) s_mine[r] = part;
        }
      }
    }
    float pr[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
      pr[r] = 0.f;
      if (r < p.rows) {
        const int kp = base + lane;
        bool valid = lane < nk;
        if (p.causal) valid = valid && (kp <= p.input_pos + (r % p.sq));
        const float s = valid ? s_mine[r] : -INFINITY;
        const float m_new = fmaxf(m_run[r], warp_max(s));
        if (m_new != -INFINITY) {   // otherwise every key so far is masked for this row
          const float corr = exp2f(m_run[r] - m_new);   // exp2(-inf) = 0 on the first block
          pr[r] = valid ? exp2f(s - m_new) : 0.f;
          l_run[r] = l_run[r] * corr + warp_sum(pr[r]);
#pragma unroll
          for (int e = 0; e < EPL; ++e) acc[r][e] *= corr;
          m_run[r] = m_new;
        }
      }
    }
#pragma unroll
    for (int j = 0; j < KB; ++j) {
      float vf[EPL];
      widen<T, EPL>(vreg[j], vf);
#pragma unroll
      for (int r = 0; r < R; ++r) {
        if (r < p.rows) {
          const float pj = __shfl_sync(0xffffffffu, pr[r], j);   // 0 for masked / repeated rows
#pragma unroll
          for (int e = 0; e < EPL; ++e) acc[r][e] = fmaf(pj, vf[e], acc[r][e]);
        }
      }
    }
    base += WARPS * KB;
    if (base < c1) load_batch(base);
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
#pragma unroll
    for (int e = 0; e < EPL; ++e) sm_acc[warp][r][lane * EPL + e] = acc[r][e];
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
__global__ void __launch_bounds__(kDecThreads, 4)
fmha_decode_kernel(const DecodeParams p) {
  __shared__ float cta_ml[2 * R];
  __shared__ float cta_acc[R * D];
  const int split = blockIdx.x;
  const int b = blockIdx.y / p.heads_kv, hkv = blockIdx.y % p.heads_kv;
  const int c0 = split * p.chunk;
  decode_cta_partial<T, D, R, kDecWarps>(p, b, hkv, c0, min(p.sk, c0 + p.chunk), cta_ml, cta_acc);
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

// Split-KV, one kernel: the eight CTAs of a cluster share one (batch, KV head); after its
// chunk every CTA leaves its partial in shared memory, and each CTA merges D / 8 output
// columns of all rows by reading the eight partials over distributed shared memory.
constexpr int kClusterSplits = 8;
constexpr int kClusterThreads = 256;

template <typename T, int D, int R>
__global__ void __cluster_dims__(kClusterSplits, 1, 1) __launch_bounds__(kClusterThreads, 2)
fmha_decode_cluster_kernel(const DecodeParams p) {
  __shared__ float cta_ml[2 * R];
  __shared__ float cta_acc[R * D];
  const int split = static_cast<int>(cluster_ctarank());
  const int b = blockIdx.y / p.heads_kv, hkv = blockIdx.y % p.heads_kv;
  const int c0 = split * p.chunk;
  decode_cta_partial<T, D, R, kClusterThreads / 32>(p, b, hkv, c0, min(p.sk, c0 + p.chunk), cta_ml, cta_acc);
  cluster_sync_all();   // every partial of the cluster is in place
  constexpr int kCols = D / kClusterSplits;
  const uint32_t ml_addr = smem_u32(cta_ml), acc_addr = smem_u32(cta_acc);
  for (int idx = threadIdx.x; idx < p.rows * kCols; idx += kClusterThreads) {
    const int r = idx / kCols, d = split * kCols + idx % kCols;
    float ms[kClusterSplits];
    float m = -INFINITY;
#pragma unroll
    for (int c = 0; c < kClusterSplits; ++c) {
      ms[c] = ld_shared_cluster_f32(map_to_cta(ml_addr + 4u * r, c));
      m = fmaxf(m, ms[c]);
    }
    float l = 0.f, o = 0.f;
#pragma unroll
    for (int c = 0; c < kClusterSplits; ++c) {
      const float f = (ms[c] == -INFINITY) ? 0.f : exp2f(ms[c] - m);
      l += ld_shared_cluster_f32(map_to_cta(ml_addr + 4u * (R + r), c)) * f;
      o += ld_shared_cluster_f32(map_to_cta(acc_addr + 4u * (r * D + d), c)) * f;
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
  bool cluster;    // one kernel, eight CTAs per (batch, KV head) merged over DSMEM
};

DecodePlan plan_decode(int64_t batch, int64_t heads_kv, int64_t sk, int sms) {
  const int64_t groups = batch * heads_kv;
  DecodePlan plan;
  // enough (batch, KV head) pairs to fill the GPU with clusters of eight: no scratch, no
  // second launch
  if (groups * kClusterSplits >= sms) {
    plan.cluster = true;
    plan.splits = kClusterSplits;
    plan.chunk = static_cast<int>(ceil_div(ceil_div(sk, kClusterSplits), 16) * 16);
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
    if (p.rows <= 1) fmha_decode_cluster_kernel<T, D, 1><<<grid, kClusterThreads, 0, stream>>>(p);
    else if (p.rows <= 2) fmha_decode_cluster_kernel<T, D, 2><<<grid, kClusterThreads, 0, stream>>>(p);
    else if (p.rows <= 4) fmha_decode_cluster_kernel<T, D, 4><<<grid, kClusterThreads, 0, stream>>>(p);
    else fmha_decode_cluster_kernel<T, D, 8><<<grid, kClusterThreads, 0, stream>>>(p);
    B200K_CHECK_LAUNCH("fmha decode (cluster) launch");
    return B200K_OK;
  }
  if (p.rows <= 1) fmha_decode_kernel<T, D, 1><<<grid, kDecThreads, 0, stream>>>(p);
  else if (p.rows <= 2) fmha_decode_kernel<T, D, 2><<<grid, kDecThreads, 0, stream>>>(p);
  else if (p.rows <= 4) fmha_decode_kernel<T, D, 4><<<grid, kDecThreads, 0, stream>>>(p);
  else fmha_decode_kernel<T, D, 8><<<grid, kDecThreads, 0, stream>>>(p);
  B200K_CHECK_LAUNCH("fmha decode launch");
  fmha_decode_merge_kernel<T, D><<<static_cast<unsigned>(batch * p.heads_kv * p.rows), D, 0, stream>>>(p);
  B200K_CHECK_LAUNCH("fmha decode merge launch");
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
  return a->seq_q * a->query_group_size <= kFmhaDecodeMaxRows && a->batch * a->heads_kv <= 65535;
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
