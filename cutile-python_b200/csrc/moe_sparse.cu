// MoE FFN for sparse routing: about one token per expert (the reference's second bench shape,
// test/bench_moe.py:16-19: 256 tokens x 1408 experts x top-6, intermediate 32).  On the
// grouped tensor-core path every routed expert costs a 128-row tile that holds one real row;
// here every token replica streams its expert's weights once through the CUDA cores instead
// (two matrix-vector products per replica), which is what the problem is: HBM-bound, the
// algorithmic bytes are the routed experts' weights.  Same arithmetic as the dense path of
// cutile_moe (samples/MoE.py:197-288): fp32 accumulation, SiLU(gate) * up rounded to the
// activation type, down projection scaled by the routing weight and rounded, top-k sum after.
//
//   moe_sparse_up    act[r, i] = silu(W1[e][i, :] . x[t]) * (W1[e][I + i, :] . x[t])
//   moe_sparse_down  y[r, h]   = w[r] * (W2[e][h, :] . act[r, :])
// with r = t * topk + slot and e = topk_ids[r]; replicas routed outside [0, experts) give
// zero rows.  A group of G lanes (G = 4, 8, 16 or 32 by the length of a weight row) owns one
// output element and walks its weight row in 16-byte vectors against the input vector in
// shared memory (in its own type, unpacked to fp32 at use); rows of at most eight vectors take
// one lane per row with the input in registers.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "common.cuh"
#include "host.h"

namespace b200k {
namespace {

template <typename T> struct Vec16;
template <> struct Vec16<__nv_bfloat16> { static constexpr int kElems = 8; };
template <> struct Vec16<__half> { static constexpr int kElems = 8; };
template <> struct Vec16<float> { static constexpr int kElems = 4; };

template <typename T>
__device__ __forceinline__ void unpack16(const uint4& q, float (&f)[Vec16<T>::kElems]) {
  if constexpr (sizeof(T) == 4) {
    f[0] = __uint_as_float(q.x); f[1] = __uint_as_float(q.y);
    f[2] = __uint_as_float(q.z); f[3] = __uint_as_float(q.w);
  } else {
    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      if constexpr (std::is_same<T, __nv_bfloat16>::value) {
        f[2 * i] = __uint_as_float(w[i] << 16);
        f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
      } else {
        const __half2 h = *reinterpret_cast<const __half2*>(&w[i]);
        const float2 v = __half22float2(h);
        f[2 * i] = v.x;
        f[2 * i + 1] = v.y;
      }
    }
  }
}

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }

// dot of one weight row (k elements, 16-byte aligned) with the input vector in shared memory
// (kept in its own type: a 16-byte weight vector meets one 16-byte read of the input), over
// the G lanes of a group; every lane of the group returns the sum.
template <typename T, int G>
__device__ __forceinline__ float group_dot(const T* __restrict__ row, const T* __restrict__ vec, int k,
                                           int lane_in_group) {
  constexpr int E = Vec16<T>::kElems;
  float acc = 0.0f;
  const uint4* r4 = reinterpret_cast<const uint4*>(row);
  const uint4* v4 = reinterpret_cast<const uint4*>(vec);
  for (int v = lane_in_group; v * E < k; v += G) {
    const uint4 q = __ldg(r4 + v);
    float f[E], x[E];
    unpack16<T>(q, f);
    unpack16<T>(v4[v], x);
#pragma unroll
    for (int i = 0; i < E; ++i) acc = fmaf(f[i], x[i], acc);
  }
#pragma unroll
  for (int o = G / 2; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o, G);
  return acc;
}

// The same dot product with the lane's share of the input vector held in registers: lane l of
// a group owns the 16-byte vectors l, l + G, ... of every row, VPL of them, so its slice of
// the (fp32) input is loaded once per block instead of being read from shared memory for
// every weight vector (twice the bytes of the weights themselves).
template <typename T, int G, int VPL>
__device__ __forceinline__ float group_dot_reg(const T* __restrict__ row,
                                               const float (&xr)[VPL * Vec16<T>::kElems], int lane_in_group) {
  constexpr int E = Vec16<T>::kElems;
  const uint4* r4 = reinterpret_cast<const uint4*>(row);
  uint4 q[VPL];
#pragma unroll
  for (int j = 0; j < VPL; ++j) q[j] = __ldg(r4 + lane_in_group + j * G);
  float acc = 0.0f;
#pragma unroll
  for (int j = 0; j < VPL; ++j) {
    float f[E];
    unpack16<T>(q[j], f);
#pragma unroll
    for (int i = 0; i < E; ++i) acc = fmaf(f[i], xr[j * E + i], acc);
  }
#pragma unroll
  for (int o = G / 2; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o, G);
  return acc;
}

template <typename IdT>
__device__ __forceinline__ long long load_id(const void* ids, int64_t r) {
  return static_cast<long long>(static_cast<const IdT*>(ids)[r]);
}

// grid (row blocks, replicas); UP: rows are the I (gate, up) pairs of W1, k = hidden;
// otherwise rows are the hidden rows of W2, k = intermediate.
// VPL > 0: a weight row is exactly G * VPL 16-byte vectors and the lane's slice of the input
// lives in registers (used with G = 1: short rows); VPL == 0: any row length, input in shared
// memory.
template <typename T, int G, bool UP, int VPL>
__global__ void __launch_bounds__(256)
moe_sparse_kernel(const T* __restrict__ in, int64_t in_stride, const T* __restrict__ w, int64_t w_stride_e,
                  int64_t w_ld, const void* __restrict__ ids, int ids_are_int64, const float* __restrict__ route_w,
                  int topk, int experts, int rows, int k, T* __restrict__ out, int64_t out_stride, int* status) {
  extern __shared__ __align__(16) uint8_t s_raw[];
  T* s_vec = reinterpret_cast<T*>(s_raw);
  const int64_t r = blockIdx.y;
  const long long e = ids_are_int64 ? load_id<long long>(ids, r) : load_id<int>(ids, r);
  const bool live = e >= 0 && e < experts;
  const int groups = blockDim.x / G;
  const int g = threadIdx.x / G, lg = threadIdx.x % G;
  const int rows_per_block = (rows + gridDim.x - 1) / gridDim.x;
  const int row0 = blockIdx.x * rows_per_block;
  const int row1 = min(rows, row0 + rows_per_block);
  T* o = out + r * out_stride;
  if (!live) {      // dropped entry: a defined (zero) row, recorded like the alignment does
    if (UP && blockIdx.x == 0 && threadIdx.x == 0) report_status(status, 40, 0);
    for (int j = row0 + threadIdx.x; j < row1; j += blockDim.x) o[j] = from_f32<T>(0.0f);
    return;
  }
  // UP reads token r / topk of the hidden states, DOWN reads replica r of the activations
  const T* v = in + (UP ? r / topk : r) * in_stride;
  constexpr int E = Vec16<T>::kElems;
  float xr[(VPL > 0 ? VPL : 1) * E];
  if constexpr (VPL > 0) {
#pragma unroll
    for (int j = 0; j < VPL; ++j) {
      const uint4 q = *reinterpret_cast<const uint4*>(v + static_cast<int64_t>(lg + j * G) * E);
      float f[E];
      unpack16<T>(q, f);
#pragma unroll
      for (int i = 0; i < E; ++i) xr[j * E + i] = f[i];
    }
  } else {
    for (int i = threadIdx.x; i < k; i += blockDim.x) s_vec[i] = v[i];
    __syncthreads();
  }
  auto dot = [&](const T* row) {
    if constexpr (VPL > 0) return group_dot_reg<T, G, VPL>(row, xr, lg);
    else return group_dot<T, G>(row, s_vec, k, lg);
  };
  const T* we = w + e * w_stride_e;
  const float scale = UP ? 1.0f : (route_w != nullptr ? route_w[r] : 1.0f);
  // every group of a warp takes the same number of trips (the shuffles inside group_dot are
  // warp-wide): a group past the last row recomputes that row and does not store
  for (int j0 = row0; j0 < row1; j0 += groups) {
    const bool mine = j0 + g < row1;
    const int j = mine ? j0 + g : row1 - 1;
    if constexpr (UP) {
      const float gate = dot(we + static_cast<int64_t>(j) * w_ld);
      const float up = dot(we + static_cast<int64_t>(rows + j) * w_ld);
      // rounded to the activation type exactly where the dense path rounds it
      if (mine && lg == 0) o[j] = from_f32<T>(__fdividef(gate, 1.0f + __expf(-gate)) * up);
    } else {
      const float y = dot(we + static_cast<int64_t>(j) * w_ld);
      if (mine && lg == 0) o[j] = from_f32<T>(y * scale);
    }
  }
}

template <typename T, bool UP>
int launch_sparse(const b200k_moe_sparse_args* a, cudaStream_t stream) {
  const int rows = static_cast<int>(UP ? a->intermediate : a->hidden);
  const int k = static_cast<int>(UP ? a->hidden : a->intermediate);
  const T* in = static_cast<const T*>(UP ? a->hidden_states : a->act);
  const int64_t in_stride = UP ? a->hidden_stride : a->intermediate;
  const T* w = static_cast<const T*>(UP ? a->w1 : a->w2);
  const int64_t w_stride_e = UP ? a->w1_stride_e : a->w2_stride_e;
  const int64_t w_ld = UP ? a->w1_ld : a->w2_ld;
  T* out = static_cast<T*>(UP ? a->act : a->per_replica);
  const int64_t out_stride = UP ? a->intermediate : a->hidden;
  const int vecs = k / Vec16<T>::kElems;          // 16-byte vectors per weight row
  const int64_t replicas = a->tokens * a->topk;
  // rows per block: enough blocks to fill the GPU, no fewer than one pass of the block's groups
  int sms = current_sm_count();
  if (sms <= 0) sms = 148;
  // the input vector must be readable as 16-byte vectors for the register form
  const bool in_vec_ok = reinterpret_cast<uintptr_t>(in) % 16 == 0 && (in_stride * sizeof(T)) % 16 == 0;
  auto launch = [&](auto group_tag, auto vpl_tag) {
    constexpr int G = decltype(group_tag)::value;
    constexpr int VPL = decltype(vpl_tag)::value;
    const int groups = 256 / G;
    int64_t want_blocks = ceil_div(static_cast<int64_t>(sms) * 8, replicas);
    const int64_t max_blocks = ceil_div(rows, groups);
    if (want_blocks > max_blocks) want_blocks = max_blocks;
    if (want_blocks < 1) want_blocks = 1;
    const dim3 grid(static_cast<unsigned>(want_blocks), static_cast<unsigned>(replicas));
    const size_t smem = VPL > 0 ? 0 : static_cast<size_t>(k) * sizeof(T);
    moe_sparse_kernel<T, G, UP, VPL><<<grid, 256, smem, stream>>>(
        in, in_stride, w, w_stride_e, w_ld, a->topk_ids, a->ids_are_int64, a->topk_weights, a->topk,
        a->num_experts, rows, k, out, out_stride, device_status_word());
  };
  using std::integral_constant;
  // rows of at most eight vectors (the down projection of a narrow expert): one lane per row, no
  // shuffles, the whole input in registers; longer rows: a lane group per row, the input in
  // shared memory in its own type (held as fp32 there it cost twice the bytes of the weights;
  // a lane's slice held in registers instead leaves too few warps per SM: 131 against 108 us
  // for the whole step at 256 tokens x 1408 experts x top-6)
  if (in_vec_ok && (vecs == 1 || vecs == 2 || vecs == 4 || vecs == 8)) {
    if (vecs == 8) launch(integral_constant<int, 1>(), integral_constant<int, 8>());
    else if (vecs == 4) launch(integral_constant<int, 1>(), integral_constant<int, 4>());
    else if (vecs == 2) launch(integral_constant<int, 1>(), integral_constant<int, 2>());
    else launch(integral_constant<int, 1>(), integral_constant<int, 1>());
  }
  else if (vecs >= 32) launch(integral_constant<int, 32>(), integral_constant<int, 0>());
  else if (vecs >= 16) launch(integral_constant<int, 16>(), integral_constant<int, 0>());
  else if (vecs >= 8) launch(integral_constant<int, 8>(), integral_constant<int, 0>());
  else launch(integral_constant<int, 4>(), integral_constant<int, 0>());
  B200K_CHECK_LAUNCH("moe_sparse launch");
  return B200K_OK;
}

template <typename T>
int run_sparse(const b200k_moe_sparse_args* a, cudaStream_t stream) {
  if (int rc = launch_sparse<T, true>(a, stream)) return rc;
  return launch_sparse<T, false>(a, stream);
}

}  // namespace
}  // namespace b200k

using namespace b200k;

extern "C" int b200k_moe_sparse(const b200k_moe_sparse_args* a, b200k_stream stream_) {
  if (a == nullptr) return fail(B200K_INVALID_ARG, "null args");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (a->tokens < 0 || a->topk <= 0 || a->hidden <= 0 || a->intermediate <= 0 || a->num_experts <= 0)
    return fail(B200K_INVALID_ARG, "bad sizes");
  if (a->tokens == 0) return B200K_OK;
  if (a->tokens * a->topk > 65535) return fail(B200K_UNSUPPORTED, "at most 65535 token replicas on this path");
  if (!a->hidden_states || !a->w1 || !a->w2 || !a->topk_ids || !a->act || !a->per_replica)
    return fail(B200K_INVALID_ARG, "null pointer");
  const int esz = a->dtype == B200K_F32 ? 4 : 2;
  if (a->dtype != B200K_F32 && a->dtype != B200K_BF16 && a->dtype != B200K_F16)
    return fail(B200K_INVALID_ARG, "dtype must be f16, bf16 or f32");
  const int per = 16 / esz;
  if (a->hidden % per || a->intermediate % per || a->w1_ld % per || a->w2_ld % per || a->w1_stride_e % per ||
      a->w2_stride_e % per || reinterpret_cast<uintptr_t>(a->w1) % 16 || reinterpret_cast<uintptr_t>(a->w2) % 16)
    return fail(B200K_UNSUPPORTED, "weight rows must be multiples of 16 bytes on 16-byte boundaries");
  if (a->hidden * 4 > 48 * 1024 || a->intermediate * 4 > 48 * 1024)
    return fail(B200K_UNSUPPORTED, "hidden / intermediate size above 12288 is not supported on this path");
  switch (a->dtype) {
    case B200K_F32: return run_sparse<float>(a, stream);
    case B200K_BF16: return run_sparse<__nv_bfloat16>(a, stream);
    default: return run_sparse<__half>(a, stream);
  }
}
