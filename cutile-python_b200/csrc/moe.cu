// Mixture-of-experts plumbing around the grouped GEMM: routing alignment (a stable
// counting sort of token replicas by expert, padded per expert to the GEMM's row tile),
// row gather, SiLU-and-multiply and the top-k reduction.  All of it is integer / byte
// work bound by HBM (or by launch latency at small sizes); nothing here touches the
// tensor cores.
//
//   moe_align      follows moe_align_tile_size_torch (reference:
//                  test/kernels/fused_moe.py:113-173) without its host loop and device
//                  syncs: same sorted_token_ids / sorted_expert_ids, bit for bit, written
//                  into worst-case-sized buffers with the block count left on the device
//   gather_rows    A_sorted[i] = A[sorted_token_ids[i] / replicas], zero rows for the
//                  sentinel (the gather of fused_moe_kernel, test/kernels/fused_moe.py:56-68)
//   silu_and_mul   silu_and_mul_kernel (test/kernels/fused_moe.py:85-108)
//   topk_sum       torch.sum(intermediate_cache3, dim=1) (samples/MoE.py:288)
#include "common.cuh"
#include "host.h"

namespace b200k {
namespace {

constexpr int kChunk = 512;          // token replicas per warp
constexpr int kAlignWarps = 4;       // warps per block in the count / scatter kernels

template <typename IdT>
__device__ __forceinline__ int load_expert(const IdT* ids, int64_t i, int num_experts, int* status) {
  const long long e = static_cast<long long>(ids[i]);
  if (e < 0 || e >= num_experts) {
    report_status(status, 40, 0);   // routing entry outside [0, num_experts): dropped
    return -1;
  }
  return static_cast<int>(e);
}

// Pass 1: per-chunk histogram over experts.  counts[chunk * E + e].
template <typename IdT>
__global__ void __launch_bounds__(kAlignWarps * 32)
moe_count_kernel(const IdT* __restrict__ ids, int64_t total, int num_experts,
                 int* __restrict__ counts, int* status) {
  extern __shared__ int smem_counts[];
  // The alignment kernels and the row gather behind them are launched with programmatic
  // stream serialisation: each is set up while the one before it runs and waits for it in
  // pdl_wait(), which takes the launch gaps out of a chain of four short kernels.
  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int* mine = smem_counts + warp * num_experts;
  const int64_t chunk = static_cast<int64_t>(blockIdx.x) * kAlignWarps + warp;
  const int64_t begin = chunk * kChunk;
  if (begin >= total) return;
  for (int e = lane; e < num_experts; e += 32) mine[e] = 0;
  __syncwarp();
  const int64_t end = begin + kChunk < total ? begin + kChunk : total;
  // the chunk's ids are fetched up front (sixteen independent loads per lane): one load per
  // round of the loop below would put a memory latency into each of its sixteen rounds
  int mine_e[kChunk / 32];
#pragma unroll
  for (int j = 0; j < kChunk / 32; ++j) {
    const int64_t i = begin + j * 32 + lane;
    mine_e[j] = i < end ? load_expert(ids, i, num_experts, status) : -1;
  }
#pragma unroll
  for (int j = 0; j < kChunk / 32; ++j) {
    if (begin + j * 32 >= end) break;
    const int e = mine_e[j];
    const unsigned peers = __match_any_sync(0xffffffffu, e);
    if (e >= 0 && (peers & ((1u << lane) - 1)) == 0) mine[e] += __popc(peers);
    __syncwarp();
  }
  for (int e = lane; e < num_experts; e += 32) counts[chunk * num_experts + e] = mine[e];
}

// Pass 2 (one block): turns the histograms into write offsets, emits the per-block expert
// ids, the block count and every sentinel slot.
__global__ void __launch_bounds__(1024)
moe_offsets_kernel(int* __restrict__ counts, int num_chunks, int num_experts, int tile_m,
                   int64_t total, int* __restrict__ sorted_token_ids, int64_t capacity,
                   int* __restrict__ sorted_expert_ids, int64_t block_capacity,
                   int* __restrict__ num_blocks_out) {
  extern __shared__ int sm[];
  pdl_wait();
  pdl_launch_dependents();
  int* totals = sm;                      // [E] replicas per expert
  int* starts = sm + num_experts;        // [E] first slot of the expert's padded run
  int* partial = sm + 2 * num_experts;   // [groups][E] replicas per expert in a group of chunks
  __shared__ int total_blocks;
  // two-level prefix over the chunks of every expert: thread (group, expert) first sums its
  // group's chunks, a short scan over the groups follows, then each thread rewrites its
  // chunks' histogram entries as write offsets
  const int groups = max(1, static_cast<int>(blockDim.x) / num_experts);
  const int per_group = (num_chunks + groups - 1) / groups;
  for (int t = threadIdx.x; t < groups * num_experts; t += blockDim.x) {
    const int e = t % num_experts, g = t / num_experts;
    const int c0 = g * per_group, c1 = min(num_chunks, c0 + per_group);
    int sum = 0;
    for (int c = c0; c < c1; ++c) sum += counts[c * num_experts + e];
    partial[g * num_experts + e] = sum;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < num_experts; e += blockDim.x) {
    int run = 0;
    for (int g = 0; g < groups; ++g) {
      const int v = partial[g * num_experts + e];
      partial[g * num_experts + e] = run;
      run += v;
    }
    totals[e] = run;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int slot = 0;
    for (int e = 0; e < num_experts; ++e) {
      starts[e] = slot;
      slot += (totals[e] + tile_m - 1) / tile_m * tile_m;
    }
    total_blocks = slot / tile_m;
    *num_blocks_out = total_blocks;
  }
  __syncthreads();
  const int sentinel = static_cast<int>(total);
  for (int t = threadIdx.x; t < groups * num_experts; t += blockDim.x) {
    const int e = t % num_experts, g = t / num_experts;
    const int c0 = g * per_group, c1 = min(num_chunks, c0 + per_group);
    int run = starts[e] + partial[g * num_experts + e];
    for (int c = c0; c < c1; ++c) {
      const int v = counts[c * num_experts + e];
      counts[c * num_experts + e] = run;
      run += v;
    }
  }
  // expert id of every tile_m block, -1 beyond the blocks in use (skipped when the caller
  // only wants the sorted order): binary search of the padded run that holds the block
  if (sorted_expert_ids != nullptr) {
    for (int64_t b = threadIdx.x; b < block_capacity; b += blockDim.x) {
      int owner = -1;
      if (b < total_blocks) {
        const int slot = static_cast<int>(b) * tile_m;
        int lo = 0, hi = num_experts - 1;   // last expert whose run starts at or before slot
        while (lo < hi) {
          const int mid = (lo + hi + 1) >> 1;
          if (starts[mid] <= slot) lo = mid; else hi = mid - 1;
        }
        // runs of experts without replicas are empty and share their start with the next
        // run: the owner is the last expert among them that has rows
        while (lo > 0 && totals[lo] == 0) --lo;
        owner = lo;
      }
      sorted_expert_ids[b] = owner;
    }
  }
  // sentinels: the padding tail of every run and everything beyond the last block
  for (int e = 0; e < num_experts; ++e) {
    const int padded = (totals[e] + tile_m - 1) / tile_m * tile_m;
    for (int i = totals[e] + threadIdx.x; i < padded; i += blockDim.x)
      sorted_token_ids[starts[e] + i] = sentinel;
  }
  for (int64_t i = static_cast<int64_t>(total_blocks) * tile_m + threadIdx.x; i < capacity;
       i += blockDim.x)
    sorted_token_ids[i] = sentinel;
}

// Pass 3: stable scatter.  A warp walks its chunk in index order, so replicas of one
// expert keep their original order (the order torch.argsort(stable=True) gives).
template <typename IdT>
__global__ void __launch_bounds__(kAlignWarps * 32)
moe_scatter_kernel(const IdT* __restrict__ ids, int64_t total, int num_experts,
                   const int* __restrict__ offsets, int* __restrict__ sorted_token_ids,
                   int* status) {
  extern __shared__ int smem_counts[];
  pdl_wait();
  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int* next = smem_counts + warp * num_experts;
  const int64_t chunk = static_cast<int64_t>(blockIdx.x) * kAlignWarps + warp;
  const int64_t begin = chunk * kChunk;
  if (begin >= total) return;
  for (int e = lane; e < num_experts; e += 32) next[e] = offsets[chunk * num_experts + e];
  __syncwarp();
  const int64_t end = begin + kChunk < total ? begin + kChunk : total;
  int mine_e[kChunk / 32];   // fetched up front, as in the count kernel
#pragma unroll
  for (int j = 0; j < kChunk / 32; ++j) {
    const int64_t i = begin + j * 32 + lane;
    mine_e[j] = i < end ? load_expert(ids, i, num_experts, status) : -1;
  }
#pragma unroll
  for (int j = 0; j < kChunk / 32; ++j) {
    if (begin + j * 32 >= end) break;
    const int64_t i = begin + j * 32 + lane;
    const int e = mine_e[j];
    const unsigned peers = __match_any_sync(0xffffffffu, e);
    const unsigned before = peers & ((1u << lane) - 1);
    if (e >= 0) sorted_token_ids[next[e] + __popc(before)] = static_cast<int>(i);
    __syncwarp();
    if (e >= 0 && before == 0) next[e] += __popc(peers);
    __syncwarp();
  }
}

// A block copies four destination rows at a time with 16-byte vectors: their four indices are
// fetched together and every thread has four loads in flight before its first store (one row
// at a time, the chain index -> row load -> store of each row ran back to back and the copy
// was bound by that latency: 332 us for 1.07 GB of rows where the memory system takes 200).
constexpr int kGatherRowsPerTrip = 4;

__global__ void __launch_bounds__(256)
gather_rows_kernel(const uint8_t* __restrict__ src, int64_t src_rows, int64_t row_bytes,
                   int64_t src_stride, const int* __restrict__ index, int divisor,
                   const int* __restrict__ num_blocks, int tile_m, int64_t max_rows,
                   uint8_t* __restrict__ dst, int64_t dst_stride) {
  pdl_wait();
  int64_t rows = max_rows;
  if (num_blocks != nullptr) {
    const int64_t live = static_cast<int64_t>(*num_blocks) * tile_m;
    rows = live < rows ? live : rows;
  }
  const int64_t vecs = row_bytes / 16;
  for (int64_t r0 = static_cast<int64_t>(blockIdx.x) * kGatherRowsPerTrip; r0 < rows;
       r0 += static_cast<int64_t>(gridDim.x) * kGatherRowsPerTrip) {
    const uint4* in[kGatherRowsPerTrip];
    uint4* out[kGatherRowsPerTrip];
#pragma unroll
    for (int u = 0; u < kGatherRowsPerTrip; ++u) {
      const int64_t r = r0 + u;
      in[u] = nullptr;
      out[u] = nullptr;
      if (r < rows) {
        const int ix = index[r];
        const int64_t s = ix / divisor;
        out[u] = reinterpret_cast<uint4*>(dst + r * dst_stride);
        if (ix >= 0 && s < src_rows) in[u] = reinterpret_cast<const uint4*>(src + s * src_stride);
      }
    }
    for (int64_t i = threadIdx.x; i < vecs; i += blockDim.x) {
      uint4 v[kGatherRowsPerTrip];
#pragma unroll
      for (int u = 0; u < kGatherRowsPerTrip; ++u) v[u] = in[u] != nullptr ? in[u][i] : make_uint4(0, 0, 0, 0);
#pragma unroll
      for (int u = 0; u < kGatherRowsPerTrip; ++u)
        if (out[u] != nullptr) out[u][i] = v[u];
    }
  }
}

// ---- the same gather, source row by source row ---------------------------------------
// With top-k replicas every source row has k destinations scattered over the sorted order.
// Walking the destinations reads the source k times at random (134 MB of tokens do not stay in
// the L2 under 1 GB of streaming stores: the copy then moves 2 GB through DRAM); walking the
// sources reads each row once and stores it k times.  That needs the inverse of `index`.

// inv[id] = position of replica id in the sorted order (inv is preset to -1); rows whose index
// is a sentinel are zero-filled here, so that the destination is fully defined.
__global__ void __launch_bounds__(256)
invert_index_kernel(const int* __restrict__ index, int64_t ids, const int* __restrict__ num_blocks, int tile_m,
                    int64_t max_rows, int* __restrict__ inv, uint8_t* __restrict__ dst, int64_t dst_stride,
                    int64_t row_bytes) {
  pdl_wait();
  int64_t rows = max_rows;
  if (num_blocks != nullptr) {
    const int64_t live = static_cast<int64_t>(*num_blocks) * tile_m;
    rows = live < rows ? live : rows;
  }
  __shared__ int s_id[256];
  for (int64_t base = static_cast<int64_t>(blockIdx.x) * 256; base < rows; base += static_cast<int64_t>(gridDim.x) * 256) {
    const int64_t pos = base + threadIdx.x;
    int id = -1;
    if (pos < rows) {
      id = index[pos];
      if (id >= 0 && id < ids) inv[id] = static_cast<int>(pos);
      else id = -1;
    }
    s_id[threadIdx.x] = (pos < rows) ? id : 0;      // past the end: nothing to fill
    __syncthreads();
    const int64_t vecs = row_bytes / 16;
    for (int j = 0; j < 256; ++j) {
      if (s_id[j] >= 0) continue;
      uint4* out = reinterpret_cast<uint4*>(dst + (base + j) * dst_stride);
      for (int64_t i = threadIdx.x; i < vecs; i += 256) out[i] = make_uint4(0, 0, 0, 0);
    }
    __syncthreads();
  }
}

// One block per source row: the row is read once into registers (up to four 16-byte vectors per
// thread; longer rows in passes) and stored to each of its `divisor` destinations.
__global__ void __launch_bounds__(256)
scatter_rows_kernel(const uint8_t* __restrict__ src, int64_t src_rows, int64_t row_bytes, int64_t src_stride,
                    const int* __restrict__ inv, int divisor, uint8_t* __restrict__ dst, int64_t dst_stride) {
  pdl_wait();
  const int64_t vecs = row_bytes / 16;
  for (int64_t s = blockIdx.x; s < src_rows; s += gridDim.x) {
    const uint4* in = reinterpret_cast<const uint4*>(src + s * src_stride);
    for (int64_t i0 = 0; i0 < vecs; i0 += 4 * 256) {
      uint4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int64_t i = i0 + u * 256 + threadIdx.x;
        if (i < vecs) v[u] = in[i];
      }
      for (int k = 0; k < divisor; ++k) {
        const int pos = inv[s * divisor + k];
        if (pos < 0) continue;                         // a replica that is not in the sorted order
        uint4* out = reinterpret_cast<uint4*>(dst + static_cast<int64_t>(pos) * dst_stride);
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int64_t i = i0 + u * 256 + threadIdx.x;
          if (i < vecs) out[i] = v[u];
        }
      }
    }
  }
}

template <bool BF16>
__device__ __forceinline__ float2 unpack2(uint32_t w) {
  if constexpr (BF16) {
    return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w));
  } else {
    return __half22float2(*reinterpret_cast<const __half2*>(&w));
  }
}

template <bool BF16>
__device__ __forceinline__ uint32_t pack2(float a, float b) {
  return BF16 ? pack_bf16x2(a, b) : pack_f16x2(a, b);
}

// C[r, j] = silu(AB[r, j]) * AB[r, j + n]; fp32 math, one rounding.
template <bool BF16>
__global__ void __launch_bounds__(256)
silu_and_mul_kernel(const uint16_t* __restrict__ ab, int64_t rows, int64_t n, int64_t ld_ab,
                    uint16_t* __restrict__ c, int64_t ld_c) {
  const int64_t pairs = n / 2;
  const int64_t total = rows * pairs;
  for (int64_t idx = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t r = idx / pairs;
    const int64_t j = (idx - r * pairs) * 2;
    const uint32_t g = *reinterpret_cast<const uint32_t*>(ab + r * ld_ab + j);
    const uint32_t u = *reinterpret_cast<const uint32_t*>(ab + r * ld_ab + n + j);
    const float2 gf = unpack2<BF16>(g), uf = unpack2<BF16>(u);
    const float a = gf.x / (1.0f + __expf(-gf.x)) * uf.x;
    const float b = gf.y / (1.0f + __expf(-gf.y)) * uf.y;
    *reinterpret_cast<uint32_t*>(c + r * ld_c + j) = pack2<BF16>(a, b);
  }
}

// Which (token, slot) entries take part in the sum: with routing ids given, an entry whose
// expert id lies outside [0, num_experts) was dropped by the alignment, its row was never
// written, and it contributes nothing.
struct SlotFilter {
  const void* ids;
  int ids_are_int64;
  int num_experts;
  __device__ __forceinline__ bool live(int64_t entry) const {
    if (ids == nullptr) return true;
    const long long e = ids_are_int64 ? static_cast<const long long*>(ids)[entry]
                                      : static_cast<long long>(static_cast<const int*>(ids)[entry]);
    return e >= 0 && e < num_experts;
  }
};

// out[t, :] = sum_j x[t, j, :], fp32 accumulation, 8 columns per thread.
template <bool BF16>
__global__ void __launch_bounds__(256)
topk_sum_kernel(const uint16_t* __restrict__ x, const int* __restrict__ index, int64_t tokens,
                int topk, int64_t h, uint16_t* __restrict__ out, const SlotFilter filter) {
  const int64_t vecs = h / 8;
  const int64_t total = tokens * vecs;
  for (int64_t idx = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t t = idx / vecs;
    const int64_t v = idx - t * vecs;
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    // eight slots at a time: their loads are issued together (a zero vector stands in for a
    // slot that is absent or dropped), then summed in slot order
    for (int j0 = 0; j0 < topk; j0 += 8) {
      uint4 q[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int j = j0 + u;
        q[u] = make_uint4(0u, 0u, 0u, 0u);
        if (j < topk && filter.live(t * topk + j)) {
          const int64_t src = index != nullptr ? index[t * topk + j] : t * topk + j;
          q[u] = *reinterpret_cast<const uint4*>(x + src * h + v * 8);
        }
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const uint32_t w[4] = {q[u].x, q[u].y, q[u].z, q[u].w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 f = unpack2<BF16>(w[i]);
          acc[2 * i] += f.x;
          acc[2 * i + 1] += f.y;
        }
      }
    }
    uint4 o;
    o.x = pack2<BF16>(acc[0], acc[1]);
    o.y = pack2<BF16>(acc[2], acc[3]);
    o.z = pack2<BF16>(acc[4], acc[5]);
    o.w = pack2<BF16>(acc[6], acc[7]);
    *reinterpret_cast<uint4*>(out + t * h + v * 8) = o;
  }
}

// fp32 forms of the two kernels above (the grouped GEMMs multiply fp32 operands as tf32 and
// keep fp32 results; these stay in fp32 throughout).
__global__ void __launch_bounds__(256)
silu_and_mul_f32_kernel(const float* __restrict__ ab, int64_t rows, int64_t n, int64_t ld_ab,
                        float* __restrict__ c, int64_t ld_c) {
  const int64_t pairs = n / 2;
  const int64_t total = rows * pairs;
  for (int64_t idx = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t r = idx / pairs;
    const int64_t j = (idx - r * pairs) * 2;
    const float2 gf = *reinterpret_cast<const float2*>(ab + r * ld_ab + j);
    const float2 uf = *reinterpret_cast<const float2*>(ab + r * ld_ab + n + j);
    float2 o;
    o.x = gf.x / (1.0f + __expf(-gf.x)) * uf.x;
    o.y = gf.y / (1.0f + __expf(-gf.y)) * uf.y;
    *reinterpret_cast<float2*>(c + r * ld_c + j) = o;
  }
}

__global__ void __launch_bounds__(256)
topk_sum_f32_kernel(const float* __restrict__ x, const int* __restrict__ index, int64_t tokens, int topk,
                    int64_t h, float* __restrict__ out, const SlotFilter filter) {
  const int64_t vecs = h / 4;
  const int64_t total = tokens * vecs;
  for (int64_t idx = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t t = idx / vecs;
    const int64_t v = idx - t * vecs;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int j = 0; j < topk; ++j) {
      if (!filter.live(t * topk + j)) continue;
      const int64_t src = index != nullptr ? index[t * topk + j] : t * topk + j;
      const float4 q = *reinterpret_cast<const float4*>(x + src * h + v * 4);
      acc.x += q.x;
      acc.y += q.y;
      acc.z += q.z;
      acc.w += q.w;
    }
    *reinterpret_cast<float4*>(out + t * h + v * 4) = acc;
  }
}

// Any hidden size / alignment: one output element per thread.  DT: 0 = f16, 1 = bf16, 2 = f32.
template <int DT>
__global__ void __launch_bounds__(256)
topk_sum_scalar_kernel(const void* __restrict__ x_, const int* __restrict__ index, int64_t tokens, int topk,
                       int64_t h, void* __restrict__ out_, const SlotFilter filter) {
  const int64_t total = tokens * h;
  for (int64_t idx = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t t = idx / h;
    const int64_t c = idx - t * h;
    float acc = 0.0f;
    for (int j = 0; j < topk; ++j) {
      if (!filter.live(t * topk + j)) continue;
      const int64_t src = index != nullptr ? index[t * topk + j] : t * topk + j;
      if constexpr (DT == 2) acc += static_cast<const float*>(x_)[src * h + c];
      else if constexpr (DT == 1) acc += __bfloat162float(static_cast<const __nv_bfloat16*>(x_)[src * h + c]);
      else acc += __half2float(static_cast<const __half*>(x_)[src * h + c]);
    }
    if constexpr (DT == 2) static_cast<float*>(out_)[idx] = acc;
    else if constexpr (DT == 1) static_cast<__nv_bfloat16*>(out_)[idx] = __float2bfloat16_rn(acc);
    else static_cast<__half*>(out_)[idx] = __float2half_rn(acc);
  }
}

int blocks_for(int64_t items, int threads, int per_sm = 8) {
  int sms = current_sm_count();
  if (sms <= 0) sms = 148;
  int64_t b = ceil_div(items, threads);
  int64_t cap = static_cast<int64_t>(sms) * per_sm;
  if (b < 1) b = 1;
  return static_cast<int>(b < cap ? b : cap);
}

}  // namespace
}  // namespace b200k

using namespace b200k;

extern "C" int64_t b200k_moe_align_workspace_bytes(int64_t num_replicas, int32_t num_experts) {
  if (num_replicas < 0 || num_experts <= 0) return 0;
  const int64_t chunks = ceil_div(num_replicas > 0 ? num_replicas : 1, kChunk);
  return chunks * num_experts * static_cast<int64_t>(sizeof(int));
}

extern "C" int b200k_moe_align(const b200k_moe_align_args* a, b200k_stream stream_) {
  if (a == nullptr) return fail(B200K_INVALID_ARG, "null args");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (a->num_replicas < 0 || a->num_experts <= 0 || a->tile_m <= 0)
    return fail(B200K_INVALID_ARG, "bad sizes");
  if (a->num_experts > 2048) return fail(B200K_UNSUPPORTED, "at most 2048 experts");
  if (a->num_replicas >= INT32_MAX) return fail(B200K_UNSUPPORTED, "too many token replicas");
  if (!a->sorted_token_ids || !a->num_blocks || !a->workspace)
    return fail(B200K_INVALID_ARG, "null pointer");
  if (a->num_replicas > 0 && !a->topk_ids) return fail(B200K_INVALID_ARG, "null topk_ids");
  // worst case: every expert wastes tile_m - 1 slots
  const int64_t need = a->num_replicas + static_cast<int64_t>(a->num_experts) * (a->tile_m - 1);
  const int64_t need_blocks = ceil_div(need, a->tile_m);
  if (a->capacity < need_blocks * a->tile_m || a->block_capacity < need_blocks)
    return fail(B200K_INVALID_ARG, "capacity %lld / %lld too small: need %lld slots, %lld blocks",
                (long long)a->capacity, (long long)a->block_capacity,
                (long long)(need_blocks * a->tile_m), (long long)need_blocks);
  const int chunks = static_cast<int>(ceil_div(a->num_replicas > 0 ? a->num_replicas : 1, kChunk));
  if (a->workspace_bytes < static_cast<int64_t>(chunks) * a->num_experts * 4)
    return fail(B200K_INVALID_ARG, "workspace too small");
  int* counts = static_cast<int*>(a->workspace);
  int* status = device_status_word();
  const int grid = static_cast<int>(ceil_div(chunks, kAlignWarps));
  const size_t smem = static_cast<size_t>(kAlignWarps) * a->num_experts * sizeof(int);
  cudaError_t e = cudaMemsetAsync(counts, 0, static_cast<size_t>(chunks) * a->num_experts * 4, stream);
  if (e != cudaSuccess) return fail(B200K_CUDA_ERROR, "memset: %s", cudaGetErrorString(e));
  if (a->num_replicas > 0) {
    if (a->ids_are_int64)
      moe_count_kernel<long long><<<grid, kAlignWarps * 32, smem, stream>>>(
          static_cast<const long long*>(a->topk_ids), a->num_replicas, a->num_experts, counts, status);
    else
      moe_count_kernel<int><<<grid, kAlignWarps * 32, smem, stream>>>(
          static_cast<const int*>(a->topk_ids), a->num_replicas, a->num_experts, counts, status);
  }
  const size_t offsets_smem =
      (2 + (1024 / a->num_experts > 1 ? 1024 / a->num_experts : 1)) * a->num_experts * sizeof(int);
  e = launch_after_predecessor(moe_offsets_kernel, dim3(1), dim3(1024), offsets_smem, stream, counts, chunks,
                               a->num_experts, a->tile_m, a->num_replicas, a->sorted_token_ids, a->capacity,
                               a->sorted_expert_ids, a->block_capacity, a->num_blocks);
  if (e == cudaSuccess && a->num_replicas > 0) {
    if (a->ids_are_int64)
      e = launch_after_predecessor(moe_scatter_kernel<long long>, dim3(grid), dim3(kAlignWarps * 32), smem, stream,
                                   static_cast<const long long*>(a->topk_ids), a->num_replicas, a->num_experts,
                                   counts, a->sorted_token_ids, status);
    else
      e = launch_after_predecessor(moe_scatter_kernel<int>, dim3(grid), dim3(kAlignWarps * 32), smem, stream,
                                   static_cast<const int*>(a->topk_ids), a->num_replicas, a->num_experts, counts,
                                   a->sorted_token_ids, status);
  }
  if (e != cudaSuccess) return fail(B200K_CUDA_ERROR, "moe_align launch: %s", cudaGetErrorString(e));
  B200K_CHECK_LAUNCH("moe_align launch");
  return B200K_OK;
}

extern "C" int b200k_gather_rows(const void* src, int64_t src_rows, int64_t row_bytes,
                                 int64_t src_stride_bytes, const int32_t* index, int32_t divisor,
                                 const int32_t* num_blocks, int32_t tile_m, int64_t max_rows,
                                 void* dst, int64_t dst_stride_bytes, b200k_stream stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (max_rows < 0 || row_bytes < 0 || divisor <= 0) return fail(B200K_INVALID_ARG, "bad sizes");
  if (max_rows == 0 || row_bytes == 0) return B200K_OK;
  if (!src || !index || !dst) return fail(B200K_INVALID_ARG, "null pointer");
  if (row_bytes % 16 || src_stride_bytes % 16 || dst_stride_bytes % 16 ||
      (reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) % 16)
    return fail(B200K_UNSUPPORTED, "rows must be multiples of 16 bytes on 16-byte boundaries");
  const int grid = blocks_for(ceil_div(max_rows, kGatherRowsPerTrip) * 256, 256, 16);
  const cudaError_t e = launch_after_predecessor(gather_rows_kernel, dim3(grid), dim3(256), 0, stream,
                                                 static_cast<const uint8_t*>(src), src_rows, row_bytes,
                                                 src_stride_bytes, index, divisor, num_blocks, tile_m, max_rows,
                                                 static_cast<uint8_t*>(dst), dst_stride_bytes);
  if (e != cudaSuccess) return fail(B200K_CUDA_ERROR, "gather_rows launch: %s", cudaGetErrorString(e));
  return B200K_OK;
}

extern "C" int b200k_gather_rows_by_source(const void* src, int64_t src_rows, int64_t row_bytes,
                                           int64_t src_stride_bytes, const int32_t* index, int32_t divisor,
                                           const int32_t* num_blocks, int32_t tile_m, int64_t max_rows,
                                           void* dst, int64_t dst_stride_bytes, int32_t* scratch,
                                           b200k_stream stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (src_rows < 0 || row_bytes < 0 || max_rows < 0 || divisor <= 0)
    return fail(B200K_INVALID_ARG, "bad sizes");
  if (max_rows == 0 || row_bytes == 0) return B200K_OK;
  if (!src || !index || !dst || !scratch) return fail(B200K_INVALID_ARG, "null pointer");
  if (row_bytes % 16 || src_stride_bytes % 16 || dst_stride_bytes % 16 ||
      (reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) % 16)
    return fail(B200K_UNSUPPORTED, "rows must be multiples of 16 bytes on 16-byte boundaries");
  const int64_t ids = src_rows * divisor;
  if (ids > INT32_MAX || max_rows > INT32_MAX) return fail(B200K_UNSUPPORTED, "more than 2^31 rows");
  if (ids > 0) {
    const cudaError_t em = cudaMemsetAsync(scratch, 0xff, static_cast<size_t>(ids) * sizeof(int32_t), stream);
    if (em != cudaSuccess) return fail(B200K_CUDA_ERROR, "memset: %s", cudaGetErrorString(em));
  }
  invert_index_kernel<<<blocks_for(max_rows, 256, 8), 256, 0, stream>>>(
      index, ids, num_blocks, tile_m, max_rows, scratch, static_cast<uint8_t*>(dst), dst_stride_bytes, row_bytes);
  B200K_CHECK_LAUNCH("invert_index launch");
  if (src_rows > 0) {
    scatter_rows_kernel<<<blocks_for(src_rows * 256, 256, 8), 256, 0, stream>>>(
        static_cast<const uint8_t*>(src), src_rows, row_bytes, src_stride_bytes, scratch, divisor,
        static_cast<uint8_t*>(dst), dst_stride_bytes);
    B200K_CHECK_LAUNCH("scatter_rows launch");
  }
  return B200K_OK;
}

extern "C" int b200k_silu_and_mul(const void* ab, int64_t rows, int64_t n, int64_t ld_ab, void* c,
                                  int64_t ld_c, int32_t dtype, b200k_stream stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (rows < 0 || n < 0) return fail(B200K_INVALID_ARG, "negative dimension");
  if (rows == 0 || n == 0) return B200K_OK;
  if (!ab || !c) return fail(B200K_INVALID_ARG, "null pointer");
  if (n % 2 || ld_ab % 2 || ld_c % 2 ||
      (reinterpret_cast<uintptr_t>(ab) | reinterpret_cast<uintptr_t>(c)) % (dtype == B200K_F32 ? 8 : 4))
    return fail(B200K_UNSUPPORTED, "columns and leading dimensions must be even");
  const int grid = blocks_for(rows * n / 2, 256);
  if (dtype == B200K_F32)
    silu_and_mul_f32_kernel<<<grid, 256, 0, stream>>>(static_cast<const float*>(ab), rows, n, ld_ab,
                                                      static_cast<float*>(c), ld_c);
  else if (dtype == B200K_BF16)
    silu_and_mul_kernel<true><<<grid, 256, 0, stream>>>(static_cast<const uint16_t*>(ab), rows, n, ld_ab,
                                                        static_cast<uint16_t*>(c), ld_c);
  else if (dtype == B200K_F16)
    silu_and_mul_kernel<false><<<grid, 256, 0, stream>>>(static_cast<const uint16_t*>(ab), rows, n, ld_ab,
                                                         static_cast<uint16_t*>(c), ld_c);
  else
    return fail(B200K_INVALID_ARG, "dtype must be f16, bf16 or f32");
  B200K_CHECK_LAUNCH("silu_and_mul launch");
  return B200K_OK;
}

extern "C" int b200k_topk_sum(const void* x, const int32_t* index, int64_t tokens, int32_t topk,
                              int64_t hidden, void* out, int32_t dtype, const void* expert_ids,
                              int32_t ids_are_int64, int32_t num_experts, b200k_stream stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (tokens < 0 || topk <= 0 || hidden < 0) return fail(B200K_INVALID_ARG, "bad sizes");
  if (tokens == 0 || hidden == 0) return B200K_OK;
  if (!x || !out) return fail(B200K_INVALID_ARG, "null pointer");
  if (dtype != B200K_F32 && dtype != B200K_BF16 && dtype != B200K_F16)
    return fail(B200K_INVALID_ARG, "dtype must be f16, bf16 or f32");
  const SlotFilter filter = {expert_ids, ids_are_int64, num_experts};
  const bool vectors = hidden % 8 == 0 &&
                       (reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(out)) % 16 == 0;
  if (!vectors) {   // odd hidden sizes or unaligned buffers: one element per thread
    const int grid = blocks_for(tokens * hidden, 256);
    if (dtype == B200K_F32)
      topk_sum_scalar_kernel<2><<<grid, 256, 0, stream>>>(x, index, tokens, topk, hidden, out, filter);
    else if (dtype == B200K_BF16)
      topk_sum_scalar_kernel<1><<<grid, 256, 0, stream>>>(x, index, tokens, topk, hidden, out, filter);
    else
      topk_sum_scalar_kernel<0><<<grid, 256, 0, stream>>>(x, index, tokens, topk, hidden, out, filter);
    B200K_CHECK_LAUNCH("topk_sum launch");
    return B200K_OK;
  }
  const int grid = blocks_for(tokens * hidden / 8, 256);
  if (dtype == B200K_F32)
    topk_sum_f32_kernel<<<grid, 256, 0, stream>>>(static_cast<const float*>(x), index, tokens, topk, hidden,
                                                  static_cast<float*>(out), filter);
  else if (dtype == B200K_BF16)
    topk_sum_kernel<true><<<grid, 256, 0, stream>>>(static_cast<const uint16_t*>(x), index, tokens, topk, hidden,
                                                    static_cast<uint16_t*>(out), filter);
  else
    topk_sum_kernel<false><<<grid, 256, 0, stream>>>(static_cast<const uint16_t*>(x), index, tokens, topk, hidden,
                                                     static_cast<uint16_t*>(out), filter);
  B200K_CHECK_LAUNCH("topk_sum launch");
  return B200K_OK;
}
