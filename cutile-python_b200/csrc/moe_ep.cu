// Expert-parallel MoE plumbing: experts sharded over the ranks of one node, tokens sharded
// over the same ranks, rows exchanged over NVLink by plain peer stores from these kernels.
//
// The reference has no multi-GPU MoE (its only distributed code is the AllGather sample);
// the single-GPU pipeline this must equal is samples/MoE.py:197-288.  Per layer and rank:
//
//   ep_count     histogram of this rank's routing ids per (global) expert, written into every
//                rank's table hist[world][experts]                       (push, experts ints)
//   -- barrier --
//   ep_plan      from the table: where this rank's rows for each expert start in the owner's
//                receive buffer (moe_ep_plan.h), and for the experts this rank owns the tile
//                list of the grouped GEMM (expert per row tile, live tile count, padding rows
//                marked)
//   ep_dispatch  one warp per token replica: the token's row (already quantised once per
//                token when the experts are MXFP8: e4m3 codes + one row of scale bytes) is
//                stored into the owner's receive buffer at its final, tile-aligned position,
//                together with the id of the replica it came from and its routing weight
//   -- barrier --
//   grouped GEMMs on the received rows; the down projection's epilogue stores every result
//   row straight into the y buffer of the rank the row came from (b200k_gemm c_peers)
//   -- barrier --
//   top-k sum on the source rank
//
// Counts never leave the device and nothing is read back by the host.  The barrier is a
// kernel of its own between the phases (every rank launches it; ranks are on different
// GPUs): flags in peer memory, monotonic epochs, a bounded wait that reports through the
// status word instead of spinning forever.
#include "common.cuh"
#include "host.h"
#include "moe_ep_plan.h"

namespace b200k {
namespace {

constexpr int kMaxPeers = 16;
constexpr int kMaxExperts = 2048;

struct PeerInts {
  int32_t* p[kMaxPeers];
};

template <typename IdT>
__global__ void __launch_bounds__(256)
ep_count_kernel(const IdT* __restrict__ ids, int64_t total, int experts, int32_t* __restrict__ hist_local,
                unsigned int* __restrict__ ticket, PeerInts peers, int world, int rank, int* status) {
  extern __shared__ int32_t s_hist[];
  for (int e = threadIdx.x; e < experts; e += blockDim.x) s_hist[e] = 0;
  __syncthreads();
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const long long e = static_cast<long long>(ids[i]);
    if (e < 0 || e >= experts) {
      report_status(status, 40, 0);   // routing entry outside [0, experts): dropped
      continue;
    }
    atomicAdd(&s_hist[e], 1);
  }
  __syncthreads();
  for (int e = threadIdx.x; e < experts; e += blockDim.x)
    if (s_hist[e] != 0) atomicAdd(&hist_local[e], s_hist[e]);
  __threadfence();
  __syncthreads();
  __shared__ bool last;
  if (threadIdx.x == 0) last = atomicAdd(ticket, 1u) == gridDim.x - 1;
  __syncthreads();
  if (!last) return;
  // the last block to finish publishes the table row to every rank and clears the scratch
  // for the next call
  __threadfence();
  for (int e = threadIdx.x; e < experts; e += blockDim.x) {
    const int32_t v = atomicExch(&hist_local[e], 0);
    for (int p = 0; p < world; ++p) peers.p[p][static_cast<int64_t>(rank) * experts + e] = v;
  }
  if (threadIdx.x == 0) *ticket = 0;
}

// One warp per expert (the lanes compute the same few sums, then share the stores: up to a
// tile of padding marks and the expert's tile list).
__global__ void __launch_bounds__(1024)
ep_plan_kernel(const int32_t* __restrict__ hist, int world, int rank, int experts, int tile,
               int64_t capacity_rows, int64_t* __restrict__ first_row, int32_t* __restrict__ cursor,
               int32_t* __restrict__ tile_group, int32_t* __restrict__ num_row_tiles,
               int32_t* __restrict__ meta, int* status) {
  const int local = experts / world;
  const int lane = threadIdx.x & 31;
  for (int e = threadIdx.x >> 5; e < experts; e += blockDim.x >> 5) {
    const int64_t start = ep_tile_start(hist, world, experts, local, tile, e);
    if (lane == 0) {
      first_row[e] = start * tile + ep_before(hist, experts, rank, e);
      cursor[e] = 0;
    }
    if (ep_owner(e, local) != rank) continue;
    // an expert this rank owns: its row tiles, and the padding rows behind its last real row
    const int64_t total = ep_total(hist, world, experts, e);
    const int64_t tiles = ep_tiles(total, tile);
    const bool last = e == (rank + 1) * local - 1;
    if ((start + tiles) * tile > capacity_rows) {
      if (lane == 0) {
        report_status(status, 61, e);   // more rows than the receive buffer holds: plan nothing
        if (last) *num_row_tiles = 0;
      }
      continue;
    }
    for (int64_t t = lane; t < tiles; t += 32) tile_group[start + t] = e - rank * local;
    for (int64_t r = start * tile + total + lane; r < (start + tiles) * tile; r += 32) meta[r] = -1;
    if (last && lane == 0) *num_row_tiles = static_cast<int32_t>(start + tiles);
  }
}

struct DispatchPeers {
  uint8_t* rows[kMaxPeers];
  uint8_t* aux[kMaxPeers];
  int32_t* meta[kMaxPeers];
  float* weight[kMaxPeers];
};

// One warp per token replica.
template <typename IdT>
__global__ void __launch_bounds__(256)
ep_dispatch_kernel(const IdT* __restrict__ ids, const float* __restrict__ weights, int64_t replicas,
                   int topk, int experts, int local, int rank, const uint8_t* __restrict__ src,
                   int64_t src_stride, int row_bytes, const uint8_t* __restrict__ aux,
                   int64_t aux_stride, int aux_bytes, const int64_t* __restrict__ first_row,
                   int32_t* __restrict__ cursor, int64_t capacity_rows, DispatchPeers peers) {
  const int lane = threadIdx.x & 31;
  const int64_t warps = static_cast<int64_t>(gridDim.x) * (blockDim.x >> 5);
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x >> 5) + (threadIdx.x >> 5); i < replicas;
       i += warps) {
    const long long e = static_cast<long long>(ids[i]);
    if (e < 0 || e >= experts) continue;          // dropped (ep_count has reported it)
    int64_t r = 0;
    if (lane == 0) r = first_row[e] + atomicAdd(&cursor[e], 1);
    r = __shfl_sync(0xffffffffu, r, 0);
    if (r >= capacity_rows) continue;             // the plan reported the overflow
    const int d = static_cast<int>(e) / local;
    const int64_t token = i / topk;
    const uint4* s = reinterpret_cast<const uint4*>(src + token * src_stride);
    uint4* dst = reinterpret_cast<uint4*>(peers.rows[d] + r * row_bytes);
    // eight 16-byte vectors per lane in flight (a 4 KB row in one round)
    const int nv = row_bytes / 16;
    for (int v0 = 0; v0 < nv; v0 += 256) {
      uint4 t[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int v = v0 + u * 32 + lane;
        if (v < nv) t[u] = s[v];
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int v = v0 + u * 32 + lane;
        if (v < nv) dst[v] = t[u];
      }
    }
    if (aux_bytes > 0) {
      const uint4* sa = reinterpret_cast<const uint4*>(aux + token * aux_stride);
      uint4* da = reinterpret_cast<uint4*>(peers.aux[d] + r * aux_bytes);
      for (int v = lane; v < aux_bytes / 16; v += 32) da[v] = sa[v];
    }
    if (lane == 0) {
      peers.meta[d][r] = static_cast<int32_t>(static_cast<int64_t>(rank) * replicas + i);
      peers.weight[d][r] = weights != nullptr ? weights[i] : 1.0f;
    }
  }
}

__device__ __forceinline__ void st_release_sys(int32_t* p, int32_t v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int32_t ld_acquire_sys(const int32_t* p) {
  int32_t v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Thread p tells rank p "this rank has reached barrier number `epoch`" and waits until rank p
// has said the same.  Epochs only grow, so flags are never reset; a wait that runs out of its
// budget is reported and the kernel returns (the data behind the barrier is then undefined).
__global__ void __launch_bounds__(32)
peer_barrier_kernel(PeerInts flags, int world, int rank, int32_t* __restrict__ epoch_counter,
                    uint64_t budget_ns, int* status) {
  const int32_t epoch = *epoch_counter + 1;
  const int p = threadIdx.x;
  if (p < world) {
    __threadfence_system();
    st_release_sys(flags.p[p] + rank, epoch);
    const int32_t* mine = flags.p[rank] + p;
    uint64_t t0 = 0;
    for (uint32_t it = 1;; ++it) {
      if (ld_acquire_sys(mine) - epoch >= 0) break;
      if ((it & 0x3f) == 0) {
        const uint64_t now = global_timer_ns();
        if (t0 == 0) t0 = now;
        else if (now - t0 > budget_ns) {
          report_status(status, 60, p);
          break;
        }
      }
      __nanosleep(100);
    }
  }
  __syncwarp();
  if (p == 0) *epoch_counter = epoch;
}

int fill_peers(PeerInts* out, const void* const* ptrs, int world, const char* what) {
  if (ptrs == nullptr) return fail(B200K_INVALID_ARG, "%s: null pointer table", what);
  for (int i = 0; i < world; ++i) {
    if (ptrs[i] == nullptr || reinterpret_cast<uintptr_t>(ptrs[i]) % 4)
      return fail(B200K_INVALID_ARG, "%s: pointer %d is null or not 4-byte aligned", what, i);
    out->p[i] = static_cast<int32_t*>(const_cast<void*>(ptrs[i]));
  }
  return B200K_OK;
}

int check_world(int world, int rank, int experts) {
  if (world <= 0 || world > kMaxPeers || rank < 0 || rank >= world)
    return fail(B200K_INVALID_ARG, "world must be in [1, %d] and rank inside it", kMaxPeers);
  if (experts <= 0 || experts > kMaxExperts || experts % world)
    return fail(B200K_INVALID_ARG, "experts must be in [1, %d] and a multiple of world", kMaxExperts);
  return B200K_OK;
}

int blocks_for(int64_t items, int per_block) {
  int sms = current_sm_count();
  if (sms <= 0) sms = 148;
  int64_t b = ceil_div(items, per_block);
  const int64_t cap = static_cast<int64_t>(sms) * 8;
  if (b < 1) b = 1;
  return static_cast<int>(b < cap ? b : cap);
}

}  // namespace
}  // namespace b200k

using namespace b200k;

extern "C" int64_t b200k_moe_ep_capacity_rows(int64_t replicas_per_rank, int32_t world,
                                              int32_t num_experts, int32_t tile_rows) {
  if (replicas_per_rank < 0 || world <= 0 || num_experts <= 0 || num_experts % world || tile_rows <= 0) return 0;
  return ep_capacity_rows(replicas_per_rank, world, num_experts / world, tile_rows);
}

extern "C" int b200k_moe_ep_count(const b200k_moe_ep_count_args* a, b200k_stream stream_) {
  if (a == nullptr) return fail(B200K_INVALID_ARG, "null args");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (int rc = check_world(a->world, a->rank, a->num_experts)) return rc;
  if (a->num_replicas < 0 || a->num_replicas >= INT32_MAX) return fail(B200K_INVALID_ARG, "bad replica count");
  if (!a->scratch || (a->num_replicas > 0 && !a->topk_ids)) return fail(B200K_INVALID_ARG, "null pointer");
  PeerInts peers = {};
  if (int rc = fill_peers(&peers, a->hist_peers, a->world, "hist_peers")) return rc;
  int32_t* hist_local = static_cast<int32_t*>(a->scratch);
  unsigned int* ticket = reinterpret_cast<unsigned int*>(hist_local + a->num_experts);
  const int grid = blocks_for(a->num_replicas, 256 * 8);
  const size_t smem = static_cast<size_t>(a->num_experts) * sizeof(int32_t);
  if (a->ids_are_int64)
    ep_count_kernel<long long><<<grid, 256, smem, stream>>>(static_cast<const long long*>(a->topk_ids),
                                                            a->num_replicas, a->num_experts, hist_local, ticket,
                                                            peers, a->world, a->rank, device_status_word());
  else
    ep_count_kernel<int><<<grid, 256, smem, stream>>>(static_cast<const int*>(a->topk_ids), a->num_replicas,
                                                      a->num_experts, hist_local, ticket, peers, a->world,
                                                      a->rank, device_status_word());
  B200K_CHECK_LAUNCH("moe_ep_count launch");
  return B200K_OK;
}

extern "C" int b200k_moe_ep_plan(const b200k_moe_ep_plan_args* a, b200k_stream stream_) {
  if (a == nullptr) return fail(B200K_INVALID_ARG, "null args");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (int rc = check_world(a->world, a->rank, a->num_experts)) return rc;
  if (a->tile_rows != 128 && a->tile_rows != 256) return fail(B200K_INVALID_ARG, "tile_rows must be 128 or 256");
  if (!a->hist || !a->first_row || !a->cursor || !a->tile_group || !a->num_row_tiles || !a->meta)
    return fail(B200K_INVALID_ARG, "null pointer");
  if (a->capacity_rows <= 0 || a->capacity_rows % a->tile_rows)
    return fail(B200K_INVALID_ARG, "capacity_rows must be a positive multiple of tile_rows");
  ep_plan_kernel<<<1, 1024, 0, stream>>>(a->hist, a->world, a->rank, a->num_experts, a->tile_rows,
                                         a->capacity_rows, a->first_row, a->cursor, a->tile_group,
                                         a->num_row_tiles, a->meta, device_status_word());
  B200K_CHECK_LAUNCH("moe_ep_plan launch");
  return B200K_OK;
}

extern "C" int b200k_moe_ep_dispatch(const b200k_moe_ep_dispatch_args* a, b200k_stream stream_) {
  if (a == nullptr) return fail(B200K_INVALID_ARG, "null args");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (int rc = check_world(a->world, a->rank, a->num_experts)) return rc;
  if (a->num_replicas < 0 || a->topk <= 0 || a->num_replicas % a->topk)
    return fail(B200K_INVALID_ARG, "num_replicas must be tokens * topk");
  if (a->num_replicas == 0) return B200K_OK;
  if (!a->topk_ids || !a->src || !a->first_row || !a->cursor || !a->row_peers || !a->meta_peers ||
      !a->weight_peers || (a->aux_bytes > 0 && (!a->aux || !a->aux_peers)))
    return fail(B200K_INVALID_ARG, "null pointer");
  if (a->row_bytes <= 0 || a->row_bytes % 16 || a->src_stride_bytes % 16 || a->aux_bytes % 16 ||
      a->aux_stride_bytes % 16 || reinterpret_cast<uintptr_t>(a->src) % 16 ||
      reinterpret_cast<uintptr_t>(a->aux) % 16)
    return fail(B200K_UNSUPPORTED, "rows must be multiples of 16 bytes on 16-byte boundaries");
  DispatchPeers peers = {};
  for (int i = 0; i < a->world; ++i) {
    if (!a->row_peers[i] || !a->meta_peers[i] || !a->weight_peers[i] || (a->aux_bytes > 0 && !a->aux_peers[i]) ||
        reinterpret_cast<uintptr_t>(a->row_peers[i]) % 16 ||
        (a->aux_bytes > 0 && reinterpret_cast<uintptr_t>(a->aux_peers[i]) % 16))
      return fail(B200K_INVALID_ARG, "peer buffer %d is null or not 16-byte aligned", i);
    peers.rows[i] = static_cast<uint8_t*>(a->row_peers[i]);
    peers.aux[i] = a->aux_bytes > 0 ? static_cast<uint8_t*>(a->aux_peers[i]) : nullptr;
    peers.meta[i] = static_cast<int32_t*>(a->meta_peers[i]);
    peers.weight[i] = static_cast<float*>(a->weight_peers[i]);
  }
  const int grid = blocks_for(a->num_replicas, 8);
  const int local = a->num_experts / a->world;
#define B200K_EP_DISPATCH(T)                                                                            \
  ep_dispatch_kernel<T><<<grid, 256, 0, stream>>>(                                                      \
      static_cast<const T*>(a->topk_ids), a->weights, a->num_replicas, a->topk, a->num_experts, local,  \
      a->rank, static_cast<const uint8_t*>(a->src), a->src_stride_bytes, static_cast<int>(a->row_bytes), \
      static_cast<const uint8_t*>(a->aux), a->aux_stride_bytes, static_cast<int>(a->aux_bytes),         \
      a->first_row, a->cursor, a->capacity_rows, peers)
  if (a->ids_are_int64) B200K_EP_DISPATCH(long long);
  else B200K_EP_DISPATCH(int);
#undef B200K_EP_DISPATCH
  B200K_CHECK_LAUNCH("moe_ep_dispatch launch");
  return B200K_OK;
}

extern "C" int b200k_peer_barrier(const void* const* flag_peers, int32_t world, int32_t rank,
                                  int32_t* epoch_counter, int32_t budget_us, b200k_stream stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (world <= 0 || world > kMaxPeers || rank < 0 || rank >= world)
    return fail(B200K_INVALID_ARG, "world must be in [1, %d] and rank inside it", kMaxPeers);
  if (!epoch_counter) return fail(B200K_INVALID_ARG, "null epoch counter");
  PeerInts flags = {};
  if (int rc = fill_peers(&flags, flag_peers, world, "flag_peers")) return rc;
  const uint64_t budget_ns = budget_us > 0 ? static_cast<uint64_t>(budget_us) * 1000ull : kWaitBudgetNs;
  peer_barrier_kernel<<<1, 32, 0, stream>>>(flags, world, rank, epoch_counter, budget_ns, device_status_word());
  B200K_CHECK_LAUNCH("peer_barrier launch");
  return B200K_OK;
}
