// Peer-memory gather for the AllGather GEMM: every rank pulls the other ranks' row shards
// of A out of their (peer-mapped) buffers into one local buffer, with plain 16-byte loads
// over NVLink, all peers at once.  The GEMM then reads A from local HBM, so a remote tile
// crosses NVLink once instead of once per column tile of the output.
//
// Replaces the in-kernel remote tile loads of gather_matmul_kernel (reference:
// samples/AllGatherMatmul.py:28-81), whose semantics it keeps: out rows
// [p * rows, (p + 1) * rows) come from rank p's shard.  The caller orders this against the
// peers' writes exactly as the sample does (a barrier before, a barrier after).
#include "common.cuh"
#include "host.h"
#include "peer_gather_index.h"

namespace b200k {
namespace {

constexpr int kMaxPeers = 16;

struct PeerPtrs {
  const uint8_t* p[kMaxPeers];
};

// fp32 -> tf32 with round-to-nearest (ties away), kept in an fp32 container: what the
// reference's astype(tf32) does before its MMA.
__device__ __forceinline__ uint32_t round_tf32(uint32_t bits) {
  uint32_t out;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(out) : "f"(__uint_as_float(bits)));
  return out;
}

__global__ void __launch_bounds__(256)
peer_gather_kernel(PeerPtrs peers, int world, int rank, int64_t rows, int64_t row_vecs,
                   int64_t src_stride, uint8_t* __restrict__ dst, int64_t dst_stride,
                   int round_to_tf32) {
  const int64_t items = peer_gather_items(world, rows, row_vecs);
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < items;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const PeerGatherItem it = peer_gather_item(i, world, rank, rows, row_vecs);
    if (!it.valid) continue;
    const int peer = it.peer;
    const int64_t r = it.row, c = it.col;
    uint4 q = *reinterpret_cast<const uint4*>(peers.p[peer] + r * src_stride + c * 16);
    if (round_to_tf32) {
      q.x = round_tf32(q.x);
      q.y = round_tf32(q.y);
      q.z = round_tf32(q.z);
      q.w = round_tf32(q.w);
    }
    *reinterpret_cast<uint4*>(dst + (static_cast<int64_t>(peer) * rows + r) * dst_stride + c * 16) = q;
  }
}

// out[p * rows + i] = the fp32 scalar rank p holds, for every rank: per-row scales of a
// gathered operand whose shards carry one tensor scale each.
__global__ void __launch_bounds__(256)
peer_scalar_expand_kernel(PeerPtrs peers, int64_t rows, float* __restrict__ out) {
  const float v = *reinterpret_cast<const float*>(peers.p[blockIdx.y]);
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < rows;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x)
    out[static_cast<int64_t>(blockIdx.y) * rows + i] = v;
}

}  // namespace
}  // namespace b200k

using namespace b200k;

extern "C" int b200k_peer_gather(const b200k_peer_gather_args* a, b200k_stream stream_) {
  if (a == nullptr) return fail(B200K_INVALID_ARG, "null args");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (a->world <= 0 || a->world > kMaxPeers || a->rank < 0 || a->rank >= a->world)
    return fail(B200K_INVALID_ARG, "world must be in [1, %d] and rank inside it", kMaxPeers);
  if (a->rows < 0 || a->row_bytes < 0) return fail(B200K_INVALID_ARG, "negative size");
  if (a->rows == 0 || a->row_bytes == 0) return B200K_OK;
  if (!a->shards || !a->dst) return fail(B200K_INVALID_ARG, "null pointer");
  if (a->row_bytes % 16 || a->src_stride_bytes % 16 || a->dst_stride_bytes % 16 ||
      reinterpret_cast<uintptr_t>(a->dst) % 16)
    return fail(B200K_UNSUPPORTED, "rows must be multiples of 16 bytes on 16-byte boundaries");
  PeerPtrs peers = {};
  for (int i = 0; i < a->world; ++i) {
    if (a->shards[i] == nullptr || reinterpret_cast<uintptr_t>(a->shards[i]) % 16)
      return fail(B200K_INVALID_ARG, "shard %d pointer is null or not 16-byte aligned", i);
    peers.p[i] = static_cast<const uint8_t*>(a->shards[i]);
  }
  int sms = current_sm_count();
  if (sms <= 0) return fail(B200K_CUDA_ERROR, "no current CUDA device");
  const int64_t vecs = a->rows * (a->row_bytes / 16) * a->world;
  int64_t blocks = ceil_div(vecs, 256);
  if (blocks > static_cast<int64_t>(sms) * 8) blocks = static_cast<int64_t>(sms) * 8;
  peer_gather_kernel<<<static_cast<int>(blocks), 256, 0, stream>>>(
      peers, a->world, a->rank, a->rows, a->row_bytes / 16, a->src_stride_bytes,
      static_cast<uint8_t*>(a->dst), a->dst_stride_bytes, a->round_tf32);
  B200K_CHECK_LAUNCH("peer_gather launch");
  return B200K_OK;
}

extern "C" int b200k_peer_scalar_expand(const void* const* shards, int32_t world, int64_t rows,
                                        float* out, b200k_stream stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (world <= 0 || world > kMaxPeers) return fail(B200K_INVALID_ARG, "world must be in [1, %d]", kMaxPeers);
  if (rows < 0) return fail(B200K_INVALID_ARG, "negative size");
  if (rows == 0) return B200K_OK;
  if (!shards || !out) return fail(B200K_INVALID_ARG, "null pointer");
  PeerPtrs peers = {};
  for (int i = 0; i < world; ++i) {
    if (shards[i] == nullptr || reinterpret_cast<uintptr_t>(shards[i]) % 4)
      return fail(B200K_INVALID_ARG, "shard %d pointer is null or not 4-byte aligned", i);
    peers.p[i] = static_cast<const uint8_t*>(shards[i]);
  }
  const dim3 grid(static_cast<unsigned>(rows / 256 + 1 < 64 ? rows / 256 + 1 : 64), static_cast<unsigned>(world));
  peer_scalar_expand_kernel<<<grid, 256, 0, stream>>>(peers, rows, out);
  B200K_CHECK_LAUNCH("peer_scalar_expand launch");
  return B200K_OK;
}
