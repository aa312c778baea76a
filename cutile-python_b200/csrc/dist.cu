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

// A block of 256 threads takes whole 4 KB runs (thread = vector inside the run), four runs
// at a time so that every thread has four 16-byte loads in flight: two blocks per SM put
// 4.8 MB on the wire, enough for NVLink's latency, from a kernel whose index arithmetic is a
// handful of instructions per vector - it runs beside the GEMM of the rank's own rows and
// must leave it the issue slots.
constexpr int kGatherInFlight = 4;
static_assert(kPeerGatherChunkVecs == 256, "one thread per vector of a run");

__global__ void __launch_bounds__(256)
peer_gather_kernel(PeerPtrs peers, int world, int rank, int64_t rows, int64_t row_vecs,
                   int64_t src_stride, uint8_t* __restrict__ dst, int64_t dst_stride,
                   int round_to_tf32) {
  const int64_t runs = peer_gather_runs(world, rows, row_vecs);
  const int64_t shard_vecs = rows * row_vecs;
  const bool dense = src_stride == row_vecs * 16 && dst_stride == row_vecs * 16;   // rows back to back
  const bool small = shard_vecs < (1ll << 31);
  for (int64_t run0 = blockIdx.x; run0 < runs; run0 += static_cast<int64_t>(gridDim.x) * kGatherInFlight) {
    uint4 q[kGatherInFlight];
    uint8_t* out[kGatherInFlight];
#pragma unroll
    for (int u = 0; u < kGatherInFlight; ++u) {
      const int64_t run = run0 + static_cast<int64_t>(u) * gridDim.x;
      out[u] = nullptr;
      if (run >= runs) continue;
      const PeerGatherRun r = peer_gather_run(run, world, rank);
      const int64_t v = r.first_vec + threadIdx.x;
      if (v >= shard_vecs) continue;
      int64_t src_off, dst_off;
      if (dense) {
        src_off = dst_off = v * 16;
      } else {
        int64_t row, col;
        if (small) {
          row = static_cast<uint32_t>(v) / static_cast<uint32_t>(row_vecs);
          col = static_cast<uint32_t>(v) - static_cast<uint32_t>(row) * static_cast<uint32_t>(row_vecs);
        } else {
          row = v / row_vecs;
          col = v - row * row_vecs;
        }
        src_off = row * src_stride + col * 16;
        dst_off = row * dst_stride + col * 16;
      }
      q[u] = *reinterpret_cast<const uint4*>(peers.p[r.peer] + src_off);
      out[u] = dst + static_cast<int64_t>(r.peer) * rows * dst_stride + dst_off;
    }
#pragma unroll
    for (int u = 0; u < kGatherInFlight; ++u) {
      if (out[u] == nullptr) continue;
      if (round_to_tf32) {
        q[u].x = round_tf32(q[u].x);
        q[u].y = round_tf32(q[u].y);
        q[u].z = round_tf32(q[u].z);
        q[u].w = round_tf32(q[u].w);
      }
      *reinterpret_cast<uint4*>(out[u]) = q[u];
    }
  }
}

// The same gather through the copy engine of the SM (untiled bulk copies, no multicast): one
// warp per block, one lane issuing.  A 4 KB run is pulled into a ring slot in shared memory
// and pushed to the gathered tensor from there, three runs in flight per block.  The point is
// what the kernel does NOT take: 32 threads, a few registers and 16 KB of shared memory fit
// on an SM beside a CTA of the GEMM (224 threads x 242 registers, 197 KB), where a block of
// the load / store kernel above does not and waits for the GEMM of the rank's own rows to
// leave.  Dense shards only (rows back to back), no tf32 rounding.
constexpr int kBulkStages = 4;
constexpr int kBulkRunBytes = kPeerGatherChunkVecs * 16;

constexpr int kMaxBatch = kPeerGatherMaxBatch;

struct BulkJob {
  PeerPtrs peers;
  int64_t shard_bytes;
  uint8_t* dst;
  int first_block;      // blocks [first_block, next job's first_block) work on this job
};

struct BulkBatch {
  BulkJob job[kMaxBatch];
  int jobs;
  int world, rank;
  // optional: out[p * rows + i] = the fp32 scalar of rank p (lanes 1..31 of every block)
  PeerPtrs scalars;
  int64_t scalar_rows;
  float* scalar_out;
};

__global__ void __launch_bounds__(32)
peer_gather_bulk_kernel(const __grid_constant__ BulkBatch b, int* status) {
  __shared__ __align__(128) uint8_t ring[kBulkStages][kBulkRunBytes];
  __shared__ __align__(8) uint64_t full[kBulkStages];
  __shared__ int abort_flag, never;
  if (threadIdx.x != 0) {
    if (b.scalar_out != nullptr) {
      const int64_t n = b.scalar_rows * b.world;
      for (int64_t i = blockIdx.x * 31ll + (threadIdx.x - 1); i < n; i += gridDim.x * 31ll)
        b.scalar_out[i] = *reinterpret_cast<const float*>(b.scalars.p[i / b.scalar_rows]);
    }
    return;
  }
  int j = 0;
  while (j + 1 < b.jobs && static_cast<int>(blockIdx.x) >= b.job[j + 1].first_block) ++j;
  const BulkJob& job = b.job[j];
  const int block = blockIdx.x - job.first_block;
  const int blocks = (j + 1 < b.jobs ? b.job[j + 1].first_block : static_cast<int>(gridDim.x)) - job.first_block;
  const int64_t shard_bytes = job.shard_bytes;
  // every run holds at least one vector (peer_gather_items rounds the shard up to whole runs)
  const int64_t runs = peer_gather_runs(b.world, shard_bytes / 16, 1);
  for (int s = 0; s < kBulkStages; ++s) mbar_init(smem_u32(&full[s]), 1);
  abort_flag = 0;
  never = 0;
  fence_barrier_init();
  const int64_t mine = block < runs ? (runs - block + blocks - 1) / blocks : 0;
  struct Run { const uint8_t* src; uint8_t* out; uint32_t bytes; };
  auto run_of = [&](int64_t k) {   // k-th run of this block
    const PeerGatherRun r = peer_gather_run(block + k * blocks, b.world, b.rank);
    const int64_t off = r.first_vec * 16;
    const int64_t left = shard_bytes - off;
    Run x;
    x.src = job.peers.p[r.peer] + off;
    x.out = job.dst + static_cast<int64_t>(r.peer) * shard_bytes + off;
    x.bytes = static_cast<uint32_t>(left < kBulkRunBytes ? left : kBulkRunBytes);
    return x;
  };
  auto load = [&](int64_t k) {     // into slot k % stages
    const Run x = run_of(k);
    const uint32_t bar = smem_u32(&full[k % kBulkStages]);
    mbar_arrive_expect_tx(bar, x.bytes);
    bulk_load(smem_u32(ring[k % kBulkStages]), x.src, x.bytes, bar);
  };
  int64_t loaded = 0;
  for (; loaded < kBulkStages - 1 && loaded < mine; ++loaded) load(loaded);
  for (int64_t k = 0; k < mine; ++k) {
    if (!mbar_wait_lane(smem_u32(&full[k % kBulkStages]), (k / kBulkStages) & 1, &abort_flag)) {
      // a load that did not land in the budget: report, give the other loads in flight a last
      // (short) chance to land in this block's ring before the block gives the ring up
      report_status(status, 90, static_cast<int>(k & 0xffff));
      for (int64_t i = k + 1; i < loaded; ++i)
        mbar_wait_lane(smem_u32(&full[i % kBulkStages]), (i / kBulkStages) & 1, &never, 100ull * 1000 * 1000);
      break;
    }
    fence_proxy_async_smem();
    const Run x = run_of(k);
    bulk_store(x.out, smem_u32(ring[k % kBulkStages]), x.bytes);
    tma_store_commit();
    // the slot of run k + stages - 1 is the one store k - 1 read: all but the newest group
    // must be done with shared memory
    tma_store_wait_read<1>();
    if (loaded < mine) load(loaded++);
  }
  tma_store_wait<0>();
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

namespace {

// what the bulk-copy kernel takes: rows back to back on both sides, payload copied as it is
bool dense_plain(const b200k_peer_gather_args* a) {
  return !a->round_tf32 && a->src_stride_bytes == a->row_bytes && a->dst_stride_bytes == a->row_bytes;
}

bool bulk_form_applies(const b200k_peer_gather_args* a) {
  const char* form = getenv("B200K_GATHER");      // B200K_GATHER=ldst keeps the load / store kernel
  return dense_plain(a) && !(form != nullptr && form[0] == 'l');
}

int check_gather_args(const b200k_peer_gather_args* a) {
  if (a->world <= 0 || a->world > kMaxPeers || a->rank < 0 || a->rank >= a->world)
    return fail(B200K_INVALID_ARG, "world must be in [1, %d] and rank inside it", kMaxPeers);
  if (a->rows < 0 || a->row_bytes < 0) return fail(B200K_INVALID_ARG, "negative size");
  if (a->rows == 0 || a->row_bytes == 0) return B200K_OK;
  if (!a->shards || !a->dst) return fail(B200K_INVALID_ARG, "null pointer");
  if (a->row_bytes % 16 || a->src_stride_bytes % 16 || a->dst_stride_bytes % 16 ||
      reinterpret_cast<uintptr_t>(a->dst) % 16)
    return fail(B200K_UNSUPPORTED, "rows must be multiples of 16 bytes on 16-byte boundaries");
  for (int i = 0; i < a->world; ++i)
    if (a->shards[i] == nullptr || reinterpret_cast<uintptr_t>(a->shards[i]) % 16)
      return fail(B200K_INVALID_ARG, "shard %d pointer is null or not 16-byte aligned", i);
  return B200K_OK;
}

// One launch of the bulk-copy kernel over `count` dense gathers (blocks dealt in proportion
// to the runs of each) and, optionally, the scalar expansion.
int launch_bulk_batch(const b200k_peer_gather_args* args, int count, const void* const* scalar_shards,
                      int64_t scalar_rows, float* scalar_out, cudaStream_t stream) {
  int sms = current_sm_count();
  if (sms <= 0) return fail(B200K_CUDA_ERROR, "no current CUDA device");
  BulkBatch b = {};
  int64_t runs[kMaxBatch] = {};
  for (int j = 0; j < count; ++j) {
    const b200k_peer_gather_args* a = &args[j];
    if (a->rows == 0 || a->row_bytes == 0) continue;
    BulkJob& job = b.job[b.jobs];
    for (int i = 0; i < a->world; ++i) job.peers.p[i] = static_cast<const uint8_t*>(a->shards[i]);
    job.shard_bytes = a->rows * a->row_bytes;
    job.dst = static_cast<uint8_t*>(a->dst);
    runs[b.jobs] = peer_gather_runs(a->world, job.shard_bytes / 16, 1);
    b.world = a->world;
    b.rank = a->rank;
    ++b.jobs;
  }
  if (b.jobs == 0 && scalar_out == nullptr) return B200K_OK;
  int grid = 1;
  if (b.jobs > 0) {
    int first[kMaxBatch];
    grid = peer_gather_batch_blocks(runs, b.jobs, sms, first);
    for (int j = 0; j < b.jobs; ++j) b.job[j].first_block = first[j];
  }
  if (scalar_out != nullptr) {
    b.world = args[0].world;
    b.rank = args[0].rank;
    for (int i = 0; i < b.world; ++i) b.scalars.p[i] = static_cast<const uint8_t*>(scalar_shards[i]);
    b.scalar_rows = scalar_rows;
    b.scalar_out = scalar_out;
  }
  peer_gather_bulk_kernel<<<grid, 32, 0, stream>>>(b, device_status_word());
  B200K_CHECK_LAUNCH("peer_gather (bulk) launch");
  return B200K_OK;
}

}  // namespace

extern "C" int b200k_peer_gather(const b200k_peer_gather_args* a, b200k_stream stream_) {
  if (a == nullptr) return fail(B200K_INVALID_ARG, "null args");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (int rc = check_gather_args(a)) return rc;
  if (a->rows == 0 || a->row_bytes == 0) return B200K_OK;
  // dense shards without rounding go through the bulk-copy form
  if (bulk_form_applies(a)) return launch_bulk_batch(a, 1, nullptr, 0, nullptr, stream);
  PeerPtrs peers = {};
  for (int i = 0; i < a->world; ++i) peers.p[i] = static_cast<const uint8_t*>(a->shards[i]);
  int sms = current_sm_count();
  if (sms <= 0) return fail(B200K_CUDA_ERROR, "no current CUDA device");
  const int64_t vecs = a->rows * (a->row_bytes / 16) * a->world;
  int64_t blocks = ceil_div(vecs, 256 * kGatherInFlight);
  if (blocks > 2 * sms) blocks = 2 * sms;
  peer_gather_kernel<<<static_cast<int>(blocks), 256, 0, stream>>>(
      peers, a->world, a->rank, a->rows, a->row_bytes / 16, a->src_stride_bytes,
      static_cast<uint8_t*>(a->dst), a->dst_stride_bytes, a->round_tf32);
  B200K_CHECK_LAUNCH("peer_gather launch");
  return B200K_OK;
}

extern "C" int b200k_peer_gather_batch(const b200k_peer_gather_args* args, int32_t count,
                                       const void* const* scalar_shards, int64_t scalar_rows,
                                       float* scalar_out, b200k_stream stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (args == nullptr || count < 1 || count > kMaxBatch)
    return fail(B200K_INVALID_ARG, "1 to %d gathers per batch", kMaxBatch);
  for (int j = 0; j < count; ++j) {
    if (int rc = check_gather_args(&args[j])) return rc;
    if (args[j].world != args[0].world || args[j].rank != args[0].rank)
      return fail(B200K_INVALID_ARG, "every gather of a batch must have the same world and rank");
    if (!dense_plain(&args[j]))
      return fail(B200K_UNSUPPORTED, "a batch takes dense gathers without rounding only (both strides == row_bytes)");
  }
  if (scalar_shards != nullptr || scalar_out != nullptr) {
    if (scalar_shards == nullptr || scalar_out == nullptr || scalar_rows < 0)
      return fail(B200K_INVALID_ARG, "scalar expansion needs shards, rows >= 0 and an output");
    for (int i = 0; i < args[0].world; ++i)
      if (scalar_shards[i] == nullptr || reinterpret_cast<uintptr_t>(scalar_shards[i]) % 4)
        return fail(B200K_INVALID_ARG, "scalar shard %d is null or misaligned", i);
    if (scalar_rows == 0) scalar_out = nullptr;
  }
  return launch_bulk_batch(args, count, scalar_shards, scalar_rows, scalar_out, stream);
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
