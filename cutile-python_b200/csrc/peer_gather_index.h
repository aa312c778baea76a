// Work decomposition of the peer gather, shared by the kernel and by a host-side test
// harness (this header is plain C++: no CUDA types).
//
// Every shard is rows x row_vecs 16-byte vectors.  The flat vector index v of a shard is cut
// into chunks of kPeerGatherChunkVecs vectors (4 KB); work item i addresses one vector:
//
//   within = i % chunk            position inside a 4 KB run
//   run    = i / chunk            runs are dealt round-robin over the peers ...
//   slot   = run % world          ... so consecutive runs hit different NVLink peers
//   chunk# = run / world
//   peer   = (rank + 1 + slot) % world    remote shards first, this rank's own shard last
//
// The kernel gives a run to a block of kPeerGatherChunkVecs threads (item = run, thread), so the
// divisions by `world` are per block and only the row / column split is per thread.
// Items whose vector index falls behind the end of the shard (the last chunk's tail) are
// invalid.  Every (peer, vector) pair is produced by exactly one valid item.
#ifndef B200K_PEER_GATHER_INDEX_H_
#define B200K_PEER_GATHER_INDEX_H_

#include <stdint.h>

#ifndef B200K_HD
#ifdef __CUDACC__
#define B200K_HD __host__ __device__ __forceinline__
#else
#define B200K_HD inline
#endif
#endif

namespace b200k {

constexpr int kPeerGatherChunkVecs = 256;   // 4 KB runs per peer keep every link busy at once

struct PeerGatherItem {
  int peer;       // shard the vector comes from; also its slot in the gathered tensor
  int64_t row;    // row inside the shard
  int64_t col;    // 16-byte vector inside the row
  bool valid;
};

B200K_HD int64_t peer_gather_items(int world, int64_t rows, int64_t row_vecs) {
  const int64_t shard_vecs = rows * row_vecs;
  const int64_t chunks = (shard_vecs + kPeerGatherChunkVecs - 1) / kPeerGatherChunkVecs;
  return chunks * world * kPeerGatherChunkVecs;
}

// A run of kPeerGatherChunkVecs consecutive items: one peer, consecutive vectors of its shard.
struct PeerGatherRun {
  int peer;
  int64_t first_vec;   // flat vector index inside the shard of the run's first item
};

B200K_HD int64_t peer_gather_runs(int world, int64_t rows, int64_t row_vecs) {
  return peer_gather_items(world, rows, row_vecs) / kPeerGatherChunkVecs;
}

B200K_HD PeerGatherRun peer_gather_run(int64_t run, int world, int rank) {
  PeerGatherRun r;
  const int slot = static_cast<int>(run % world);
  r.peer = (rank + 1 + slot) % world;
  r.first_vec = (run / world) * kPeerGatherChunkVecs;
  return r;
}

B200K_HD PeerGatherItem peer_gather_item(int64_t i, int world, int rank, int64_t rows, int64_t row_vecs) {
  PeerGatherItem it;
  const PeerGatherRun r = peer_gather_run(i / kPeerGatherChunkVecs, world, rank);
  const int64_t v = r.first_vec + i % kPeerGatherChunkVecs;
  it.valid = v < rows * row_vecs;
  it.peer = r.peer;
  it.row = v / row_vecs;
  it.col = v - it.row * row_vecs;
  return it;
}

// A batch launch (several gathers in one grid of one-warp blocks): the blocks are dealt over the
// jobs in proportion to their runs - one block per SM in all and never more, so that the whole
// grid is resident at once beside another kernel's CTAs, at least one block per job.  Block b
// of a job that owns `blocks` blocks takes the job's runs b, b + blocks, b + 2 * blocks, ...
// Returns the grid size; first_block[j] is job j's first block.
constexpr int kPeerGatherMaxBatch = 4;

B200K_HD int peer_gather_batch_blocks(const int64_t* runs, int jobs, int sms, int* first_block) {
  int64_t total = 0;
  for (int j = 0; j < jobs; ++j) total += runs[j];
  int64_t want = total < sms ? total : sms;
  if (want < jobs) want = jobs;
  int64_t left_blocks = want, left_runs = total;
  int grid = 0;
  for (int j = 0; j < jobs; ++j) {
    first_block[j] = grid;
    const int jobs_after = jobs - 1 - j;
    int64_t share = left_runs > 0 ? (runs[j] * left_blocks + left_runs / 2) / left_runs : 1;
    if (share < 1) share = 1;
    if (share > left_blocks - jobs_after) share = left_blocks - jobs_after;
    grid += static_cast<int>(share);
    left_blocks -= share;
    left_runs -= runs[j];
  }
  return grid;
}

}  // namespace b200k
#endif  // B200K_PEER_GATHER_INDEX_H_
