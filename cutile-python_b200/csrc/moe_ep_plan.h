// Placement arithmetic of the expert-parallel MoE dispatch, shared by the planning kernel and
// by a host-side test harness (plain C++: no CUDA types).
//
// Every rank owns `local` = experts / world consecutive experts and a receive buffer whose
// rows are laid out for the grouped GEMM: expert after expert, each expert's run padded to
// whole row tiles.  Inside an expert's run the rows of source rank 0 come first, then rank
// 1's, and so on.  All of that follows from one table every rank holds after the first
// exchange: hist[s * experts + e] = how many token replicas rank s routes to (global) expert
// e.  From it every rank computes, without talking to anyone,
//
//   total(e)        rows expert e receives                      = sum over s of hist[s][e]
//   before(s, e)    rows of ranks < s inside expert e's run      = sum over s' < s of hist[s'][e]
//   tiles(e)        row tiles of expert e                        = ceil(total(e) / tile)
//   tile_start(e)   first row tile of e in its owner's buffer    = sum of tiles(e') over the
//                                                                  owner's experts e' < e
//   first_row(s, e) where rank s writes its first row for e      = tile_start(e) * tile + before(s, e)
//
// A source then numbers its own rows for e with a counter (the order inside a run does not
// matter: rows are independent, and every row carries the id of the replica it came from).
#ifndef B200K_MOE_EP_PLAN_H_
#define B200K_MOE_EP_PLAN_H_

#include <stdint.h>

#ifndef B200K_HD
#ifdef __CUDACC__
#define B200K_HD __host__ __device__ __forceinline__
#else
#define B200K_HD inline
#endif
#endif

namespace b200k {

B200K_HD int ep_owner(int expert, int local) { return expert / local; }

B200K_HD int64_t ep_total(const int32_t* hist, int world, int experts, int e) {
  int64_t t = 0;
  for (int s = 0; s < world; ++s) t += hist[static_cast<int64_t>(s) * experts + e];
  return t;
}

B200K_HD int64_t ep_before(const int32_t* hist, int experts, int rank, int e) {
  int64_t t = 0;
  for (int s = 0; s < rank; ++s) t += hist[static_cast<int64_t>(s) * experts + e];
  return t;
}

B200K_HD int64_t ep_tiles(int64_t total, int tile) { return (total + tile - 1) / tile; }

// First row tile of expert e inside its owner's buffer.
B200K_HD int64_t ep_tile_start(const int32_t* hist, int world, int experts, int local, int tile, int e) {
  const int first = ep_owner(e, local) * local;
  int64_t t = 0;
  for (int q = first; q < e; ++q) t += ep_tiles(ep_total(hist, world, experts, q), tile);
  return t;
}

B200K_HD int64_t ep_first_row(const int32_t* hist, int world, int experts, int local, int tile, int rank,
                              int e) {
  return ep_tile_start(hist, world, experts, local, tile, e) * tile + ep_before(hist, experts, rank, e);
}

// Rows a receive buffer must hold in the worst case (every replica of every rank routed to
// this rank's experts, every expert wasting tile - 1 rows), rounded up to whole tiles.
B200K_HD int64_t ep_capacity_rows(int64_t replicas_per_rank, int world, int local, int tile) {
  const int64_t need = replicas_per_rank * world + static_cast<int64_t>(local) * (tile - 1);
  return (need + tile - 1) / tile * tile;
}

}  // namespace b200k
#endif  // B200K_MOE_EP_PLAN_H_
