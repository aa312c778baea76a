// GEMM on CTA pairs (tcgen05 cta_group::2): two CTAs of a cluster share one 256 x 256
// output tile.  Each CTA loads its 128 rows of A and its 128 of the 256 rows of B per
// stage (32 KB instead of 48 KB, and 4.3 GB instead of 6.4 GB out of L2 for an 8192^3
// problem), the pair's leader issues 256 x 256 MMAs that read both halves, and each CTA
// drains its own 128 accumulator rows from its own tensor memory.
//
// No load in this file is a multicast: every CTA fetches its own tiles (scale-factor
// atoms of B are simply fetched by both) and reports the bytes to the leader's mbarrier.
//
//   warp 0      TMA producer, one lane, in both CTAs
//   warp 1      MMA issuer of the even k-steps, one lane, leader CTA only (allocates TMEM)
//   warps 2..5  epilogue, both CTAs
//   warp 6      MMA issuer of the odd k-steps, one lane, leader CTA only
//
// Two issuers because one thread cannot feed the tensor pipe of a block-scaled kind: a
// tcgen05 instruction costs its issuing thread 25 to 30 cycles, and an NVFP4 k-step is
// twelve scale-factor copies (tcgen05.cp), four MMAs of 132 cycles and two commits, 430
// cycles of issue against 529 of MMA time before any barrier wait.  The k-steps of a tile
// alternate between the issuers, each with its own scale-factor slot in tensor memory, so
// copies and MMAs of one k-step stay in one thread's program order.  Only the first k-step
// of a tile (the one that overwrites the accumulator) has to be complete before the other
// issuer may add to it; after that the order of the additions does not matter.
//
// Two accumulator windows let a tile's epilogue overlap the next tile's mainloop.  The
// block-scaled kinds also need TMEM columns for the two scale-factor slots, so their
// windows overlap by 32 (MXFP8) or 96 (NVFP4) columns: the epilogue drains the shared
// columns first and releases them early; the next tile's first MMA waits only for that.
#include <stdlib.h>

#include "gemm_common.cuh"
#include "gemm_pair.h"
#include "mx_quant.cuh"

namespace b200k {


template <int KIND>
struct PairCfg {
  using T = KindTraits<KIND>;
  static constexpr bool kScaled = T::kScaled;
  static constexpr int kBKElems = 128 * 8 / T::kElemBits;
  static constexpr int kStages = (KIND == kKindNVF4) ? 5 : 6;
  static constexpr int kABytes = 128 * 128;
  static constexpr int kBBytes = 128 * 128;          // this CTA's half of the 256 B rows
  static constexpr int kStageBytes = kABytes + kBBytes;
  // N-contiguous ("MN-major") B: boxes of 128 bytes of N by kBKElems rows of K
  static constexpr int kBBoxN = 128 * 8 / T::kElemBits;
  static constexpr int kBBoxBytes = kBKElems * 128;
  static constexpr int kMmaK = kBKElems / 4;
  static constexpr int kSfAtoms = kScaled ? (KIND == kKindNVF4 ? 4 : 1) : 0;  // along K, per stage
  static constexpr int kSfBytes = kSfAtoms * 512 * 3;                       // SFA + both SFB row tiles
  static constexpr int kAccStride = !kScaled ? 256 : (KIND == kKindNVF4 ? 160 : 224);
  static constexpr int kOverlapChunks = (256 - kAccStride) / 32;
  static constexpr int kSfBase = 2 * kAccStride + 32 * kOverlapChunks;     // 480 / 416
  static constexpr int kSfSlots = 2;
  static constexpr int kSfaCols = kSfAtoms * 4;
  static constexpr int kSfSlotCols = kSfAtoms * 12;
  static constexpr int kThreads = 224;
  static constexpr int kStagingBytes = 4 * 4096;   // epilogue: 32 rows x 128 bytes per warp
  static constexpr int kSmemBytes = 1024 + kStages * (kStageBytes + kSfBytes) + 256 + kStagingBytes;
  static_assert(!kScaled || kSfBase + kSfSlots * kSfSlotCols <= 512, "TMEM budget");
  static_assert(kSmemBytes <= 232448, "shared memory budget");
};

template <int KIND, int OUT>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(PairCfg<KIND>::kThreads, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                 const __grid_constant__ CUtensorMap tmap_sfa,
                 const __grid_constant__ CUtensorMap tmap_sfb, const GemmParams p) {
  using Cfg = PairCfg<KIND>;
  constexpr int S = Cfg::kStages;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t tiles_base = smem_base;
  const uint32_t sf_base = tiles_base + S * Cfg::kStageBytes;
  uint8_t* tail = smem + S * (Cfg::kStageBytes + Cfg::kSfBytes);
  const uint32_t staging_base = smem_u32(tail) + 256;   // behind the barriers
  const uint32_t bar_base = smem_u32(tail);
  // full[S], empty[S], acc_full[2], acc_empty[2], ovl_free, tile_open[2]
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (S + s); };
  auto acc_full_bar = [&](int a) { return bar_base + 8u * (2 * S + a); };
  auto acc_empty_bar = [&](int a) { return bar_base + 8u * (2 * S + 2 + a); };
  const uint32_t ovl_free_bar = bar_base + 8u * (2 * S + 4);
  auto tile_open_bar = [&](int a) { return bar_base + 8u * (2 * S + 5 + a); };   // leader's
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tail + 8 * (2 * S + 7));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tail + 8 * (2 * S + 7) + 8);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  // Where the caller asks for a programmatic launch (b200k_gemm_config): the kernel behind
  // this one in the stream may be set up while this one runs, and this one's own set-up
  // (barriers, tensor memory) overlaps the tail of the kernel before it.  Nothing below
  // touches global memory before pdl_wait() has seen that kernel complete.  Both calls are
  // no-ops under an ordinary launch.
  pdl_launch_dependents();

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(acc_full_bar(a), p.k_iters > 1 ? 2 : 1);   // one commit per issuer with work
      mbar_init(acc_empty_bar(a), 8);   // 4 epilogue warps in each CTA of the pair
      mbar_init(tile_open_bar(a), 1);
    }
    mbar_init(ovl_free_bar, 8);
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
  }
  if (warp == 1) {
    tmem_alloc_pair(smem_u32(tmem_slot), kTmemCols);
    tmem_relinquish_pair();
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  pdl_wait();

  // grouped mode: 256-row tiles, the live count comes from the device
  int tiles_m = (p.m + 255) / 256;
  if (p.num_row_tiles != nullptr) tiles_m = min(tiles_m, *p.num_row_tiles);
  // rows left out of the product (the AllGather GEMM's own shard, multiplied earlier from
  // the rank's own buffer): the raster runs over the remaining tile rows
  tiles_m -= p.skip_tiles;
  auto coord_of = [&](int tile) {
    TileCoord c = tile_coord(tile, tiles_m, p.tiles_n, p.group_m);
    if (c.pid_m >= p.skip_tile0) c.pid_m += p.skip_tiles;
    return c;
  };
  const int num_tiles = tiles_m * p.tiles_n * p.batch;
  const bool swiglu = p.epilogue == B200K_EPI_SWIGLU;
  const int bn = p.pair_bn;         // tile width: 256, or 128 when that wastes less of the last wave
  const int b_rows = bn / 2;        // rows (columns of C) of B this CTA stages
  const int cluster_id = blockIdx.x >> 1;
  const int num_clusters = gridDim.x >> 1;

  if (warp == 0) {
    // ---------------- TMA producer (both CTAs) ----------------
    // warp-uniform loop, one elected lane issues (see the MMA warp)
    {
      const bool elected = elect_one();
      uint32_t it = 0;
      bool ok = true;
      for (int tile = cluster_id; tile < num_tiles && ok; tile += num_clusters) {
        const TileCoord tc = coord_of(tile);
        int group = tc.batch, a_batch = tc.batch;
        if (p.tile_group != nullptr) {
          group = p.tile_group[tc.pid_m];
          a_batch = 0;
          if (group < 0) continue;
        }
        const int m0 = tc.pid_m * 256 + rank * 128;
        // SwiGLU: the leader stages 128 gate rows of B, its peer the matching up rows
        const int nb = swiglu ? tc.pid_n * 128 + static_cast<int>(rank) * (p.n / 2)
                              : tc.pid_n * bn + static_cast<int>(rank) * b_rows;
        const int sfb_tile0 = group * p.sfb_group_tiles + (swiglu ? tc.pid_n : tc.pid_n * 2);
        for (int kb = 0; kb < p.k_iters; ++kb, ++it) {
          const int s = it % S;
          const uint32_t ph = (it / S) & 1;
          if (!mbar_wait_relaxed(empty_bar(s), ph ^ 1, abort_flag, 64, p.wait_budget_ns)) {
            report_status(p.status, 51, s);
            *abort_flag = 1;
            ok = false;
            break;
          }
          // the leader's barrier collects the bytes of both CTAs
          const uint32_t lead_full = map_to_cta(full_bar(s), 0);
          const uint32_t a_dst = tiles_base + s * Cfg::kStageBytes;
          const uint32_t b_dst = a_dst + Cfg::kABytes;
          const int kx = kb * (KIND == kKindNVF4 ? 128 : Cfg::kBKElems);
          if (elected) {
            if (leader) mbar_arrive_expect_tx(full_bar(s), 2 * (Cfg::kABytes + b_rows * 128 + Cfg::kSfBytes));
            tma_load_3d_pair(a_dst, &tmap_a, lead_full, kx, m0, a_batch);
            if (!p.b_mn) {
              tma_load_3d_pair(b_dst, &tmap_b, lead_full, kx, nb, group);   // box of b_rows rows
            } else {
              // N-contiguous B: boxes of 128 bytes of N by one k-step of K rows
              for (int j = 0; j < b_rows / Cfg::kBBoxN; ++j)
                tma_load_3d_pair(b_dst + j * Cfg::kBBoxBytes, &tmap_b, lead_full, nb + j * Cfg::kBBoxN,
                                 kb * Cfg::kBKElems, group);
            }
            if constexpr (Cfg::kScaled) {
              const uint32_t sfa_dst = sf_base + s * Cfg::kSfBytes;
              const uint32_t sfb_dst = sfa_dst + Cfg::kSfAtoms * 512;
              tma_load_3d_pair(sfa_dst, &tmap_sfa, lead_full, 0, kb * Cfg::kSfAtoms, tc.pid_m * 2 + rank);
              if (!swiglu) {
                // both 128-row tiles of SFB in one box: [row tile][atom][512 B] in shared memory
                tma_load_3d_pair(sfb_dst, &tmap_sfb, lead_full, 0, kb * Cfg::kSfAtoms, sfb_tile0);
              } else {
                // gate and up tiles are N / 256 row tiles apart: one-tile boxes
                tma_load_3d_pair(sfb_dst, &tmap_sfb, lead_full, 0, kb * Cfg::kSfAtoms, sfb_tile0);
                tma_load_3d_pair(sfb_dst + Cfg::kSfAtoms * 512, &tmap_sfb, lead_full, 0, kb * Cfg::kSfAtoms,
                                 sfb_tile0 + p.n / 256);
              }
            }
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1 || warp == 6) {
    // ---------------- MMA issuers (leader only) ----------------
    // The whole warp walks the loop so that descriptors and addresses stay warp-uniform
    // (uniform registers feed the MMA directly); one elected lane issues the tcgen05 work.
    // Issuer q takes the k-steps kb = q, q + 2, ... of every tile.
    if (leader) {
      const int q = warp == 1 ? 0 : 1;
      const bool elected = elect_one();
      uint32_t it_base = 0;
      uint32_t lt = 0;
      bool ok = true;
      uint32_t tsfa = 0, tsfb = 0;
      if constexpr (Cfg::kScaled) {
        tsfa = tmem_base + Cfg::kSfBase + q * Cfg::kSfSlotCols;
        tsfb = tsfa + Cfg::kSfaCols;
      }
      if (q >= p.k_iters) ok = false;   // a single k-step: nothing for the second issuer
      for (int tile = cluster_id; tile < num_tiles && ok; tile += num_clusters) {
        if (p.tile_group != nullptr && p.tile_group[coord_of(tile).pid_m] < 0) continue;
        const int w = lt & 1;
        if (!mbar_wait(acc_empty_bar(w), ((lt >> 1) & 1) ^ 1, abort_flag, p.wait_budget_ns)) {
          report_status(p.status, 52, 100 + w);
          *abort_flag = 1;
          break;
        }
        if (Cfg::kOverlapChunks > 0 && lt > 0) {
          if (!mbar_wait(ovl_free_bar, (lt - 1) & 1, abort_flag, p.wait_budget_ns)) {
            report_status(p.status, 52, 200);
            *abort_flag = 1;
            break;
          }
        }
        if (q == 1) {
          // the k-step that overwrites the accumulator must be complete before this
          // issuer adds to it
          if (!mbar_wait(tile_open_bar(w), (lt >> 1) & 1, abort_flag, p.wait_budget_ns)) {
            report_status(p.status, 52, 300 + w);
            *abort_flag = 1;
            break;
          }
        }
        tc_fence_after_sync();
        const uint32_t tmem_acc = tmem_base + w * Cfg::kAccStride;
        for (int kb = q; kb < p.k_iters; kb += 2) {
          const uint32_t it = it_base + kb;
          const int s = it % S;
          const uint32_t ph = (it / S) & 1;
          if (!mbar_wait(full_bar(s), ph, abort_flag, p.wait_budget_ns)) {
            report_status(p.status, 52, s);
            *abort_flag = 1;
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t a_addr = tiles_base + s * Cfg::kStageBytes;
          const uint32_t b_addr = a_addr + Cfg::kABytes;
          const uint64_t a_desc = make_smem_desc(a_addr, 16, 1024, kSwizzle128B);
          // MN-major: groups of eight k-rows 1024 bytes apart; tf32: groups of four, 512 apart
          const uint64_t b_desc = p.b_mn ? make_smem_desc(b_addr, Cfg::kBBoxBytes, KIND == kKindTF32 ? 512 : 1024,
                                                          KIND == kKindTF32 ? kSwizzle128BBase32B : kSwizzle128B)
                                         : make_smem_desc(b_addr, 16, 1024, kSwizzle128B);
          const uint32_t b_step = p.b_mn ? Cfg::kMmaK * 128 / 16 : 2;   // descriptor advance per MMA
          const int n_mma = (kb == p.k_iters - 1) ? p.k_tail_mmas : 4;
          if constexpr (Cfg::kScaled) {
            // this issuer's slot: its previous MMAs precede these copies in program order
            const uint32_t sfa_addr = sf_base + s * Cfg::kSfBytes;
            const uint32_t sfb_addr = sfa_addr + Cfg::kSfAtoms * 512;
#pragma unroll
            for (int ka = 0; ka < Cfg::kSfAtoms; ++ka) {
              const uint64_t da = make_smem_desc(sfa_addr + ka * 512, 128, 128, kSwizzleNone);
              if (elected) tmem_cp_sf_atom_pair(tsfa + ka * 4, da);
#pragma unroll
              for (int j = 0; j < 2; ++j) {
                const uint64_t db = make_smem_desc(sfb_addr + (j * Cfg::kSfAtoms + ka) * 512, 128, 128, kSwizzleNone);
                if (elected) tmem_cp_sf_atom_pair(tsfb + ka * 8 + j * 4, db);
              }
            }
          }
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) {
            if (kk < n_mma && elected) {
              const uint32_t acc = (kb > 0 || kk > 0) ? 1u : 0u;
              const uint64_t a_d = a_desc + static_cast<uint64_t>(kk * 2);
              const uint64_t b_d = b_desc + static_cast<uint64_t>(kk * b_step);
              if constexpr (KIND == kKindMXF8) {
                umma_block_scaled_pair<KIND>(tmem_acc, a_d, b_d,
                                             p.idesc | (uint32_t(kk) << 29) | (uint32_t(kk) << 4), acc, tsfa, tsfb);
              } else if constexpr (KIND == kKindNVF4) {
                umma_block_scaled_pair<KIND>(tmem_acc, a_d, b_d, p.idesc, acc, tsfa + kk * 4, tsfb + kk * 8);
              } else {
                umma_pair<KIND>(tmem_acc, a_d, b_d, p.idesc, acc);
              }
            }
          }
          // release the stage in both CTAs
          const uint32_t e0 = map_to_cta(empty_bar(s), 0), e1 = map_to_cta(empty_bar(s), 1);
          if (elected) {
            tc_commit_pair(e0);
            tc_commit_pair(e1);
            if (kb == 0 && p.k_iters > 1 && !p.withhold_arrival) tc_commit_pair(map_to_cta(tile_open_bar(w), 0));
          }
        }
        if (ok) {
          const uint32_t f0 = map_to_cta(acc_full_bar(w), 0), f1 = map_to_cta(acc_full_bar(w), 1);
          if (elected) {
            tc_commit_pair(f0);
            tc_commit_pair(f1);
          }
        }
        ++lt;
        it_base += p.k_iters;
      }
    }
    __syncwarp();
  } else if (warp < 6) {
    // ---------------- epilogue (both CTAs) ----------------
    const int quarter = warp & 3;
    float alpha = p.alpha;
    if (p.alpha_a != nullptr) alpha *= *p.alpha_a;
    if (p.alpha_b != nullptr) alpha *= *p.alpha_b;
    constexpr bool kQuantOut = (OUT == kOutMX8 || OUT == kOutNVF4);
    // bytes of `e` output elements (kOutNVF4: two elements per byte, even counts only)
    constexpr int elem_bytes = (OUT == kOutF32) ? 4 : (kQuantOut ? 1 : 2);
    auto out_bytes = [](int64_t e) { return OUT == kOutNVF4 ? e / 2 : e * elem_bytes; };
    const bool vec_ok = (out_bytes(p.ldc) % 16 == 0) && (out_bytes(p.stride_c) % 16 == 0) &&
                        (reinterpret_cast<uintptr_t>(p.c) % 16 == 0);
    float nv_st = 0.0f, nv_six_st = 0.0f;   // kOutNVF4: tensor scale of the output and 6 x it
    if constexpr (OUT == kOutNVF4) {
      nv_st = *p.c_scale;
      nv_six_st = __fmul_rn(6.0f, nv_st);
    }
    const uint32_t lead_ovl = map_to_cta(ovl_free_bar, 0);
    uint32_t lt = 0;
    for (int tile = cluster_id; tile < num_tiles; tile += num_clusters) {
      const TileCoord tc = coord_of(tile);
      if (p.tile_group != nullptr && p.tile_group[tc.pid_m] < 0) continue;
      const int w = lt & 1;
      if (!mbar_wait_relaxed(acc_full_bar(w), (lt >> 1) & 1, abort_flag, 64, p.wait_budget_ns)) {
        report_status(p.status, 53, w);
        *abort_flag = 1;
        break;
      }
      tc_fence_after_sync();
      const int row = tc.pid_m * 256 + rank * 128 + quarter * 32 + lane;
      int64_t out_row = row;
      bool row_ok = row < p.m;
      float scale = alpha;
      uint8_t* c_base = static_cast<uint8_t*>(p.c);
      if (p.row_map != nullptr && row_ok) {
        out_row = p.row_map[row];
        if (p.num_c_peers > 0) {
          // the row belongs to buffer out_row / c_peer_rows (a peer's, or this GPU's own)
          row_ok = out_row >= 0 && out_row < p.c_peer_rows * p.num_c_peers;
          if (row_ok) {
            const int64_t buf = out_row / p.c_peer_rows;
            out_row -= buf * p.c_peer_rows;
            c_base = static_cast<uint8_t*>(p.c_peers[buf]);
            if (p.row_scale != nullptr) scale *= p.row_scale[row];
          }
        } else {
          row_ok = out_row >= 0 && out_row < p.c_rows;
          if (p.row_scale != nullptr && row_ok) scale *= p.row_scale[out_row];
        }
      } else if (p.row_scale != nullptr && row_ok) {
        scale *= p.row_scale[out_row];
      }
      uint8_t* c_row = c_base +
                       out_bytes(static_cast<int64_t>(p.tile_group ? 0 : tc.batch) * p.stride_c + out_row * p.ldc);
      const uint32_t taddr = tmem_base + w * Cfg::kAccStride + (uint32_t(quarter * 32) << 16);
      // Columns shared with the other window first (the last chunks of window 0, the first
      // chunks of window 1): they are pulled into registers back to back and released
      // before anything is converted or stored, so the next tile's first MMA waits only
      // for these loads.
      const int first = (w == 0) ? (8 - Cfg::kOverlapChunks) & 7 : 0;
      constexpr int kOvl = Cfg::kOverlapChunks > 0 ? Cfg::kOverlapChunks : 1;
      uint32_t held[kOvl][32];
      if constexpr (Cfg::kOverlapChunks > 0) {
#pragma unroll
        for (int ci = 0; ci < Cfg::kOverlapChunks; ++ci)
          tmem_ld_32x32b_x32(taddr + ((first + ci) & 7) * 32, held[ci]);
        tmem_ld_wait();
        tc_fence_before_sync();
      }
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster_relaxed(lead_ovl);
      // kOutMX8: the 32 columns of a chunk are one MX block of the row.  The values are
      // first rounded to bf16, so the bytes equal those of writing a bf16 tensor and
      // running the MXFP8 quantiser over it.
      auto store_mx = [&](int col, float (&v)[32]) {
        if constexpr (OUT == kOutMX8) {
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = __bfloat162float(__float2bfloat16_rn(v[i]));
          uint32_t pk[8];
          const uint8_t sf = mx_quantize_block32(v, pk);
          uint8_t* dst = c_row + col;
          if (vec_ok) {
            reinterpret_cast<uint4*>(dst)[0] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
            reinterpret_cast<uint4*>(dst)[1] = make_uint4(pk[4], pk[5], pk[6], pk[7]);
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) dst[i] = (pk[i >> 2] >> (8 * (i & 3))) & 0xff;
          }
          p.c_sf[swizzled_sf_offset(out_row, col >> 5, p.c_sf_k_atoms)] = sf;
        } else if constexpr (OUT == kOutNVF4) {
          // two NVFP4 blocks of 16 columns: 16 bytes of codes, two neighbouring scale bytes;
          // again the bytes of quantising the bf16-rounded values with the given tensor scale
          float lo16[16], hi16[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            lo16[i] = __bfloat162float(__float2bfloat16_rn(v[i]));
            hi16[i] = __bfloat162float(__float2bfloat16_rn(v[16 + i]));
          }
          uint32_t w[4];
          const uint8_t s0 = nvfp4_block(lo16, nv_six_st, nv_st, &w[0], &w[1]);
          const uint8_t s1 = nvfp4_block(hi16, nv_six_st, nv_st, &w[2], &w[3]);
          uint8_t* dst = c_row + (col >> 1);
          if (vec_ok) {
            *reinterpret_cast<uint4*>(dst) = make_uint4(w[0], w[1], w[2], w[3]);
          } else {
#pragma unroll
            for (int i = 0; i < 16; ++i) dst[i] = (w[i >> 2] >> (8 * (i & 3))) & 0xff;
          }
          *reinterpret_cast<uint16_t*>(p.c_sf + swizzled_sf_offset(out_row, col >> 4, p.c_sf_k_atoms)) =
              static_cast<uint16_t>(s0) | (static_cast<uint16_t>(s1) << 8);
        }
      };
      // Coalesced store path (plain STORE epilogue, 16-byte-aligned rows): a lane holds 128
      // bytes of ONE row per group of columns, so storing from registers makes every warp
      // store touch 32 different cache lines - 4096 store wavefronts per tile and CTA, more
      // LSU time than a tile of 12 - 16 k-steps has MMA time.  Each warp therefore turns its
      // 32 x 128-byte block through shared memory (XOR-swizzled 16-byte pieces, conflict
      // free both ways) and writes it back with eight lanes per row: four full lines per
      // instruction.  The host selects this form unless the caller asks for direct stores.
      constexpr int kGroupCols = (OUT == kOutF32) ? 32 : 64;     // 128 bytes of a row
      const bool coalesced = !kQuantOut && p.coalesce_store && !swiglu && vec_ok &&
                             ((p.n * elem_bytes) % 16 == 0);
      if (coalesced) {
        const int n0 = tc.pid_n * bn;
        const uint32_t stg = staging_base + (warp - 2) * 4096;
        const int piece = lane & 7;
        // the eight rows this lane stores (row i * 4 + lane / 8 of the warp's 32): their
        // output pointers and validity come from the lanes that own those rows
        const uint64_t my_ptr = reinterpret_cast<uint64_t>(c_row);
        uint64_t row_ptr[8];
        uint32_t row_valid = 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int src = i * 4 + (lane >> 3);
          row_ptr[i] = __shfl_sync(0xffffffffu, my_ptr, src);
          row_valid |= (__shfl_sync(0xffffffffu, row_ok ? 1u : 0u, src) & 1u) << i;
        }
        const int64_t n_bytes = static_cast<int64_t>(p.n) * elem_bytes;
        auto fetch = [&](int c, uint32_t (&r)[32]) {
          bool from_held = false;
          if constexpr (Cfg::kOverlapChunks > 0) {
#pragma unroll
            for (int ci = 0; ci < Cfg::kOverlapChunks; ++ci) {
              if (c == ((first + ci) & 7)) {
#pragma unroll
                for (int i = 0; i < 32; ++i) r[i] = held[ci][i];
                from_held = true;
              }
            }
          }
          if (!from_held) tmem_ld_32x32b_x32(taddr + c * 32, r);
        };
#pragma unroll 1
        for (int g = 0; g < bn / kGroupCols; ++g) {
          uint32_t out[32];   // this lane's 128 bytes of the group
          if constexpr (OUT == kOutF32) {
            uint32_t r[32];
            fetch(g, r);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) out[i] = __float_as_uint(__uint_as_float(r[i]) * scale);
          } else {
            uint32_t ra[32], rb[32];
            fetch(2 * g, ra);
            fetch(2 * g + 1, rb);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              const float a0 = __uint_as_float(ra[2 * i]) * scale, a1 = __uint_as_float(ra[2 * i + 1]) * scale;
              const float b0 = __uint_as_float(rb[2 * i]) * scale, b1 = __uint_as_float(rb[2 * i + 1]) * scale;
              out[i] = (OUT == kOutBF16) ? pack_bf16x2(a0, a1) : pack_f16x2(a0, a1);
              out[16 + i] = (OUT == kOutBF16) ? pack_bf16x2(b0, b1) : pack_f16x2(b0, b1);
            }
          }
#pragma unroll
          for (int j = 0; j < 8; ++j)
            st_shared_v4(stg + lane * 128 + ((j ^ (lane & 7)) << 4), out[4 * j], out[4 * j + 1], out[4 * j + 2],
                         out[4 * j + 3]);
          __syncwarp();
          const int64_t col_byte = static_cast<int64_t>(n0 + g * kGroupCols) * elem_bytes + piece * 16;
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int row_in_warp = i * 4 + (lane >> 3);
            uint32_t q[4];
            ld_shared_v4(stg + row_in_warp * 128 + ((piece ^ (row_in_warp & 7)) << 4), q);
            if (((row_valid >> i) & 1u) && col_byte + 16 <= n_bytes)
              *reinterpret_cast<uint4*>(row_ptr[i] + col_byte) = make_uint4(q[0], q[1], q[2], q[3]);
          }
          __syncwarp();
        }
      } else if (!swiglu) {
        const int n0 = tc.pid_n * bn;
        const int chunks = bn / 32;
        auto emit = [&](int c, const uint32_t (&r)[32]) {
          if (row_ok && n0 + c * 32 < p.n) {
            float v[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]) * scale;
            if constexpr (kQuantOut) store_mx(n0 + c * 32, v);
            else store_row_chunk<OUT>(c_row, n0 + c * 32, p.n, v, vec_ok);
          }
        };
        if constexpr (Cfg::kOverlapChunks > 0) {
#pragma unroll
          for (int ci = 0; ci < Cfg::kOverlapChunks; ++ci) emit((first + ci) & 7, held[ci]);
        }
#pragma unroll 1
        for (int ci = Cfg::kOverlapChunks; ci < chunks; ++ci) {
          const int c = (first + ci) & 7;
          uint32_t r[32];
          tmem_ld_32x32b_x32(taddr + c * 32, r);
          tmem_ld_wait();
          emit(c, r);
        }
      } else if constexpr (Cfg::kOverlapChunks <= 1) {
        // columns [0, 128) of the tile are gate, [128, 256) the matching up projections
        const int n_out = p.n / 2;
        const int n0 = tc.pid_n * 128;
        auto fetch = [&](int c, uint32_t (&r)[32]) {
          if (Cfg::kOverlapChunks == 1 && c == first) {
#pragma unroll
            for (int i = 0; i < 32; ++i) r[i] = held[0][i];
          } else {
            tmem_ld_32x32b_x32(taddr + c * 32, r);
          }
        };
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          uint32_t g[32], u[32];
          fetch(c, g);
          fetch(c + 4, u);
          tmem_ld_wait();
          if (row_ok && n0 + c * 32 < n_out) {
            float v[32];
#pragma unroll
            for (int i = 0; i < 32; ++i)
              v[i] = silu(__uint_as_float(g[i]) * scale) * (__uint_as_float(u[i]) * scale);
            if constexpr (kQuantOut) store_mx(n0 + c * 32, v);
            else store_row_chunk<OUT>(c_row, n0 + c * 32, n_out, v, vec_ok);
          }
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster_relaxed(map_to_cta(acc_empty_bar(w), 0));
      ++lt;
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();   // the peer may still be reading our barriers / TMEM pairing
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc_pair(tmem_base, kTmemCols);
  }
}

namespace {

template <int KIND, int OUT>
int launch_pair(const CUtensorMap* maps, const GemmParams& p, int grid, cudaStream_t stream) {
  using Cfg = PairCfg<KIND>;
  auto kernel = gemm_pair_kernel<KIND, OUT>;
  static bool configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes);
    if (e != cudaSuccess)
      return fail(B200K_CUDA_ERROR, "cudaFuncSetAttribute(%d bytes): %s", Cfg::kSmemBytes, cudaGetErrorString(e));
    configured[dev] = true;
  }
  if (!p.programmatic_launch) {
    kernel<<<grid, Cfg::kThreads, Cfg::kSmemBytes, stream>>>(maps[0], maps[1], maps[2], maps[3], p);
  } else {
    cudaError_t e = launch_after_predecessor(kernel, dim3(grid), dim3(Cfg::kThreads), Cfg::kSmemBytes, stream,
                                             maps[0], maps[1], maps[2], maps[3], p);
    if (e != cudaSuccess) return fail(B200K_CUDA_ERROR, "gemm (CTA pair) launch: %s", cudaGetErrorString(e));
  }
  B200K_CHECK_LAUNCH("gemm (CTA pair) launch");
  return B200K_OK;
}

template <int KIND>
int launch_pair_out(int out, const CUtensorMap* maps, const GemmParams& p, int grid, cudaStream_t stream) {
  switch (out) {
    case B200K_F16: return launch_pair<KIND, kOutF16>(maps, p, grid, stream);
    case B200K_BF16: return launch_pair<KIND, kOutBF16>(maps, p, grid, stream);
    case B200K_F32: return launch_pair<KIND, kOutF32>(maps, p, grid, stream);
    case B200K_E4M3:
      if constexpr (KIND == kKindMXF8) return launch_pair<KIND, kOutMX8>(maps, p, grid, stream);
      return fail(B200K_UNSUPPORTED, "MXFP8 output is available for MXFP8 operands only");
    case B200K_E2M1X2:
      if constexpr (KIND == kKindMXF8 || KIND == kKindNVF4)
        return launch_pair<KIND, kOutNVF4>(maps, p, grid, stream);
      return fail(B200K_UNSUPPORTED, "NVFP4 output is available for block-scaled operands only");
    default: return fail(B200K_INVALID_ARG, "unsupported output dtype %d", out);
  }
}

}  // namespace

int launch_gemm_pair(int kind, int out_dtype, const CUtensorMap* maps, const GemmParams& p_in, int sms,
                     cudaStream_t stream) {
  GemmParams p = p_in;
  if (p.pair_bn != 128) p.pair_bn = 256;
  if (p.wait_budget_ns == 0) p.wait_budget_ns = kWaitBudgetNs;
  if (p.group_m <= 0) p.group_m = kGroupM;
  // Stores staged through shared memory unless the caller asks for the direct form: direct
  // stores take about 8000 cycles per tile (16-bit output; twice the store instructions for
  // fp32) against about 530 per k-step, which decides short-K problems, and measured on
  // 8192-deep problems the staged form is also ahead (MXFP8 8192 cubed +1 %, NVFP4
  // 8192 x 28672 x 8192 +4 %).
  p.coalesce_store = p.store_mode != 1;
  const int64_t tiles = static_cast<int64_t>((p.m + 255) / 256) * p.tiles_n * p.batch;
  int clusters = static_cast<int>(tiles < sms / 2 ? tiles : sms / 2);
  if (clusters < 1) clusters = 1;
  const int grid = clusters * 2;
  switch (kind) {
    case kKindF16: return launch_pair_out<kKindF16>(out_dtype, maps, p, grid, stream);
    case kKindTF32: return launch_pair_out<kKindTF32>(out_dtype, maps, p, grid, stream);
    case kKindF8: return launch_pair_out<kKindF8>(out_dtype, maps, p, grid, stream);
    case kKindMXF8: return launch_pair_out<kKindMXF8>(out_dtype, maps, p, grid, stream);
    case kKindNVF4: return launch_pair_out<kKindNVF4>(out_dtype, maps, p, grid, stream);
    default: return fail(B200K_INVALID_ARG, "unknown kind %d", kind);
  }
}

}  // namespace b200k
