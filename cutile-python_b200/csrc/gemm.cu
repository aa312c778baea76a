// Dense and block-scaled GEMM for sm_100a: one persistent, warp-specialised kernel
// template built on TMA loads, an mbarrier ring and tcgen05 MMA with the
// accumulator in tensor memory.
//
//   warp 0      TMA producer (one lane): A / B / scale-factor tiles -> shared memory
//   warp 1      MMA issuer (one lane): [scale factors smem -> TMEM,] 4 MMAs per stage
//   warps 2..5  epilogue: TMEM -> registers -> global (each warp owns 32 TMEM lanes)
//
// CTA tile: 128 x BN, one 128-byte swizzle atom of K per stage (64 f16 / 32 tf32 /
// 128 fp8 / 256 fp4 elements).  Tiles are walked persistently in the grouped
// raster order of the reference (GROUP_SIZE_M = 8, test/kernels/matmul.py:13-23).
//
// Semantics follow the reference kernels: fp32 accumulation, zero padding of
// partial tiles (TMA out-of-bounds fill), result rounded once to the output type
// (test/kernels/matmul.py:70-100, test/kernels/scaled_matmul.py:71-114).
#include <stdlib.h>

#include "gemm_common.cuh"
#include "gemm_pair.h"

namespace b200k {


template <int KIND, int BN, bool B_MN, int OUT>
__global__ void __launch_bounds__(kNumThreads, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
            const GemmParams p) {
  using Cfg = GemmCfg<KIND, BN, B_MN>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (smem_base - smem_u32(smem_raw));
  // split-K: the reduction kernel behind this one may take its place on the idle SMs now; it
  // blocks until this grid has finished
  if (p.split_k > 1) pdl_launch_dependents();

  // carve-up
  const uint32_t tiles_base = smem_base;
  const uint32_t sf_base = tiles_base + kStages * Cfg::kStageBytes;
  uint8_t* tail = smem + kStages * (Cfg::kStageBytes + Cfg::kSfBytes);
  uint64_t* bars = reinterpret_cast<uint64_t*>(tail);
  const uint32_t bar_base = smem_u32(bars);
  // full[kStages], empty[kStages], acc_full[2], acc_empty[2]
  const uint32_t staging_base = bar_base + 256;   // behind the barriers
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (kStages + s); };
  auto acc_full_bar = [&](int a) { return bar_base + 8u * (2 * kStages + a); };
  auto acc_empty_bar = [&](int a) { return bar_base + 8u * (2 * kStages + 2 + a); };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tail + 8 * (2 * kStages + 4));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tail + 8 * (2 * kStages + 4) + 8);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(acc_full_bar(a), 1);
      mbar_init(acc_empty_bar(a), 4);
    }
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  int tiles_m = p.tiles_m;
  if (p.num_row_tiles != nullptr) tiles_m = min(tiles_m, *p.num_row_tiles);
  const int num_tiles = tiles_m * p.tiles_n * p.batch;

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    // The whole warp walks the loop so that addresses and coordinates stay warp-uniform
    // (they feed the TMA unit from uniform registers); one elected lane issues.
    {
      const bool elected = elect_one();
      uint32_t it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        TileCoord tc = tile_coord(tile, tiles_m, p.tiles_n);
        // split-K: the batch index of the raster carries (batch, split)
        const int batch = p.split_k > 1 ? tc.batch / p.split_k : tc.batch;
        const int kb0 = p.split_k > 1 ? (tc.batch % p.split_k) * p.k_per_split : 0;
        const int kb1 = p.split_k > 1 ? min(p.k_iters, kb0 + p.k_per_split) : p.k_iters;
        int group = batch;
        if (p.tile_group != nullptr) {
          group = p.tile_group[tc.pid_m];
          if (group < 0) continue;
        }
        const int m0 = tc.pid_m * kBM;
        const int n0 = tc.pid_n * BN;
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int s = it % kStages;
          const uint32_t ph = (it / kStages) & 1;
          if (!mbar_wait(empty_bar(s), ph ^ 1, abort_flag)) {
            report_status(p.status, 1, s);
            *abort_flag = 1;
            ok = false;
            break;
          }
          uint32_t tx = Cfg::kStageBytes;
          int sfa_atoms = 0;
          if constexpr (Cfg::kScaled) {
            sfa_atoms = min(Cfg::kSfaAtoms, p.sf_k_atoms - kb * Cfg::kSfaAtoms);
            tx += sfa_atoms * 512 * (1 + BN / 128);
          }
          const uint32_t a_dst = tiles_base + s * Cfg::kStageBytes;
          const uint32_t b_dst = a_dst + Cfg::kABytes;
          // TMA x coordinate in tensor-map elements (fp4 maps are byte typed)
          const int kx = kb * (KIND == kKindNVF4 ? 128 : Cfg::kBKElems);
          if (elected) {
          mbar_arrive_expect_tx(full_bar(s), tx);
          tma_load_3d(a_dst, &tmap_a, full_bar(s), kx, m0, p.tile_group ? 0 : batch);
          if constexpr (B_MN) {
#pragma unroll
            for (int j = 0; j < Cfg::kBBoxes; ++j)
              tma_load_3d(b_dst + j * Cfg::kBBoxBytes, &tmap_b, full_bar(s),
                          n0 + j * Cfg::kBBoxN, kb * Cfg::kBKElems, group);
          } else {
#pragma unroll
            for (int j = 0; j < Cfg::kBBoxes; ++j) {
              int row = n0 + j * 128;
              // SwiGLU: the second half of the tile holds the "up" columns, which
              // live N/2 rows further down in B.
              if (p.epilogue == B200K_EPI_SWIGLU) row = n0 / 2 + (j >= Cfg::kBBoxes / 2 ? p.n / 2 + (j - Cfg::kBBoxes / 2) * 128 : j * 128);
              tma_load_3d(b_dst + j * 128 * 128, &tmap_b, full_bar(s), kx, row, group);
            }
          }
          if constexpr (Cfg::kScaled) {
            const uint32_t sfa_dst = sf_base + s * Cfg::kSfBytes;
            const uint32_t sfb_dst = sfa_dst + Cfg::kSfaAtoms * 512;
            const uint8_t* sfa_src = p.sfa + (p.tile_group ? 0 : batch) * p.stride_sfa +
                                     (static_cast<int64_t>(tc.pid_m) * p.sf_k_atoms + kb * Cfg::kSfaAtoms) * 512;
            bulk_load(sfa_dst, sfa_src, sfa_atoms * 512, full_bar(s));
#pragma unroll
            for (int j = 0; j < BN / 128; ++j) {
              int row_tile = (n0 >> 7) + j;
              if (p.epilogue == B200K_EPI_SWIGLU)
                row_tile = (n0 >> 8) + (j >= BN / 256 ? (p.n >> 8) + (j - BN / 256) : j);
              row_tile = min(row_tile, p.sfb_row_tiles - 1);
              const uint8_t* sfb_src = p.sfb + group * p.stride_sfb +
                                       (static_cast<int64_t>(row_tile) * p.sf_k_atoms + kb * Cfg::kSfaAtoms) * 512;
              bulk_load(sfb_dst + j * Cfg::kSfaAtoms * 512, sfb_src, sfa_atoms * 512, full_bar(s));
            }
          }
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    {
      const bool elected = elect_one();
      uint32_t it = 0;
      uint32_t local_tile = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        int kb0 = 0, kb1 = p.k_iters;
        if (p.tile_group != nullptr || p.split_k > 1) {
          TileCoord tc = tile_coord(tile, tiles_m, p.tiles_n);
          if (p.tile_group != nullptr && p.tile_group[tc.pid_m] < 0) continue;
          if (p.split_k > 1) {
            kb0 = (tc.batch % p.split_k) * p.k_per_split;
            kb1 = min(p.k_iters, kb0 + p.k_per_split);
          }
        }
        const int as = local_tile % Cfg::kNumAcc;
        const uint32_t aph = (local_tile / Cfg::kNumAcc) & 1;
        if (!mbar_wait(acc_empty_bar(as), aph ^ 1, abort_flag)) {
          report_status(p.status, 2, 100 + as);
          *abort_flag = 1;
          break;
        }
        tc_fence_after_sync();
        const uint32_t tmem_acc = tmem_base + as * Cfg::kAccStride;
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int s = it % kStages;
          const uint32_t ph = (it / kStages) & 1;
          if (!mbar_wait(full_bar(s), ph, abort_flag)) {
            report_status(p.status, 2, s);
            *abort_flag = 1;
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t a_addr = tiles_base + s * Cfg::kStageBytes;
          const uint32_t b_addr = a_addr + Cfg::kABytes;
          const uint64_t a_desc = make_smem_desc(a_addr, 16, 1024, kSwizzle128B);
          // MN-major: groups of eight k-rows 1024 bytes apart; tf32: groups of four, 512 apart
          const uint64_t b_desc = B_MN ? make_smem_desc(b_addr, Cfg::kBBoxBytes, KIND == kKindTF32 ? 512 : 1024,
                                                        KIND == kKindTF32 ? kSwizzle128BBase32B : kSwizzle128B)
                                       : make_smem_desc(b_addr, 16, 1024, kSwizzle128B);
          const int n_mma = (kb == p.k_iters - 1) ? p.k_tail_mmas : 4;
          uint32_t tsfa = 0, tsfb = 0;
          if constexpr (Cfg::kScaled) {
            tsfa = tmem_base + Cfg::kSfTmemBase + s * Cfg::kSfaCols;
            tsfb = tmem_base + Cfg::kSfTmemBase + kStages * Cfg::kSfaCols + s * Cfg::kSfbCols;
            const uint32_t sfa_addr = sf_base + s * Cfg::kSfBytes;
            const uint32_t sfb_addr = sfa_addr + Cfg::kSfaAtoms * 512;
            const int atoms = min(Cfg::kSfaAtoms, p.sf_k_atoms - kb * Cfg::kSfaAtoms);
            for (int ka = 0; ka < atoms; ++ka) {
              const uint64_t da = make_smem_desc(sfa_addr + ka * 512, 128, 128, kSwizzleNone);
              if (elected) tmem_cp_sf_atom(tsfa + ka * 4, da);
#pragma unroll
              for (int j = 0; j < BN / 128; ++j) {
                const uint64_t db = make_smem_desc(sfb_addr + (j * Cfg::kSfaAtoms + ka) * 512, 128, 128, kSwizzleNone);
                if (elected) tmem_cp_sf_atom(tsfb + ka * (BN / 128) * 4 + j * 4, db);
              }
            }
          }
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) {
            if (kk < n_mma && elected) {
              const uint32_t acc = (kb > kb0 || kk > 0) ? 1u : 0u;
              // K-major: 32 bytes of K per MMA inside the 128-byte swizzle atom.
              // MN-major B: kMmaK rows of 128 bytes per MMA.
              const uint64_t a_d = a_desc + static_cast<uint64_t>(kk * 2);
              const uint64_t b_d = b_desc + static_cast<uint64_t>(B_MN ? kk * (Cfg::kMmaK * 128 / 16) : kk * 2);
              if constexpr (KIND == kKindMXF8) {
                // one scale byte per 32-element block: block kk of this stage
                umma_block_scaled<KIND>(tmem_acc, a_d, b_d, p.idesc | (uint32_t(kk) << 29) | (uint32_t(kk) << 4),
                                        acc, tsfa, tsfb);
              } else if constexpr (KIND == kKindNVF4) {
                // four scale bytes per MMA: atom kk of this stage
                umma_block_scaled<KIND>(tmem_acc, a_d, b_d, p.idesc, acc, tsfa + kk * 4,
                                        tsfb + kk * (BN / 128) * 4);
              } else {
                umma<KIND>(tmem_acc, a_d, b_d, p.idesc, acc);
              }
            }
          }
          if (elected) tc_commit(empty_bar(s));
        }
        if (ok && elected) tc_commit(acc_full_bar(as));
        ++local_tile;
      }
    }
    __syncwarp();
  } else {
    // ---------------- epilogue ----------------
    const int quarter = warp & 3;  // TMEM lanes [32 * quarter, 32 * quarter + 32)
    float alpha = p.alpha;
    if (p.alpha_a != nullptr) alpha *= *p.alpha_a;
    if (p.alpha_b != nullptr) alpha *= *p.alpha_b;
    const int elem_bytes = (OUT == kOutF32) ? 4 : 2;
    const bool swiglu = p.epilogue == B200K_EPI_SWIGLU;
    const int n_out = swiglu ? p.n / 2 : p.n;
    const bool vec_ok = ((p.ldc * elem_bytes) % 16 == 0) && ((p.stride_c * elem_bytes) % 16 == 0) &&
                        (reinterpret_cast<uintptr_t>(p.c) % 16 == 0);
    uint32_t local_tile = 0;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
      TileCoord tc = tile_coord(tile, tiles_m, p.tiles_n);
      if (p.tile_group != nullptr && p.tile_group[tc.pid_m] < 0) continue;
      const int as = local_tile % Cfg::kNumAcc;
      const uint32_t aph = (local_tile / Cfg::kNumAcc) & 1;
      if (!mbar_wait(acc_full_bar(as), aph, abort_flag)) {
        report_status(p.status, 3, as);
        *abort_flag = 1;
        break;
      }
      tc_fence_after_sync();
      const int row = tc.pid_m * kBM + quarter * 32 + lane;
      int64_t out_row = row;
      bool row_ok = row < p.m;
      if (p.row_map != nullptr && row_ok) {
        out_row = p.row_map[row];
        row_ok = out_row >= 0 && out_row < p.c_rows;
      }
      float scale = alpha;
      if (p.row_scale != nullptr && row_ok) scale *= p.row_scale[out_row];
      uint8_t* c_row = static_cast<uint8_t*>(p.c) +
                       (static_cast<int64_t>(p.tile_group ? 0 : tc.batch) * p.stride_c + out_row * p.ldc) * elem_bytes;
      const uint32_t taddr = tmem_base + as * Cfg::kAccStride + (uint32_t(quarter * 32) << 16);
      // Short-K tiles (split-K partials above all) are bound by their stores: a lane owns one
      // row, so a store from registers touches 32 cache lines.  Same remedy as in the
      // CTA-pair kernel: the warp turns its 32 x 128-byte block through an XOR-swizzled
      // staging buffer and stores with eight lanes per row.
      constexpr int kGroupCols = (OUT == kOutF32) ? 32 : 64;     // 128 bytes of a row
      const bool coalesced = Cfg::kStagingBytes > 0 && p.coalesce_store && !swiglu && vec_ok &&
                             ((p.n * elem_bytes) % 16 == 0);
      if (coalesced) {
        const int n0 = tc.pid_n * BN;
        const uint32_t stg = staging_base + (warp - 2) * 4096;
        const int piece = lane & 7;
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
#pragma unroll 1
        for (int g = 0; g < BN / kGroupCols; ++g) {
          uint32_t out[32];   // this lane's 128 bytes of the group
          if constexpr (OUT == kOutF32) {
            uint32_t r[32];
            tmem_ld_32x32b_x32(taddr + g * 32, r);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) out[i] = __float_as_uint(__uint_as_float(r[i]) * scale);
          } else {
            uint32_t ra[32], rb[32];
            tmem_ld_32x32b_x32(taddr + g * 64, ra);
            tmem_ld_32x32b_x32(taddr + g * 64 + 32, rb);
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
        const int n0 = tc.pid_n * BN;
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t r[32];
          tmem_ld_32x32b_x32(taddr + c * 32, r);
          tmem_ld_wait();
          if (row_ok && n0 + c * 32 < p.n) {
            float v[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]) * scale;
            store_row_chunk<OUT>(c_row, n0 + c * 32, p.n, v, vec_ok);
          }
        }
      } else {
        const int n0 = tc.pid_n * (BN / 2);
#pragma unroll 1
        for (int c = 0; c < BN / 64; ++c) {
          uint32_t g[32], u[32];
          tmem_ld_32x32b_x32(taddr + c * 32, g);
          tmem_ld_32x32b_x32(taddr + BN / 2 + c * 32, u);
          tmem_ld_wait();
          if (row_ok && n0 + c * 32 < n_out) {
            float v[32];
#pragma unroll
            for (int i = 0; i < 32; ++i)
              v[i] = silu(__uint_as_float(g[i]) * scale) * (__uint_as_float(u[i]) * scale);
            store_row_chunk<OUT>(c_row, n0 + c * 32, n_out, v, vec_ok);
          }
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(acc_empty_bar(as));
      ++local_tile;
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// ---------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------
namespace {

template <int KIND, int BN, bool B_MN, int OUT>
int launch(const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, int grid,
           cudaStream_t stream) {
  using Cfg = GemmCfg<KIND, BN, B_MN>;
  auto kernel = gemm_kernel<KIND, BN, B_MN, OUT>;
  static bool configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         Cfg::kSmemBytes);
    if (e != cudaSuccess)
      return fail(B200K_CUDA_ERROR, "cudaFuncSetAttribute(%d bytes): %s", Cfg::kSmemBytes,
                  cudaGetErrorString(e));
    configured[dev] = true;
  }
  GemmParams pl = p;
  pl.coalesce_store = p.store_mode != 1;   // staged stores unless the caller asks for direct ones
  kernel<<<grid, kNumThreads, Cfg::kSmemBytes, stream>>>(ta, tb, pl);
  B200K_CHECK_LAUNCH("gemm launch");
  return B200K_OK;
}

template <int KIND, int BN, bool B_MN>
int launch_out(int out, const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p,
               int grid, cudaStream_t stream) {
  switch (out) {
    case B200K_F16: return launch<KIND, BN, B_MN, kOutF16>(ta, tb, p, grid, stream);
    case B200K_BF16: return launch<KIND, BN, B_MN, kOutBF16>(ta, tb, p, grid, stream);
    case B200K_F32: return launch<KIND, BN, B_MN, kOutF32>(ta, tb, p, grid, stream);
    default: return fail(B200K_INVALID_ARG, "unsupported output dtype %d", out);
  }
}

// Split-K plan for problems with far fewer output tiles than SMs: `split` CTAs share one
// tile, each reducing k_per_split k-steps into an fp32 partial; a second kernel sums the
// partials.  Returns 1 when splitting does not pay.
struct SplitPlan {
  int split = 1;
  int k_per_split = 0;
  int64_t workspace_bytes = 0;
};

// `forced`: 0 = decide by shape, 1 = never, n > 1 = up to n slices whatever the shape.
SplitPlan plan_split_k(int64_t m, int64_t n, int64_t batch, int k_iters, int sms, int forced) {
  SplitPlan plan;
  if (forced == 1) return plan;
  const int64_t tiles = ceil_div(m, kBM) * ceil_div(n, 256) * batch;
  int k_per;
  if (forced > 1) {
    k_per = static_cast<int>(ceil_div(k_iters, forced));
    if (k_per < 1) k_per = 1;
  } else {
    if (tiles * 4 > sms) return plan;
    const int max_split = static_cast<int>(sms / tiles);
    k_per = static_cast<int>(ceil_div(k_iters, max_split));
    if (k_per < 4) k_per = 4;
    // The second kernel and the fp32 round trip cost what some 40 k-steps of a lone tile
    // take: splitting pays only when it takes more than that off every CTA's K loop
    // (1024 cubed: 16-bit 14 us whole against 19 us split, tf32 18 against 21).
    if (k_iters - k_per < 48) return plan;
  }
  const int split = static_cast<int>(ceil_div(k_iters, k_per));
  if (split <= 1) return plan;
  plan.split = split;
  plan.k_per_split = k_per;
  plan.workspace_bytes = static_cast<int64_t>(split) * batch * m * n * 4;
  return plan;
}

// out[b][r][c] = sum over s of partial[b * split + s][r][c], rounded to the output type.
template <int OUT>
__global__ void __launch_bounds__(256)
splitk_reduce_kernel(const float* __restrict__ ws, int split, int64_t m, int64_t n, int64_t batch,
                     void* __restrict__ c, int64_t ldc, int64_t stride_c) {
  const int64_t quads = (n + 3) / 4;
  const int64_t total = batch * m * quads;
  pdl_wait();   // the partial tiles come from the kernel launched just before
  for (int64_t idx = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t qd = idx % quads;
    const int64_t row = (idx / quads) % m;
    const int64_t b = idx / (quads * m);
    const int64_t col = qd * 4;
    const int valid = static_cast<int>(n - col < 4 ? n - col : 4);
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    const float* src = ws + ((b * split) * m + row) * n + col;
    const bool vec = (n % 4 == 0);
    if (vec) {
      // independent loads, issued eight at a time: the partials are a few megabytes in L2
      // and the sum of one output quad is latency-bound otherwise
#pragma unroll 8
      for (int s = 0; s < split; ++s) {
        const float4 v = __ldg(reinterpret_cast<const float4*>(src + static_cast<int64_t>(s) * m * n));
        acc[0] += v.x; acc[1] += v.y; acc[2] += v.z; acc[3] += v.w;
      }
    } else {
      for (int s = 0; s < split; ++s, src += m * n)
        for (int i = 0; i < valid; ++i) acc[i] += src[i];
    }
    const int64_t off = b * stride_c + row * ldc + col;
    for (int i = 0; i < valid; ++i) {
      if constexpr (OUT == kOutF32) static_cast<float*>(c)[off + i] = acc[i];
      else if constexpr (OUT == kOutF16) static_cast<__half*>(c)[off + i] = __float2half_rn(acc[i]);
      else static_cast<__nv_bfloat16*>(c)[off + i] = __float2bfloat16_rn(acc[i]);
    }
  }
}

int launch_splitk_reduce(int out, const float* ws, int split, int64_t m, int64_t n, int64_t batch, void* c,
                         int64_t ldc, int64_t stride_c, cudaStream_t stream) {
  const int64_t total = batch * m * ((n + 3) / 4);
  const int grid = static_cast<int>(total / 256 + 1 < 4096 ? total / 256 + 1 : 4096);
  // launched with programmatic serialisation: it is set up while the GEMM still runs and
  // starts summing the moment that grid has finished (20.3 -> 18.4 us on the reference's
  // 256 x 256 x 4096 case)
  const dim3 g(grid), blk(256);
  cudaError_t e;
  switch (out) {
    case B200K_F16: e = launch_after_predecessor(splitk_reduce_kernel<kOutF16>, g, blk, 0, stream, ws, split, m, n, batch, c, ldc, stride_c); break;
    case B200K_BF16: e = launch_after_predecessor(splitk_reduce_kernel<kOutBF16>, g, blk, 0, stream, ws, split, m, n, batch, c, ldc, stride_c); break;
    case B200K_F32: e = launch_after_predecessor(splitk_reduce_kernel<kOutF32>, g, blk, 0, stream, ws, split, m, n, batch, c, ldc, stride_c); break;
    default: return fail(B200K_INVALID_ARG, "unsupported output dtype %d", out);
  }
  if (e != cudaSuccess) return fail(B200K_CUDA_ERROR, "split-K reduce launch: %s", cudaGetErrorString(e));
  return B200K_OK;
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// Output rows scattered over several (peer) buffers: checks the request and copies the
// pointer table into the launch parameters.
int set_c_peers(GemmParams* p, const void* const* c_peers, int32_t n, int64_t rows, bool grouped_pair,
                const void* row_map, int out_dtype) {
  if (c_peers == nullptr) return B200K_OK;
  if (!grouped_pair || row_map == nullptr)
    return fail(B200K_UNSUPPORTED, "c_peers needs a grouped problem over 256-row tiles (CTA-pair kernel) "
                "with row_map");
  if (out_dtype != B200K_F16 && out_dtype != B200K_BF16 && out_dtype != B200K_F32)
    return fail(B200K_UNSUPPORTED, "c_peers needs an f16, bf16 or f32 output");
  if (n <= 0 || n > 16 || rows <= 0) return fail(B200K_INVALID_ARG, "c_peers: 1 to 16 buffers of at least one row");
  for (int i = 0; i < n; ++i) {
    if (c_peers[i] == nullptr || !aligned16(c_peers[i]))
      return fail(B200K_INVALID_ARG, "c_peers[%d] is null or not 16-byte aligned", i);
    p->c_peers[i] = const_cast<void*>(c_peers[i]);
  }
  p->num_c_peers = n;
  p->c_peer_rows = rows;
  return B200K_OK;
}

// Rows left out of a plain product on the CTA-pair kernel (whole 256-row tiles).
int set_skip_rows(GemmParams* p, int64_t begin, int64_t count, int64_t m, bool plain_pair_single) {
  if (count == 0) return B200K_OK;
  if (!plain_pair_single)
    return fail(B200K_UNSUPPORTED, "skip_rows needs a plain problem (no groups, batch 1, store epilogue) on the "
                "CTA-pair kernel");
  if (begin < 0 || count < 0 || begin % 256 || count % 256 || begin + count > m)
    return fail(B200K_INVALID_ARG, "skip_rows [%lld, +%lld) must be whole 256-row tiles inside M = %lld",
                static_cast<long long>(begin), static_cast<long long>(count), static_cast<long long>(m));
  p->skip_tile0 = static_cast<int>(begin / 256);
  p->skip_tiles = static_cast<int>(count / 256);
  return B200K_OK;
}

// The caller's b200k_gemm_config, or, where it leaves a choice open, the process-wide
// diagnostic switches: B200K_SINGLE_CTA=1 (one-CTA kernels), B200K_PAIR_BN=128 (narrow
// pair tiles), B200K_EPILOGUE=c|d (staged / direct stores).
b200k_gemm_config effective_config(const b200k_gemm_config* c) {
  b200k_gemm_config r = {};
  if (c != nullptr) r = *c;
  if (r.kernel == 0) {
    const char* v = getenv("B200K_SINGLE_CTA");
    if (v != nullptr && v[0] == '1') r.kernel = 1;
  }
  if (r.tile_n == 0) {
    const char* v = getenv("B200K_PAIR_BN");
    if (v != nullptr) r.tile_n = v[0] == '1' ? 128 : 256;
  }
  if (r.epilogue_store == 0) {
    const char* v = getenv("B200K_EPILOGUE");
    if (v != nullptr) r.epilogue_store = v[0] == 'c' ? 2 : 1;
  }
  return r;
}

}  // namespace
}  // namespace b200k

using namespace b200k;

extern "C" int b200k_gemm(const b200k_gemm_args* a, b200k_stream stream_) {
  if (a == nullptr) return fail(B200K_INVALID_ARG, "null args");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (a->m < 0 || a->n < 0 || a->k < 0 || a->batch < 0)
    return fail(B200K_INVALID_ARG, "negative dimension");
  if (a->m == 0 || a->n == 0 || a->batch == 0) return B200K_OK;
  if (a->a == nullptr || a->b == nullptr || (a->c == nullptr && a->c_peers == nullptr))
    return fail(B200K_INVALID_ARG, "null operand pointer");
  if (a->k == 0) return fail(B200K_UNSUPPORTED, "K == 0 is not supported (C would be all zeros)");

  int kind, elem_bytes;
  uint32_t fmt;
  CUtensorMapDataType tdt;
  switch (a->ab_dtype) {
    case B200K_F16: kind = kKindF16; elem_bytes = 2; fmt = kFmtF16; tdt = CU_TENSOR_MAP_DATA_TYPE_FLOAT16; break;
    case B200K_BF16: kind = kKindF16; elem_bytes = 2; fmt = kFmtBF16; tdt = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16; break;
    case B200K_F32: kind = kKindTF32; elem_bytes = 4; fmt = kFmtTF32; tdt = CU_TENSOR_MAP_DATA_TYPE_FLOAT32; break;
    case B200K_E4M3: kind = kKindF8; elem_bytes = 1; fmt = kFmtE4M3; tdt = CU_TENSOR_MAP_DATA_TYPE_UINT8; break;
    case B200K_E5M2: kind = kKindF8; elem_bytes = 1; fmt = kFmtE5M2; tdt = CU_TENSOR_MAP_DATA_TYPE_UINT8; break;
    default: return fail(B200K_INVALID_ARG, "unsupported operand dtype %d", a->ab_dtype);
  }
  const bool b_mn = a->b_layout == B200K_B_KN;
  if (a->epilogue == B200K_EPI_SWIGLU && (b_mn || a->n % 256 != 0))
    return fail(B200K_UNSUPPORTED, "SwiGLU epilogue needs B stored (N, K) and N a multiple of 256");
  if ((a->lda * elem_bytes) % 16 || (a->ldb * elem_bytes) % 16 || !aligned16(a->a) || !aligned16(a->b))
    return fail(B200K_UNSUPPORTED,
                "operand rows must start on 16-byte boundaries (lda %lld, ldb %lld, %d-byte elements)",
                (long long)a->lda, (long long)a->ldb, elem_bytes);
  if (a->batch > 1 && ((a->stride_a * elem_bytes) % 16 || (a->stride_b * elem_bytes) % 16))
    return fail(B200K_UNSUPPORTED, "batch strides must be multiples of 16 bytes");
  if (a->m > INT32_MAX || a->n > INT32_MAX || a->k > INT32_MAX)
    return fail(B200K_UNSUPPORTED, "dimension exceeds 2^31 - 1");

  constexpr int BN = 256;
  const int bk = 128 / elem_bytes;
  GemmParams p = {};
  p.c = a->c;
  p.m = static_cast<int>(a->m);
  p.n = static_cast<int>(a->n);
  p.k = static_cast<int>(a->k);
  p.batch = static_cast<int>(a->batch);
  p.ldc = a->ldc;
  p.stride_c = a->stride_c;
  p.tiles_m = static_cast<int>(ceil_div(a->m, kBM));
  p.tiles_n = static_cast<int>(ceil_div(a->n, BN));
  p.k_iters = static_cast<int>(ceil_div(a->k, bk));
  {
    int rem = static_cast<int>(a->k - static_cast<int64_t>(p.k_iters - 1) * bk);
    p.k_tail_mmas = static_cast<int>(ceil_div(rem, bk / 4));
  }
  p.idesc = make_idesc(fmt, fmt, false, b_mn, kBM, BN);
  p.alpha = a->alpha;
  p.tile_group = a->tile_group;
  p.num_row_tiles = a->num_row_tiles;
  p.row_map = a->row_map;
  p.row_scale = a->row_scale;
  p.c_rows = a->row_map ? a->c_rows : a->m;
  p.epilogue = a->epilogue;
  p.status = device_status_word();
  const b200k_gemm_config cfg = effective_config(a->config);
  p.store_mode = cfg.epilogue_store;
  p.wait_budget_ns = cfg.wait_budget_us > 0 ? static_cast<uint64_t>(cfg.wait_budget_us) * 1000ull : 0;
  p.withhold_arrival = cfg.withhold_arrival;
  p.programmatic_launch = cfg.programmatic_launch;
  const bool grouped = a->tile_group != nullptr;
  if (grouped) p.batch = 1;

  CUtensorMap ta, tb;
  const uint64_t a_batches = grouped ? 1 : a->batch;
  const uint64_t sa = (a_batches > 1 ? a->stride_a : a->m * a->lda) * elem_bytes;
  if (!encode_tmap_3d(&ta, tdt, a->a, a->k, a->m, a_batches, a->lda * elem_bytes, sa, bk, kBM, 1,
                      CU_TENSOR_MAP_SWIZZLE_128B))
    return B200K_INVALID_ARG;
  const uint64_t b_batches = a->batch;
  if (b_mn) {
    const uint64_t sb = (b_batches > 1 ? a->stride_b : a->k * a->ldb) * elem_bytes;
    if (!encode_tmap_3d(&tb, tdt, a->b, a->n, a->k, b_batches, a->ldb * elem_bytes, sb, bk, bk, 1,
                        kind == kKindTF32 ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B))
      return B200K_INVALID_ARG;
  } else {
    const uint64_t sb = (b_batches > 1 ? a->stride_b : a->n * a->ldb) * elem_bytes;
    if (!encode_tmap_3d(&tb, tdt, a->b, a->k, a->n, b_batches, a->ldb * elem_bytes, sb, bk, 128, 1,
                        CU_TENSOR_MAP_SWIZZLE_128B))
      return B200K_INVALID_ARG;
  }

  int sms = current_sm_count();
  if (sms <= 0) return fail(B200K_CUDA_ERROR, "no current CUDA device");
  int64_t total_tiles = static_cast<int64_t>(p.tiles_m) * p.tiles_n * p.batch;
  int grid = static_cast<int>(total_tiles < sms ? total_tiles : sms);
  if (a->max_ctas > 0 && grid > a->max_ctas) grid = a->max_ctas;

  const int out = a->c_dtype;
  if (!grouped && a->epilogue == B200K_EPI_STORE && a->row_map == nullptr && a->workspace != nullptr &&
      a->skip_rows_count == 0) {
    // a caller that asks for the CTA-pair kernel gets no split (the split kernel is one-CTA)
    const SplitPlan plan = plan_split_k(a->m, a->n, a->batch, p.k_iters, sms,
                                        cfg.kernel == 2 && cfg.split_k == 0 ? 1 : cfg.split_k);
    if (plan.split > 1 && a->workspace_bytes >= plan.workspace_bytes && aligned16(a->workspace)) {
      GemmParams ps = p;
      ps.c = a->workspace;
      ps.ldc = a->n;
      ps.stride_c = a->m * a->n;
      ps.batch = p.batch * plan.split;
      ps.split_k = plan.split;
      ps.k_per_split = plan.k_per_split;
      const int64_t split_tiles = total_tiles * plan.split;
      const int sgrid = static_cast<int>(split_tiles < sms ? split_tiles : sms);
      int rc;
      if (kind == kKindF16)
        rc = b_mn ? launch<kKindF16, BN, true, kOutF32>(ta, tb, ps, sgrid, stream)
                  : launch<kKindF16, BN, false, kOutF32>(ta, tb, ps, sgrid, stream);
      else if (kind == kKindTF32)
        rc = b_mn ? launch<kKindTF32, BN, true, kOutF32>(ta, tb, ps, sgrid, stream)
                  : launch<kKindTF32, BN, false, kOutF32>(ta, tb, ps, sgrid, stream);
      else
        rc = b_mn ? launch<kKindF8, BN, true, kOutF32>(ta, tb, ps, sgrid, stream)
                  : launch<kKindF8, BN, false, kOutF32>(ta, tb, ps, sgrid, stream);
      if (rc != B200K_OK) return rc;
      return launch_splitk_reduce(out, static_cast<const float*>(a->workspace), plan.split, a->m, a->n,
                                  a->batch, a->c, a->ldc, a->stride_c, stream);
    }
  }
  const bool pair_plain = !grouped && a->epilogue == B200K_EPI_STORE && a->row_map == nullptr;
  const bool pair_grouped = grouped && a->tile_rows == 256 && !b_mn;
  if (int rc = set_c_peers(&p, a->c_peers, a->num_c_peers, a->c_peer_rows, pair_grouped, a->row_map, out))
    return rc;
  // N-contiguous B on the pair kernel: plain problems
  const bool pair_b_ok = !b_mn || pair_plain;
  // (a grouped problem over 256-row tiles exists on the pair kernel only: a request for the
  // one-CTA kernel is not honoured there)
  if (pair_b_ok && ((pair_plain && cfg.kernel != 1) || pair_grouped)) {
    GemmParams pp = p;
    // Tile width: 256 x 256.  256 x 128 tiles (config tile_n = 128) halve the cost of a
    // partly filled last wave on paper (4096 cubed: 256 tiles on 74 clusters are 4 rounds,
    // 512 narrow tiles 7 half rounds), but a narrow tile re-reads A twice as often and
    // pays the per-tile hand-offs twice: measured 113 against 96 us there.
    // (an N-contiguous B is loaded in boxes of 128 bytes of N: each CTA's half of a narrow
    // tile, 64 columns, is less than one box of 8-bit operands)
    // Left to the library, narrow tiles are taken when the wide ones would leave more than
    // half of the CTA pairs without work (1024 cubed, 16-bit: 16.4 -> 14.1 us).
    int want_bn = cfg.tile_n;
    if (want_bn == 0) {
      const int64_t wide_tiles = ceil_div(a->m, 256) * ceil_div(a->n, 256) * a->batch;
      want_bn = wide_tiles * 2 <= sms / 2 ? 128 : 256;
    }
    const int bn = (want_bn == 128 && pair_plain && !(b_mn && elem_bytes == 1)) ? 128 : 256;
    pp.pair_bn = bn;
    pp.b_mn = b_mn ? 1 : 0;
    if (int rc = set_skip_rows(&pp, a->skip_rows_begin, a->skip_rows_count, a->m, pair_plain && a->batch == 1))
      return rc;
    pp.group_m = grouped ? kGroupM : pick_group_m(a->m, a->lda * elem_bytes, cfg.group_m);
    pp.tiles_n = static_cast<int>(ceil_div(a->n, bn));
    pp.idesc = make_idesc(fmt, fmt, false, b_mn, 256, bn);
    CUtensorMap tbp = tb;
    if (!b_mn && bn == 128) {
      const uint64_t sb = (b_batches > 1 ? a->stride_b : a->n * a->ldb) * elem_bytes;
      if (!encode_tmap_3d(&tbp, tdt, a->b, a->k, a->n, b_batches, a->ldb * elem_bytes, sb, bk, 64, 1,
                          CU_TENSOR_MAP_SWIZZLE_128B))
        return B200K_INVALID_ARG;
    }
    const CUtensorMap maps[4] = {ta, tbp, ta, ta};
    return launch_gemm_pair(kind, out, maps, pp, sms, stream);
  }
  if (int rc = set_skip_rows(&p, a->skip_rows_begin, a->skip_rows_count, a->m, false)) return rc;
  if (grouped && a->tile_rows != 0 && a->tile_rows != 128)
    return fail(B200K_UNSUPPORTED, "tile_rows %d: 256-row tiles need B stored (N, K) and the CTA-pair "
                "kernels, otherwise tile_group entries are per 128 rows", a->tile_rows);
  if (kind == kKindF16)
    return b_mn ? launch_out<kKindF16, BN, true>(out, ta, tb, p, grid, stream)
                : launch_out<kKindF16, BN, false>(out, ta, tb, p, grid, stream);
  if (kind == kKindTF32)
    return b_mn ? launch_out<kKindTF32, BN, true>(out, ta, tb, p, grid, stream)
                : launch_out<kKindTF32, BN, false>(out, ta, tb, p, grid, stream);
  return b_mn ? launch_out<kKindF8, BN, true>(out, ta, tb, p, grid, stream)
              : launch_out<kKindF8, BN, false>(out, ta, tb, p, grid, stream);
}

extern "C" int b200k_block_scaled_gemm(const b200k_block_scaled_gemm_args* a,
                                       b200k_stream stream_) {
  if (a == nullptr) return fail(B200K_INVALID_ARG, "null args");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (a->m < 0 || a->n < 0 || a->k < 0 || a->batch < 0)
    return fail(B200K_INVALID_ARG, "negative dimension");
  if (a->m == 0 || a->n == 0 || a->batch == 0) return B200K_OK;
  if (!a->a || !a->b || (!a->c && !a->c_peers) || !a->sfa || !a->sfb)
    return fail(B200K_INVALID_ARG, "null operand pointer");
  if (a->k == 0) return fail(B200K_UNSUPPORTED, "K == 0 is not supported");

  const bool fp4 = a->ab_dtype == B200K_E2M1X2;
  if (!fp4 && a->ab_dtype != B200K_E4M3 && a->ab_dtype != B200K_E5M2)
    return fail(B200K_INVALID_ARG, "block-scaled operands must be e4m3, e5m2 or e2m1x2 (got %d)",
                a->ab_dtype);
  const int sf_block = fp4 ? 16 : 32;
  const int bk = fp4 ? 256 : 128;              // K elements per stage
  const int64_t kbytes = fp4 ? a->k / 2 : a->k;
  if (fp4 && (a->k % 2)) return fail(B200K_UNSUPPORTED, "fp4 K must be even");
  const int64_t lda_b = fp4 ? a->lda / 2 : a->lda;
  const int64_t ldb_b = fp4 ? a->ldb / 2 : a->ldb;
  if (lda_b % 16 || ldb_b % 16 || !aligned16(a->a) || !aligned16(a->b) || !aligned16(a->sfa) ||
      !aligned16(a->sfb))
    return fail(B200K_UNSUPPORTED, "operand rows and scale tensors must start on 16-byte boundaries");
  if (a->sf_k_atoms < ceil_div(a->k, 4 * sf_block))
    return fail(B200K_INVALID_ARG, "sf_k_atoms %lld too small for K %lld", (long long)a->sf_k_atoms,
                (long long)a->k);
  if (a->epilogue == B200K_EPI_SWIGLU && a->n % 256 != 0)
    return fail(B200K_UNSUPPORTED, "SwiGLU epilogue needs N a multiple of 256");
  if (a->m > INT32_MAX || a->n > INT32_MAX || a->k > INT32_MAX)
    return fail(B200K_UNSUPPORTED, "dimension exceeds 2^31 - 1");

  constexpr int BN = 256;
  GemmParams p = {};
  p.c = a->c;
  p.m = static_cast<int>(a->m);
  p.n = static_cast<int>(a->n);
  p.k = static_cast<int>(a->k);
  p.batch = static_cast<int>(a->batch);
  p.ldc = a->ldc;
  p.stride_c = a->stride_c;
  p.tiles_m = static_cast<int>(ceil_div(a->m, kBM));
  p.tiles_n = static_cast<int>(ceil_div(a->n, BN));
  p.k_iters = static_cast<int>(ceil_div(a->k, bk));
  {
    int rem = static_cast<int>(a->k - static_cast<int64_t>(p.k_iters - 1) * bk);
    p.k_tail_mmas = static_cast<int>(ceil_div(rem, bk / 4));
  }
  const uint32_t fmt = fp4 ? kFmtE2M1_MXF4 : (a->ab_dtype == B200K_E4M3 ? kFmtE4M3 : kFmtE5M2);
  p.idesc = make_idesc_block_scaled(fmt, fmt, kBM, BN, /*ue8m0=*/!fp4, 0, 0);
  p.alpha = a->alpha;
  p.alpha_a = a->alpha_a;
  p.alpha_b = a->alpha_b;
  p.sfa = static_cast<const uint8_t*>(a->sfa);
  p.sfb = static_cast<const uint8_t*>(a->sfb);
  p.sf_k_atoms = static_cast<int>(a->sf_k_atoms);
  p.sfb_row_tiles = static_cast<int>(ceil_div(a->n, 128));
  p.stride_sfa = a->stride_sfa;
  p.stride_sfb = a->stride_sfb;
  p.tile_group = a->tile_group;
  p.num_row_tiles = a->num_row_tiles;
  p.row_map = a->row_map;
  p.row_scale = a->row_scale;
  p.c_rows = a->row_map ? a->c_rows : a->m;
  p.epilogue = a->epilogue;
  p.status = device_status_word();
  const b200k_gemm_config cfg = effective_config(a->config);
  p.store_mode = cfg.epilogue_store;
  p.wait_budget_ns = cfg.wait_budget_us > 0 ? static_cast<uint64_t>(cfg.wait_budget_us) * 1000ull : 0;
  p.withhold_arrival = cfg.withhold_arrival;
  p.programmatic_launch = cfg.programmatic_launch;
  const bool grouped = a->tile_group != nullptr;
  if (grouped) p.batch = 1;
  const bool mx_out = a->c_dtype == B200K_E4M3;
  if (mx_out) {
    const int64_t n_out = a->epilogue == B200K_EPI_SWIGLU ? a->n / 2 : a->n;
    if (fp4 || a->c_sf == nullptr || a->row_map != nullptr || n_out % 32 != 0 ||
        a->c_sf_k_atoms < ceil_div(n_out, 128))
      return fail(B200K_UNSUPPORTED, "quantised (e4m3 + ue8m0) output needs MXFP8 operands, c_sf with "
                  "c_sf_k_atoms >= ceil(N_out / 128), N_out a multiple of 32 and no row_map");
    p.c_sf = static_cast<uint8_t*>(a->c_sf);
    p.c_sf_k_atoms = static_cast<int>(a->c_sf_k_atoms);
  }
  const bool nv_out = a->c_dtype == B200K_E2M1X2;
  if (nv_out) {
    const int64_t n_out = a->epilogue == B200K_EPI_SWIGLU ? a->n / 2 : a->n;
    if (a->c_sf == nullptr || a->c_scale == nullptr || a->row_map != nullptr || n_out % 32 != 0 ||
        a->ldc % 2 != 0 || a->stride_c % 2 != 0 || a->c_sf_k_atoms < ceil_div(n_out, 64))
      return fail(B200K_UNSUPPORTED, "NVFP4 (e2m1 + ue4m3) output needs c_sf with c_sf_k_atoms >= "
                  "ceil(N_out / 64), c_scale, N_out a multiple of 32, an even ldc and no row_map");
    p.c_sf = static_cast<uint8_t*>(a->c_sf);
    p.c_sf_k_atoms = static_cast<int>(a->c_sf_k_atoms);
    p.c_scale = a->c_scale;
  }

  CUtensorMap ta, tb;
  const uint64_t a_batches = grouped ? 1 : a->batch;
  const uint64_t sa = a_batches > 1 ? (fp4 ? a->stride_a / 2 : a->stride_a) : a->m * lda_b;
  const uint64_t sb = a->batch > 1 ? (fp4 ? a->stride_b / 2 : a->stride_b) : a->n * ldb_b;
  if (!encode_tmap_3d(&ta, CU_TENSOR_MAP_DATA_TYPE_UINT8, a->a, kbytes, a->m, a_batches, lda_b, sa,
                      128, kBM, 1, CU_TENSOR_MAP_SWIZZLE_128B))
    return B200K_INVALID_ARG;
  if (!encode_tmap_3d(&tb, CU_TENSOR_MAP_DATA_TYPE_UINT8, a->b, kbytes, a->n, a->batch, ldb_b, sb,
                      128, 128, 1, CU_TENSOR_MAP_SWIZZLE_128B))
    return B200K_INVALID_ARG;

  int sms = current_sm_count();
  if (sms <= 0) return fail(B200K_CUDA_ERROR, "no current CUDA device");
  int64_t total_tiles = static_cast<int64_t>(p.tiles_m) * p.tiles_n * p.batch;
  int grid = static_cast<int>(total_tiles < sms ? total_tiles : sms);
  if (a->max_ctas > 0 && grid > a->max_ctas) grid = a->max_ctas;

  const bool pair_plain = !grouped && a->batch == 1 && a->epilogue == B200K_EPI_STORE && a->row_map == nullptr;
  // grouped: scale tensors of B packed per expert in whole row tiles; SwiGLU only where one
  // chunk of accumulator columns is shared between the windows (MXFP8)
  const bool swiglu = a->epilogue == B200K_EPI_SWIGLU;
  const int64_t sfb_tile_bytes = a->sf_k_atoms * 512;
  const bool pair_grouped = grouped && a->tile_rows == 256 && !(swiglu && fp4) &&
                            a->stride_sfb % sfb_tile_bytes == 0;
  if (int rc = set_c_peers(&p, a->c_peers, a->num_c_peers, a->c_peer_rows, pair_grouped, a->row_map, a->c_dtype))
    return rc;
  // (256-row grouped tiles and quantised outputs exist on the pair kernel only: a request for
  // the one-CTA kernel is not honoured there)
  if ((pair_plain && (cfg.kernel != 1 || mx_out || nv_out)) || pair_grouped) {
    GemmParams pp = p;
    pp.idesc = make_idesc_block_scaled(fmt, fmt, 256, BN, /*ue8m0=*/!fp4, 0, 0);
    pp.sfb_group_tiles = grouped ? static_cast<int>(a->stride_sfb / sfb_tile_bytes) : 0;
    if (int rc = set_skip_rows(&pp, a->skip_rows_begin, a->skip_rows_count, a->m, pair_plain)) return rc;
    pp.group_m = grouped ? kGroupM : pick_group_m(a->m, lda_b + a->sf_k_atoms * 4, cfg.group_m);
    CUtensorMap tsa, tsb;
    const uint32_t atoms = fp4 ? 4 : 1;
    const uint64_t ka = static_cast<uint64_t>(a->sf_k_atoms);
    const uint64_t sfb_tiles = grouped ? static_cast<uint64_t>(pp.sfb_group_tiles) * a->batch
                                       : static_cast<uint64_t>(ceil_div(a->n, 128));
    // one 512-byte atom per innermost row (128 32-bit words), so every request of the copy
    // engine is a whole run of cache lines rather than a 16-byte row of the atom
    if (!encode_tmap_3d(&tsa, CU_TENSOR_MAP_DATA_TYPE_UINT32, a->sfa, 128, ka, ceil_div(a->m, 128), 512,
                        ka * 512, 128, atoms, 1, CU_TENSOR_MAP_SWIZZLE_NONE))
      return B200K_INVALID_ARG;
    if (!encode_tmap_3d(&tsb, CU_TENSOR_MAP_DATA_TYPE_UINT32, a->sfb, 128, ka, sfb_tiles, 512,
                        ka * 512, 128, atoms, swiglu ? 1 : 2, CU_TENSOR_MAP_SWIZZLE_NONE))
      return B200K_INVALID_ARG;
    const CUtensorMap maps[4] = {ta, tb, tsa, tsb};
    return launch_gemm_pair(fp4 ? kKindNVF4 : kKindMXF8, a->c_dtype, maps, pp, sms, stream);
  }
  if (int rc = set_skip_rows(&p, a->skip_rows_begin, a->skip_rows_count, a->m, false)) return rc;
  if (mx_out || nv_out)
    return fail(B200K_UNSUPPORTED, "quantised output is produced by the CTA-pair kernel only (plain "
                "problems, or grouped ones with tile_rows = 256)");
  if (grouped && a->tile_rows != 0 && a->tile_rows != 128)
    return fail(B200K_UNSUPPORTED, "tile_rows %d is not available for this grouped problem: "
                "tile_group entries are per 128 rows on the one-CTA kernel", a->tile_rows);
  if (fp4) return launch_out<kKindNVF4, BN, false>(a->c_dtype, ta, tb, p, grid, stream);
  return launch_out<kKindMXF8, BN, false>(a->c_dtype, ta, tb, p, grid, stream);
}

extern "C" int64_t b200k_gemm_workspace_bytes(const b200k_gemm_args* a) {
  if (a == nullptr || a->m <= 0 || a->n <= 0 || a->k <= 0 || a->batch <= 0) return 0;
  if (a->tile_group != nullptr || a->epilogue != B200K_EPI_STORE || a->row_map != nullptr) return 0;
  int elem_bytes;
  switch (a->ab_dtype) {
    case B200K_F16: case B200K_BF16: elem_bytes = 2; break;
    case B200K_F32: elem_bytes = 4; break;
    case B200K_E4M3: case B200K_E5M2: elem_bytes = 1; break;
    default: return 0;
  }
  const int sms = current_sm_count();
  if (sms <= 0) return 0;
  const int k_iters = static_cast<int>(ceil_div(a->k, 128 / elem_bytes));
  const b200k_gemm_config cfg = effective_config(a->config);
  return plan_split_k(a->m, a->n, a->batch, k_iters, sms,
                      cfg.kernel == 2 && cfg.split_k == 0 ? 1 : cfg.split_k).workspace_bytes;
}
