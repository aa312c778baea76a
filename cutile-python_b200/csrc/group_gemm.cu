// Grouped GEMM over a list of independent problems in ONE persistent launch: the CTAs walk
// the output tiles of all problems, problem after problem, with a running tile offset - the
// schedule of grouped_matmul_kernel (reference: test/kernels/group_gemm.py:10-38), on the
// one-CTA tcgen05 pipeline of gemm.cu (TMA producer warp, MMA warp, four epilogue warps,
// 128 x 256 tiles, two accumulator windows in tensor memory).
//
// The problem table - per problem its two tensor maps, its sizes and its output pointer -
// travels by value in the kernel parameters (up to kMaxGroupProblems per launch), so nothing
// is staged in device memory, nothing is allocated and the launch can be captured in a CUDA
// graph.  All problems of a launch share operand type, output type and the layout of B.
#include <stdlib.h>

#include "gemm_common.cuh"

namespace b200k {

constexpr int kMaxGroupProblems = 48;

struct GroupProblem {
  void* c;
  int64_t ldc;          // elements
  int m, n;
  int k_iters, k_tail_mmas;
  int tiles_n;
  int tile_end;         // tiles of this and all earlier problems
};

struct GroupMaps {
  CUtensorMap a[kMaxGroupProblems];
  CUtensorMap b[kMaxGroupProblems];
};

struct GroupTable {
  int count;
  uint32_t idesc;
  int* status;
  GroupProblem prob[kMaxGroupProblems];
};

template <int KIND, bool B_MN, int OUT>
__global__ void __launch_bounds__(kNumThreads, 1)
group_gemm_kernel(const __grid_constant__ GroupMaps maps, const __grid_constant__ GroupTable t) {
  constexpr int BN = 256;
  using Cfg = GemmCfg<KIND, BN, B_MN>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t tiles_base = smem_base;
  uint8_t* tail = smem + kStages * Cfg::kStageBytes;
  const uint32_t bar_base = smem_u32(tail);
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
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const int num_tiles = t.prob[t.count - 1].tile_end;

  // tile -> (problem, row tile, column tile); `g` only moves forward as the tile index grows
  auto locate = [&](int tile, int& g, int& pid_m, int& pid_n) {
    while (tile >= t.prob[g].tile_end) ++g;
    const int local = tile - (g > 0 ? t.prob[g - 1].tile_end : 0);
    pid_m = local / t.prob[g].tiles_n;
    pid_n = local - pid_m * t.prob[g].tiles_n;
  };

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    const bool elected = elect_one();
    uint32_t it = 0;
    bool ok = true;
    int g = 0;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      int pid_m, pid_n;
      locate(tile, g, pid_m, pid_n);
      const CUtensorMap* ma = &maps.a[g];
      const CUtensorMap* mb = &maps.b[g];
      const int m0 = pid_m * kBM, n0 = pid_n * BN;
      const int k_iters = t.prob[g].k_iters;
      for (int kb = 0; kb < k_iters; ++kb, ++it) {
        const int s = it % kStages;
        const uint32_t ph = (it / kStages) & 1;
        if (!mbar_wait(empty_bar(s), ph ^ 1, abort_flag)) {
          report_status(t.status, 71, s);
          *abort_flag = 1;
          ok = false;
          break;
        }
        const uint32_t a_dst = tiles_base + s * Cfg::kStageBytes;
        const uint32_t b_dst = a_dst + Cfg::kABytes;
        const int kx = kb * Cfg::kBKElems;
        if (elected) {
          mbar_arrive_expect_tx(full_bar(s), Cfg::kStageBytes);
          tma_load_3d(a_dst, ma, full_bar(s), kx, m0, 0);
          if constexpr (B_MN) {
#pragma unroll
            for (int j = 0; j < Cfg::kBBoxes; ++j)
              tma_load_3d(b_dst + j * Cfg::kBBoxBytes, mb, full_bar(s), n0 + j * Cfg::kBBoxN, kx, 0);
          } else {
#pragma unroll
            for (int j = 0; j < Cfg::kBBoxes; ++j)
              tma_load_3d(b_dst + j * 128 * 128, mb, full_bar(s), kx, n0 + j * 128, 0);
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    const bool elected = elect_one();
    uint32_t it = 0, local_tile = 0;
    bool ok = true;
    int g = 0;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      int pid_m, pid_n;
      locate(tile, g, pid_m, pid_n);
      const int k_iters = t.prob[g].k_iters;
      const int as = local_tile & 1;
      const uint32_t aph = (local_tile >> 1) & 1;
      if (!mbar_wait(acc_empty_bar(as), aph ^ 1, abort_flag)) {
        report_status(t.status, 72, 100 + as);
        *abort_flag = 1;
        break;
      }
      tc_fence_after_sync();
      const uint32_t tmem_acc = tmem_base + as * Cfg::kAccStride;
      for (int kb = 0; kb < k_iters; ++kb, ++it) {
        const int s = it % kStages;
        const uint32_t ph = (it / kStages) & 1;
        if (!mbar_wait(full_bar(s), ph, abort_flag)) {
          report_status(t.status, 72, s);
          *abort_flag = 1;
          ok = false;
          break;
        }
        tc_fence_after_sync();
        const uint32_t a_addr = tiles_base + s * Cfg::kStageBytes;
        const uint32_t b_addr = a_addr + Cfg::kABytes;
        const uint64_t a_desc = make_smem_desc(a_addr, 16, 1024, kSwizzle128B);
        const uint64_t b_desc = B_MN ? make_smem_desc(b_addr, Cfg::kBBoxBytes, KIND == kKindTF32 ? 512 : 1024,
                                                      KIND == kKindTF32 ? kSwizzle128BBase32B : kSwizzle128B)
                                     : make_smem_desc(b_addr, 16, 1024, kSwizzle128B);
        const int n_mma = (kb == k_iters - 1) ? t.prob[g].k_tail_mmas : 4;
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
          if (kk < n_mma && elected) {
            const uint32_t acc = (kb > 0 || kk > 0) ? 1u : 0u;
            const uint64_t a_d = a_desc + static_cast<uint64_t>(kk * 2);
            const uint64_t b_d = b_desc + static_cast<uint64_t>(B_MN ? kk * (Cfg::kMmaK * 128 / 16) : kk * 2);
            umma<KIND>(tmem_acc, a_d, b_d, t.idesc, acc);
          }
        }
        if (elected) tc_commit(empty_bar(s));
      }
      if (ok && elected) tc_commit(acc_full_bar(as));
      ++local_tile;
    }
    __syncwarp();
  } else {
    // ---------------- epilogue ----------------
    const int quarter = warp & 3;
    constexpr int elem_bytes = (OUT == kOutF32) ? 4 : 2;
    uint32_t local_tile = 0;
    int g = 0;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
      int pid_m, pid_n;
      locate(tile, g, pid_m, pid_n);
      const GroupProblem& pr = t.prob[g];
      const int as = local_tile & 1;
      const uint32_t aph = (local_tile >> 1) & 1;
      if (!mbar_wait(acc_full_bar(as), aph, abort_flag)) {
        report_status(t.status, 73, as);
        *abort_flag = 1;
        break;
      }
      tc_fence_after_sync();
      const int row = pid_m * kBM + quarter * 32 + lane;
      const bool row_ok = row < pr.m;
      uint8_t* c_row = static_cast<uint8_t*>(pr.c) + static_cast<int64_t>(row) * pr.ldc * elem_bytes;
      const bool vec_ok = ((pr.ldc * elem_bytes) % 16 == 0) && (reinterpret_cast<uintptr_t>(pr.c) % 16 == 0);
      const uint32_t taddr = tmem_base + as * Cfg::kAccStride + (uint32_t(quarter * 32) << 16);
      const int n0 = pid_n * BN;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        if (n0 + c * 32 >= pr.n) break;           // warp-uniform: the rest of the tile is padding
        uint32_t r[32];
        tmem_ld_32x32b_x32(taddr + c * 32, r);
        tmem_ld_wait();
        if (row_ok) {
          float v[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
          store_row_chunk<OUT>(c_row, n0 + c * 32, pr.n, v, vec_ok);
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

namespace {

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

template <int KIND, bool B_MN, int OUT>
int launch_group(const GroupMaps& maps, const GroupTable& table, int grid, cudaStream_t stream) {
  using Cfg = GemmCfg<KIND, 256, B_MN>;
  auto kernel = group_gemm_kernel<KIND, B_MN, OUT>;
  static bool configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes);
    if (e != cudaSuccess)
      return fail(B200K_CUDA_ERROR, "cudaFuncSetAttribute(%d bytes): %s", Cfg::kSmemBytes, cudaGetErrorString(e));
    configured[dev] = true;
  }
  kernel<<<grid, kNumThreads, Cfg::kSmemBytes, stream>>>(maps, table);
  B200K_CHECK_LAUNCH("group gemm launch");
  return B200K_OK;
}

template <int KIND, bool B_MN>
int launch_group_out(int out, const GroupMaps& maps, const GroupTable& table, int grid, cudaStream_t stream) {
  switch (out) {
    case B200K_F16: return launch_group<KIND, B_MN, kOutF16>(maps, table, grid, stream);
    case B200K_BF16: return launch_group<KIND, B_MN, kOutBF16>(maps, table, grid, stream);
    case B200K_F32: return launch_group<KIND, B_MN, kOutF32>(maps, table, grid, stream);
    default: return fail(B200K_INVALID_ARG, "unsupported output dtype %d", out);
  }
}

}  // namespace
}  // namespace b200k

using namespace b200k;

extern "C" int32_t b200k_group_gemm_max_problems(void) { return kMaxGroupProblems; }

extern "C" int b200k_group_gemm(const b200k_group_gemm_args* a, b200k_stream stream_) {
  if (a == nullptr) return fail(B200K_INVALID_ARG, "null args");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (a->num_problems < 0 || a->num_problems > kMaxGroupProblems)
    return fail(B200K_INVALID_ARG, "num_problems must be in [0, %d] per call", kMaxGroupProblems);
  if (a->num_problems == 0) return B200K_OK;
  if (a->problems == nullptr) return fail(B200K_INVALID_ARG, "null problem list");
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
  const int bk = 128 / elem_bytes;
  // the tables are large (about 14 KB): built once per thread, copied into the launch
  static thread_local GroupMaps maps;
  static thread_local GroupTable table;
  table.count = 0;
  table.idesc = make_idesc(fmt, fmt, false, b_mn, kBM, 256);
  table.status = device_status_word();
  int tiles = 0;
  for (int i = 0; i < a->num_problems; ++i) {
    const b200k_group_problem& q = a->problems[i];
    if (q.m < 0 || q.n < 0 || q.k < 0) return fail(B200K_INVALID_ARG, "problem %d: negative dimension", i);
    if (q.m == 0 || q.n == 0) continue;                       // nothing to write
    if (q.k == 0) return fail(B200K_UNSUPPORTED, "problem %d: K == 0 is not supported (C would be all zeros)", i);
    if (!q.a || !q.b || !q.c) return fail(B200K_INVALID_ARG, "problem %d: null pointer", i);
    if (q.m > INT32_MAX || q.n > INT32_MAX || q.k > INT32_MAX)
      return fail(B200K_UNSUPPORTED, "problem %d: dimension exceeds 2^31 - 1", i);
    if ((q.lda * elem_bytes) % 16 || (q.ldb * elem_bytes) % 16 || !aligned16(q.a) || !aligned16(q.b))
      return fail(B200K_UNSUPPORTED, "problem %d: operand rows must start on 16-byte boundaries", i);
    const int g = table.count;
    if (!encode_tmap_3d(&maps.a[g], tdt, q.a, q.k, q.m, 1, q.lda * elem_bytes, q.m * q.lda * elem_bytes, bk,
                        kBM, 1, CU_TENSOR_MAP_SWIZZLE_128B))
      return B200K_INVALID_ARG;
    const bool ok = b_mn ? encode_tmap_3d(&maps.b[g], tdt, q.b, q.n, q.k, 1, q.ldb * elem_bytes,
                                          q.k * q.ldb * elem_bytes, bk, bk, 1,
                                          kind == kKindTF32 ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B
                                                            : CU_TENSOR_MAP_SWIZZLE_128B)
                         : encode_tmap_3d(&maps.b[g], tdt, q.b, q.k, q.n, 1, q.ldb * elem_bytes,
                                          q.n * q.ldb * elem_bytes, bk, 128, 1, CU_TENSOR_MAP_SWIZZLE_128B);
    if (!ok) return B200K_INVALID_ARG;
    GroupProblem& pr = table.prob[g];
    pr.c = q.c;
    pr.ldc = q.ldc;
    pr.m = static_cast<int>(q.m);
    pr.n = static_cast<int>(q.n);
    pr.k_iters = static_cast<int>(ceil_div(q.k, bk));
    const int rem = static_cast<int>(q.k - static_cast<int64_t>(pr.k_iters - 1) * bk);
    pr.k_tail_mmas = static_cast<int>(ceil_div(rem, bk / 4));
    pr.tiles_n = static_cast<int>(ceil_div(q.n, 256));
    const int64_t mine = ceil_div(q.m, kBM) * pr.tiles_n;
    if (tiles + mine > INT32_MAX) return fail(B200K_UNSUPPORTED, "too many output tiles");
    tiles += static_cast<int>(mine);
    pr.tile_end = tiles;
    ++table.count;
  }
  if (table.count == 0) return B200K_OK;
  const int sms = current_sm_count();
  if (sms <= 0) return fail(B200K_CUDA_ERROR, "no current CUDA device");
  const int grid = tiles < sms ? tiles : sms;
  if (kind == kKindF16)
    return b_mn ? launch_group_out<kKindF16, true>(a->c_dtype, maps, table, grid, stream)
                : launch_group_out<kKindF16, false>(a->c_dtype, maps, table, grid, stream);
  if (kind == kKindTF32)
    return b_mn ? launch_group_out<kKindTF32, true>(a->c_dtype, maps, table, grid, stream)
                : launch_group_out<kKindTF32, false>(a->c_dtype, maps, table, grid, stream);
  return b_mn ? launch_group_out<kKindF8, true>(a->c_dtype, maps, table, grid, stream)
              : launch_group_out<kKindF8, false>(a->c_dtype, maps, table, grid, stream);
}
