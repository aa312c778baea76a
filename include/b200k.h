/*
 * b200k — C ABI of the B200 (sm_100a) dense-contraction kernels.
 *
 * This is the boundary a host program binds instead of the cuTile launch path
 * `ct.launch(stream, grid, kernel, args)` (reference: cext/tile_kernel.cpp:4569-4577)
 * for the kernels the reference's samples put first.  Every entry point
 *   - takes plain pointers, sizes and enums (no torch / Python types),
 *   - enqueues its work on the caller's stream and returns without synchronising,
 *   - borrows all buffers (the caller owns inputs, outputs and workspaces and keeps
 *     them alive until the stream has passed the call; array arguments must not alias),
 *   - returns 0 or a negative b200k_status; b200k_last_error() gives the message.
 *
 * Device-side trouble (a pipeline wait that ran out of its time budget) is recorded
 * in a per-device status word that b200k_device_status() reads after the caller has
 * synchronised the stream.
 */
#ifndef B200K_H_
#define B200K_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef void* b200k_stream;  /* a cudaStream_t */

typedef enum {
  B200K_OK = 0,
  B200K_INVALID_ARG = -1,
  B200K_UNSUPPORTED = -2,
  B200K_CUDA_ERROR = -3,
  B200K_TIMEOUT = -4
} b200k_status;

typedef enum {
  B200K_F16 = 0,
  B200K_BF16 = 1,
  B200K_F32 = 2,   /* as a GEMM operand: multiplied as tf32 */
  B200K_E4M3 = 3,
  B200K_E5M2 = 4,
  B200K_E2M1X2 = 5 /* two e2m1 values per byte, low nibble = even element */
} b200k_dtype;

typedef enum {
  B200K_B_KN = 0, /* B is (K, N), N contiguous (row-major K x N) */
  B200K_B_NK = 1  /* B is stored as (N, K), K contiguous (a transposed view) */
} b200k_b_layout;

typedef enum {
  B200K_EPI_STORE = 0,  /* C = alpha * acc */
  B200K_EPI_SWIGLU = 1  /* C[:, j] = silu(acc[:, j]) * acc[:, j + N/2]; C has N/2 columns */
} b200k_epilogue;

/* ---- library ---------------------------------------------------------- */
const char* b200k_version(void);
const char* b200k_last_error(void);             /* thread-local message of the last failure */
int b200k_sm_count(void);                       /* SMs of the current device, <0 on error */
/* Reads and clears the current device's status word.  *code is 0 or B200K_TIMEOUT,
 * *info packs (role << 8 | detail << 16) of the wait that gave up. */
int b200k_device_status(int* code, int* info);
/* The one piece of state the library owns: a mutex-guarded cache of encoded TMA tensor maps
 * keyed by (base pointer, data type, dims, strides, box, swizzle), at most 8192 entries of
 * 128 bytes of host memory.  A call whose operands were seen before pays a hash lookup per
 * operand instead of a driver call; the reference keeps the same per-kernel state as hoisted
 * descriptors (cext/tile_kernel.cpp:2884-2945, 3816-3844).  This reads its counters (any
 * pointer may be NULL). */
int b200k_tensor_map_cache_stats(uint64_t* hits, uint64_t* misses, uint64_t* entries);

/* ---- kernel-form selection ------------------------------------------------
 * Which of the library's kernel forms a GEMM call uses.  Every field is 0 for "choose
 * automatically" (the library's shape heuristics); a NULL pointer to this struct means all
 * automatic.  A request the problem cannot honour (split-K for a grouped problem, a tile
 * width the kernel does not have) is ignored rather than refused, so that one search space
 * serves every shape; results are the same for every setting up to fp32 summation order.
 * This is what the reference leaves to its tile-size arguments and tuner
 * (src/cuda/tile/tune/_tune.py:132-336): the search itself is host code above this ABI. */
typedef struct {
  int32_t kernel;          /* 1 = one-CTA kernel (128-row tiles), 2 = CTA-pair kernel (256-row tiles) */
  int32_t tile_n;          /* 128 or 256 output columns per tile (CTA-pair kernel) */
  int32_t epilogue_store;  /* 1 = straight from registers, 2 = staged through shared memory */
  int32_t split_k;         /* 1 = never split K, n > 1 = split K into (up to) n slices; needs the
                            * workspace b200k_gemm_workspace_bytes reports for the same args */
  /* CTA-pair kernel: time budget in microseconds of every wait between the kernel's roles
   * (0 = the default of two seconds).  A wait that runs out makes the kernel return normally
   * with the device status word set (b200k_device_status -> B200K_TIMEOUT, info = role and
   * stage); the output of that call is then undefined, later calls are unaffected. */
  int32_t wait_budget_us;
  /* Test hook for that path, leave 0: 1 = on the CTA-pair kernel the arrival that opens a
   * tile to the second MMA issuer is never made (a flag that nothing sets), so its wait runs
   * out of the budget.  Nothing faults, traps or spins without limit. */
  int32_t withhold_arrival;
  /* CTA-pair kernel: 1 = launch with programmatic stream serialisation, so that the kernel's
   * set-up (barriers, tensor memory) overlaps the tail of the kernel before it in the stream
   * and a chain of short GEMMs on one stream leaves no launch gaps (the kernel waits for its
   * predecessor before it touches global memory).  0 = ordinary launch.  The Python wrappers
   * set it for plain dense GEMMs. */
  int32_t programmatic_launch;
  /* CTA-pair kernel, plain problems: 256-row tiles of A per band of the tile raster (the
   * reference's GROUP_SIZE_M, test/kernels/matmul.py:13-23).  0 = from the operand sizes: as
   * many as fit a quarter of the L2, at least 8. */
  int32_t group_m;
} b200k_gemm_config;

/* ---- dense GEMM -------------------------------------------------------
 * C[b] = A[b] . B[b], fp32 accumulation, result rounded to c_dtype.
 * Replaces matmul_kernel / persistent_matmul_kernel / batch_matmul_kernel
 * (reference: test/kernels/matmul.py:32-100, 142-178, 181-253) behind
 * cutile_matmul (samples/MatMul.py:179-251) and bmm (samples/BatchMatMul.py:53-92).
 * With `tile_group` set it is the grouped (MoE) GEMM of fused_moe_kernel
 * (test/kernels/fused_moe.py:14-82) over an expert-sorted, tile-padded row list. */
typedef struct {
  const void* a;      /* (batch, M, K), K contiguous */
  const void* b;      /* per b_layout */
  void* c;            /* (batch, M, N) row-major */
  int64_t m, n, k, batch;
  int64_t lda, ldb, ldc;                 /* leading dimensions in elements */
  int64_t stride_a, stride_b, stride_c;  /* batch strides in elements */
  int32_t ab_dtype;   /* B200K_F16 | BF16 | F32 | E4M3 | E5M2 */
  int32_t c_dtype;    /* B200K_F16 | BF16 | F32 */
  int32_t b_layout;   /* b200k_b_layout */
  int32_t epilogue;   /* b200k_epilogue */
  float alpha;        /* scalar applied to the accumulator */
  int32_t max_ctas;   /* 0 = one CTA per SM (persistent) */
  /* Grouped mode (all optional, NULL = off).  `tile_group[i]` is the B batch index
   * (expert) of the i-th `tile_rows`-row tile of A, or a negative value for a tile to skip;
   * `num_row_tiles` points at the device-side count of row tiles in use. */
  const int32_t* tile_group;
  const int32_t* num_row_tiles;
  /* Output row remap: row i of the product goes to row row_map[i] of C; rows whose
   * target is outside [0, c_rows) are dropped (scatter semantics).  `row_scale[r]`
   * multiplies target row r (fp32). */
  const int32_t* row_map;
  const float* row_scale;
  int64_t c_rows;
  /* Rows of A per `tile_group` entry: 128 (also when 0) or 256.  With 256 (and B stored
   * (N, K)) the grouped GEMM runs on the CTA-pair kernel; `num_row_tiles` then counts
   * 256-row tiles. */
  int32_t tile_rows;
  /* Optional scratch for split-K (see b200k_gemm_workspace_bytes): 16-byte aligned device
   * memory, contents irrelevant before and after the call.  NULL = never split. */
  void* workspace;
  int64_t workspace_bytes;
  const b200k_gemm_config* config;  /* host pointer, read during the call; NULL = automatic */
  /* Output rows scattered over several buffers (grouped problems on the CTA-pair kernel, i.e.
   * tile_rows = 256, with row_map): `c_peers` is a host array of `num_c_peers` (<= 16) device
   * pointers this process can store through - its own buffers or peer-mapped ones - each of
   * `c_peer_rows` rows with leading dimension ldc.  row_map[i] = g then sends product row i to
   * row g % c_peer_rows of c_peers[g / c_peer_rows] (dropped when g is outside
   * [0, num_c_peers * c_peer_rows)), and row_scale is indexed by i.  This is the combine step
   * of the expert-parallel MoE fused into the down projection: results leave the epilogue
   * over NVLink to the rank their token came from.  `c` is ignored then.  NULL = off. */
  const void* const* c_peers;
  int32_t num_c_peers;
  int64_t c_peer_rows;
  /* Rows [skip_rows_begin, skip_rows_begin + skip_rows_count) of A take no part in the product
   * and the same rows of C are not written (plain problems on the CTA-pair kernel, batch 1;
   * both multiples of 256).  The AllGather GEMM multiplies the rows a rank owns out of its own
   * buffer while the others arrive, then every other row in ONE launch over the gathered A
   * (samples/AllGatherMatmul.py:28-120 computes all rows in one kernel).  0 = none. */
  int64_t skip_rows_begin;
  int64_t skip_rows_count;
} b200k_gemm_args;

int b200k_gemm(const b200k_gemm_args* args, b200k_stream stream);

/* Bytes of `workspace` with which b200k_gemm would split K for this problem on the current
 * device, 0 when it would not (enough output tiles to fill the GPU, grouped mode, ...).
 * Split-K is the reference's matmul_split_k_kernel (test/kernels/matmul.py:103-139): a few
 * output tiles with a long K are spread over many CTAs, fp32 partial tiles are summed by a
 * second kernel. */
int64_t b200k_gemm_workspace_bytes(const b200k_gemm_args* args);

/* ---- grouped GEMM over a list of problems --------------------------------
 * C_i = A_i . B_i for i < num_problems, every problem with its own sizes, in ONE persistent
 * launch whose CTAs walk the output tiles of all problems with a running tile offset.
 * Replaces grouped_matmul_kernel (reference: test/kernels/group_gemm.py:10-38, shapes of
 * test/test_group_gemm.py:14-33).  All problems of a call share the operand type, the output
 * type and the layout of B; at most b200k_group_gemm_max_problems() problems per call (the
 * table travels in the kernel parameters: nothing is staged or allocated, and the call can be
 * captured in a CUDA graph, which the reference's list arguments cannot).  Problems with
 * m == 0 or n == 0 are skipped. */
typedef struct {
  const void* a;      /* (m, k), k contiguous, leading dimension lda */
  const void* b;      /* per b_layout, leading dimension ldb */
  void* c;            /* (m, n) row-major, leading dimension ldc */
  int64_t m, n, k;
  int64_t lda, ldb, ldc;   /* in elements */
} b200k_group_problem;

typedef struct {
  const b200k_group_problem* problems;   /* host array, read during the call */
  int32_t num_problems;
  int32_t ab_dtype;   /* B200K_F16 | BF16 | F32 | E4M3 | E5M2 */
  int32_t c_dtype;    /* B200K_F16 | BF16 | F32 */
  int32_t b_layout;   /* b200k_b_layout */
} b200k_group_gemm_args;

int32_t b200k_group_gemm_max_problems(void);
int b200k_group_gemm(const b200k_group_gemm_args* args, b200k_stream stream);

/* ---- block-scaled GEMM ------------------------------------------------
 * C = alpha * (A (.) sA) . (B (.) sB), fp32 accumulation.  Replaces
 * block_scaled_matmul_kernel / ct.mma_scaled (reference:
 * test/kernels/scaled_matmul.py:12-114, src/cuda/tile/_stub.py:2198-2329) behind
 * cutile_block_scaled_matmul (samples/BlockScaledMatMul.py:229-297).
 *   MXFP8 : ab_dtype E4M3|E5M2, scales ue8m0, one per 32 elements of K
 *   NVFP4 : ab_dtype E2M1X2,    scales ue4m3, one per 16 elements of K
 * Both operands are K-contiguous: A is (M, K), B is stored (N, K).
 * Scales use the swizzle_32_4_4 layout (reference: test/kernels/kernel_utils.py:83-98):
 * [rows/128][sf_k_atoms][32][16] bytes with rows padded to 128 and sf_k_atoms =
 * ceil(K / (4 * block)). */
typedef struct {
  const void* a;
  const void* b;
  const void* sfa;
  const void* sfb;
  void* c;
  int64_t m, n, k, batch;
  int64_t lda, ldb, ldc;                 /* in elements (e2m1: two per byte) */
  int64_t stride_a, stride_b, stride_c;  /* batch strides in elements */
  int64_t sf_k_atoms;                    /* atoms along K in sfa / sfb */
  int64_t stride_sfa, stride_sfb;        /* batch strides of the scale tensors in bytes */
  int32_t ab_dtype;
  int32_t c_dtype;
  int32_t epilogue;
  float alpha;
  const float* alpha_a;  /* optional device scalars multiplied into alpha */
  const float* alpha_b;
  int32_t max_ctas;
  const int32_t* tile_group;
  const int32_t* num_row_tiles;
  const int32_t* row_map;
  const float* row_scale;
  int64_t c_rows;
  int32_t tile_rows;                     /* as in b200k_gemm_args */
  /* c_dtype B200K_E4M3 (MXFP8 operands, CTA-pair kernel): the result is rounded to bf16 and
   * quantised in the epilogue exactly as b200k_mxfp8_quantize would quantise that bf16
   * tensor: e4m3 bytes to `c` (ldc in bytes), one ue8m0 scale per 32 output columns to
   * `c_sf` in the swizzle_32_4_4 layout with `c_sf_k_atoms` atoms along N.  This is the
   * quantise-in-epilogue step between chained block-scaled GEMMs (reference pattern:
   * experimental/cuda-lang/tutorial/nvfp4_gemm_2_quantize_fp4.py:136-192). */
  void* c_sf;
  int64_t c_sf_k_atoms;
  const b200k_gemm_config* config;  /* as in b200k_gemm_args (split_k is not used here) */
  /* c_dtype B200K_E2M1X2 (MXFP8 or NVFP4 operands, CTA-pair kernel): the result is rounded to
   * bf16 and quantised to NVFP4 in the epilogue with the per-tensor scale the caller gives in
   * `c_scale` (device scalar; e.g. calibrated, or from a b200k_nvfp4_quantize of an earlier
   * result): packed e2m1 bytes to `c` (ldc in elements, even), one ue4m3 scale per 16 output
   * columns to `c_sf` (swizzle_32_4_4, `c_sf_k_atoms` >= ceil(N_out / 64) atoms along N), by
   * the block rule of b200k_nvfp4_quantize with s_t = *c_scale.  Same reference pattern as
   * above (nvfp4_gemm_2_quantize_fp4.py:136-192,976-991 quantises to fp4 with a given global
   * scale). */
  const float* c_scale;
  /* as in b200k_gemm_args */
  const void* const* c_peers;
  int32_t num_c_peers;
  int64_t c_peer_rows;
  /* as in b200k_gemm_args */
  int64_t skip_rows_begin;
  int64_t skip_rows_count;
} b200k_block_scaled_gemm_args;

int b200k_block_scaled_gemm(const b200k_block_scaled_gemm_args* args, b200k_stream stream);

/* ---- block quantisers --------------------------------------------------
 * x is (rows, K) with row stride ldx (elements); q is (rows, K) with row stride ldq
 * (bytes).  Scales are written to `sf_logical` ((rows, ceil(K/block)) bytes, dense)
 * and/or to `sf_swizzled` (swizzle_32_4_4 atoms, [ceil(rows/128)][sf_k_atoms][32][16]);
 * either may be NULL.  Padding bytes of the swizzled tensor are left untouched. */
typedef struct {
  const void* x;
  void* q;
  void* sf_logical;
  void* sf_swizzled;
  float* tensor_scale;   /* nvfp4 only: receives the fp32 per-tensor scale (device) */
  void* scratch;         /* nvfp4 only: at least 4 bytes of device memory, 4-byte aligned */
  int64_t rows, k;
  int64_t ldx, ldq;
  int64_t sf_k_atoms;
  int32_t x_dtype;       /* B200K_F32 | BF16 | F16 */
  int32_t q_dtype;       /* mxfp8: B200K_E4M3 | E5M2 */
  /* mxfp8 only, optional row gather (MoE permute fused into the quantiser): output row i
   * is quantised from x row gather_index[i] / gather_divisor; an index outside
   * [0, src_rows * gather_divisor) gives an all-zero row.  `live_blocks` (device) limits the
   * work to the first *live_blocks * tile_m output rows. */
  const int32_t* gather_index;
  int32_t gather_divisor;
  int32_t tile_m;
  int64_t src_rows;
  const int32_t* live_blocks;
  /* nvfp4 only: non-zero = `tensor_scale` is an input (a calibrated scale, or the one an
   * earlier call produced): the pass that finds the tensor maximum is skipped, `scratch` may
   * be NULL, x is read once.  Values beyond 6 * 448 * scale saturate. */
  int32_t tensor_scale_given;
} b200k_quantize_args;

/* MXFP8: replaces block_quantize(x, 32) (reference: test/kernels/kernel_utils.py:38-80)
 * evaluated in fp32: scale = 2^ceil(log2(max(amax/448, 1e-12))), q = rn_e4m3(x/scale),
 * scale byte = exponent + 127 (ue8m0). */
int b200k_mxfp8_quantize(const b200k_quantize_args* args, b200k_stream stream);

/* NVFP4 (no counterpart in the reference, which only consumes such operands through
 * ct.mma_scaled, test/test_mma_scaled.py:149-183).  Rule, all in fp32 with IEEE
 * round-to-nearest operations:
 *   s_t   = amax(x) / 2688                      (448 * 6)
 *   s_blk = rn_e4m3(amax_blk / (6 * s_t))       one per 16 elements, 0 for a zero block
 *   q     = rn_e2m1(x * rn(1 / d)), d = f32(s_blk) * s_t   ties to even, saturating at +-6
 *           (product and reciprocal each rounded to fp32; x / d when d is subnormal)
 * x ~= q * s_blk * s_t.  Byte i of a row holds elements 2i (low nibble) and 2i+1. */
int b200k_nvfp4_quantize(const b200k_quantize_args* args, b200k_stream stream);

/* Same result as b200k_nvfp4_quantize, for callers that cannot allocate device memory
 * (it has no counterpart in the reference).  Some hosts of this library may not call
 * cudaMalloc where they call us: a plugin running inside another framework's stream
 * callback or memory-pool-owned region, a process whose device memory is fully
 * pre-partitioned, code between the nodes of a captured launch sequence.  This entry
 * point allocates nothing and ignores `scratch`: its temporary (one partial maximum per
 * 65536 elements) lives in a 64 KB array inside the library image, which every GPU that
 * loads the library keeps until the process exits.
 *   - Limit: rows * K <= 16384 * 65536 (2^30) elements; larger tensors are rejected with
 *     B200K_UNSUPPORTED and a message naming the limit.
 *   - The first call on each device looks up the array's device address (a host-side
 *     runtime query, no allocation); make that first call outside any stream capture.
 *   - All calls on a device share the array.  Each call overwrites the slots it later
 *     reads, so nothing needs clearing, but two calls that overlap on the GPU (different
 *     streams) race on it: serialise them.
 *   - With `tensor_scale_given` the caller's scale is used as in b200k_nvfp4_quantize (it is
 *     read, never written): no maximum is searched, the built-in array is not touched, and
 *     neither the size limit nor the overlap rule applies. */
int b200k_nvfp4_quantize_noalloc(const b200k_quantize_args* args, b200k_stream stream);

/* Logical (rows, kblocks) scale bytes (row stride ld) -> swizzle_32_4_4 atoms; replaces
 * swizzle_32_4_4 (reference: test/kernels/kernel_utils.py:83-98).  Rows beyond `rows`
 * and blocks beyond `kblocks` inside the padded atoms are set to `fill`.  `live_tiles`
 * (optional device scalar): only the first *live_tiles * live_tile_rows rows are converted,
 * the rest of `out` is left as it is (worst-case-sized buffers whose live row count is only
 * known on the device). */
int b200k_sf_swizzle(const void* sf, int64_t rows, int64_t kblocks, int64_t ld, void* out,
                     int64_t k_atoms, int32_t fill, const int32_t* live_tiles, int32_t live_tile_rows,
                     b200k_stream stream);

/* ---- mixture-of-experts plumbing ---------------------------------------
 * b200k_moe_align replaces moe_align_tile_size_torch (reference:
 * test/kernels/fused_moe.py:113-173): token replicas (token * topk + slot) are sorted by
 * expert (stable), every expert's run is padded to a multiple of tile_m with the sentinel
 * num_replicas, and each tile_m block gets its expert id.  Unlike the reference it runs
 * entirely on the device: outputs are worst-case sized (capacity >= num_replicas +
 * num_experts * (tile_m - 1), rounded up to tile_m; block_capacity = capacity / tile_m),
 * *num_blocks receives the number of blocks in use, slots beyond them hold the sentinel and
 * block ids beyond them hold -1.  The first *num_blocks * tile_m ids and *num_blocks block
 * ids equal the reference's outputs. */
typedef struct {
  const void* topk_ids;        /* (num_replicas) int32 or int64 expert ids */
  int32_t* sorted_token_ids;   /* [capacity] */
  int32_t* sorted_expert_ids;  /* [block_capacity]; NULL when only the sorted order is wanted */
  int32_t* num_blocks;         /* device scalar */
  void* workspace;             /* b200k_moe_align_workspace_bytes() bytes of device memory */
  int64_t workspace_bytes;
  int64_t num_replicas;
  int64_t capacity, block_capacity;
  int32_t num_experts;
  int32_t tile_m;
  int32_t ids_are_int64;
} b200k_moe_align_args;

int64_t b200k_moe_align_workspace_bytes(int64_t num_replicas, int32_t num_experts);
int b200k_moe_align(const b200k_moe_align_args* args, b200k_stream stream);

/* dst row i = src row index[i] / divisor (zero row when the index is out of range): the
 * row gather of fused_moe_kernel (reference: test/kernels/fused_moe.py:56-68).  With
 * `num_blocks` only the first *num_blocks * tile_m rows are produced. */
int b200k_gather_rows(const void* src, int64_t src_rows, int64_t row_bytes,
                      int64_t src_stride_bytes, const int32_t* index, int32_t divisor,
                      const int32_t* num_blocks, int32_t tile_m, int64_t max_rows, void* dst,
                      int64_t dst_stride_bytes, b200k_stream stream);

/* The same destination as b200k_gather_rows, produced source row by source row: every source row
 * is read once and stored to each position index sends it to, instead of being read once per
 * destination row (with top-k replicas the sources do not stay in the L2 under the streaming
 * stores).  Needs the valid entries of `index` to be distinct values in [0, src_rows * divisor),
 * as b200k_moe_align produces them, and `scratch`: src_rows * divisor int32 of device memory,
 * contents irrelevant before and after. */
int b200k_gather_rows_by_source(const void* src, int64_t src_rows, int64_t row_bytes,
                                int64_t src_stride_bytes, const int32_t* index, int32_t divisor,
                                const int32_t* num_blocks, int32_t tile_m, int64_t max_rows, void* dst,
                                int64_t dst_stride_bytes, int32_t* scratch, b200k_stream stream);

/* C[r, j] = silu(AB[r, j]) * AB[r, j + n], f16/bf16/f32; replaces silu_and_mul_kernel
 * (reference: test/kernels/fused_moe.py:85-108). */
int b200k_silu_and_mul(const void* ab, int64_t rows, int64_t n, int64_t ld_ab, void* c,
                       int64_t ld_c, int32_t dtype, b200k_stream stream);

/* out[t, :] = sum over slot of x[row(t, slot), :] with fp32 accumulation, where
 * row(t, slot) = index[t * topk + slot], or t * topk + slot when index is NULL; replaces
 * torch.sum(intermediate_cache3, dim=1) (reference: samples/MoE.py:288).  With `expert_ids`
 * (the routing ids, (tokens, topk) int32 or int64) an entry whose id lies outside
 * [0, num_experts) contributes nothing: b200k_moe_align drops such entries (and records it in
 * the device status word), so their rows of x were never written. */
int b200k_topk_sum(const void* x, const int32_t* index, int64_t tokens, int32_t topk,
                   int64_t hidden, void* out, int32_t dtype, const void* expert_ids,
                   int32_t ids_are_int64, int32_t num_experts, b200k_stream stream);

/* The MoE FFN for sparse routing - about one token per expert, the reference's second bench
 * shape (test/bench_moe.py:16-19: 256 tokens x 1408 experts x top-6) - without the grouped
 * GEMM: every token replica r = token * topk + slot streams the weights of its expert
 * e = topk_ids[r] once,
 *   act[r, i]         = silu(w1[e][i, :] . x[token]) * (w1[e][I + i, :] . x[token])
 *   per_replica[r, h] = topk_weights[r] * (w2[e][h, :] . act[r, :])
 * (fp32 accumulation, both results rounded to `dtype`), which replaces the gather, the two
 * fused_moe_kernel launches and silu_and_mul_kernel of cutile_moe (samples/MoE.py:197-288)
 * where their 128-row tiles would hold one real row each; b200k_topk_sum follows.  Replicas
 * routed outside [0, num_experts) give zero rows.  At most 65535 replicas, hidden and
 * intermediate at most 12288 and multiples of 16 bytes. */
typedef struct {
  const void* hidden_states;   /* (tokens, hidden), row stride hidden_stride (elements) */
  const void* w1;              /* (experts, 2 * intermediate, hidden): w1_stride_e, w1_ld (elements) */
  const void* w2;              /* (experts, hidden, intermediate): w2_stride_e, w2_ld (elements) */
  const void* topk_ids;        /* (tokens, topk) int32 or int64 */
  const float* topk_weights;   /* (tokens, topk) fp32, NULL = 1 */
  void* act;                   /* scratch: (tokens * topk, intermediate), dense */
  void* per_replica;           /* (tokens * topk, hidden), dense */
  int64_t tokens, hidden, intermediate;
  int64_t hidden_stride, w1_stride_e, w1_ld, w2_stride_e, w2_ld;
  int32_t topk, num_experts, ids_are_int64;
  int32_t dtype;               /* B200K_F16 | BF16 | F32, of activations and weights */
} b200k_moe_sparse_args;
int b200k_moe_sparse(const b200k_moe_sparse_args* args, b200k_stream stream);

/* ---- peer-memory gather (AllGather GEMM) -------------------------------
 * dst rows [p * rows, (p + 1) * rows) = shard p, read through `shards[p]`, a pointer this
 * process can dereference (its own buffer for p == rank, peer-mapped buffers otherwise).
 * Together with b200k_gemm / b200k_block_scaled_gemm on `dst` this replaces
 * gather_matmul_kernel (reference: samples/AllGatherMatmul.py:28-120).  `round_tf32`
 * rounds fp32 payload to tf32 (nearest) on the way, as the reference kernel's cast does. */
typedef struct {
  const void* const* shards;   /* host array of `world` device pointers */
  void* dst;
  int64_t rows, row_bytes;
  int64_t src_stride_bytes, dst_stride_bytes;
  int32_t world, rank;
  int32_t round_tf32;
} b200k_peer_gather_args;

int b200k_peer_gather(const b200k_peer_gather_args* args, b200k_stream stream);

/* out[p * rows + i] = *(const float*)shards[p] for p < world, i < rows: the per-row scale
 * vector of a gathered operand whose shards carry one fp32 tensor scale each (NVFP4 form
 * of the gather GEMM).  `shards` as in b200k_peer_gather_args. */
int b200k_peer_scalar_expand(const void* const* shards, int32_t world, int64_t rows, float* out,
                             b200k_stream stream);

/* Up to 4 gathers and (optionally, scalar_shards != NULL) one scalar expansion in ONE launch:
 * what the NVFP4 form of the gather GEMM needs per step (packed operand, scale atoms, tensor
 * scales).  Every gather must be dense (both strides == row_bytes), without rounding, and of
 * the same world and rank; otherwise B200K_UNSUPPORTED and nothing is enqueued.  One launch
 * instead of three keeps the gather ahead of the GEMM it runs beside. */
int b200k_peer_gather_batch(const b200k_peer_gather_args* args, int32_t count,
                            const void* const* scalar_shards, int64_t scalar_rows, float* scalar_out,
                            b200k_stream stream);

/* ---- expert-parallel MoE (experts and tokens sharded over the ranks of one node) --------
 * No counterpart in the reference, whose only multi-GPU code is the AllGather sample; the
 * single-GPU pipeline these calls must reproduce is cutile_moe (samples/MoE.py:197-288).
 * Per layer every rank runs: count -> barrier -> plan -> dispatch -> barrier -> the two
 * grouped GEMMs on the rows it received (the second with c_peers) -> barrier -> b200k_topk_sum.
 * Nothing is read back by the host; all "peers" arguments are host arrays of `world` device
 * pointers this process can dereference (index = rank; its own buffer for its own rank).
 *
 * Layout of a rank's receive buffers (`capacity_rows` rows, see b200k_moe_ep_capacity_rows):
 * the rank's experts one after the other, every expert's rows padded to whole `tile_rows`-row
 * tiles, inside an expert the rows of source rank 0 first.  Row r carries meta[r] = source
 * rank * replicas_per_rank + replica id (token * topk + slot) at the source, or -1 for a
 * padding row, and weight[r], the replica's routing weight. */

/* Rows a receive buffer needs in the worst case (all replicas of all ranks routed to one
 * rank, every expert wasting tile_rows - 1 rows), a multiple of tile_rows. */
int64_t b200k_moe_ep_capacity_rows(int64_t replicas_per_rank, int32_t world, int32_t num_experts,
                                   int32_t tile_rows);

/* hist_peers[p][rank * num_experts + e] = number of this rank's routing ids equal to e, for
 * every rank p.  Ids outside [0, num_experts) are dropped and recorded in the status word. */
typedef struct {
  const void* topk_ids;            /* (num_replicas) int32 or int64 global expert ids */
  int64_t num_replicas;            /* tokens * topk of this rank */
  int32_t ids_are_int64;
  int32_t num_experts;
  int32_t world, rank;
  void* scratch;                   /* (num_experts + 1) ints of device memory, zero before the first call */
  const void* const* hist_peers;   /* every rank's table, (world, num_experts) int32 each */
} b200k_moe_ep_count_args;
int b200k_moe_ep_count(const b200k_moe_ep_count_args* args, b200k_stream stream);

/* From the complete table `hist` (this rank's own copy, after a barrier): first_row[e] = row of
 * the owner's receive buffer where this rank's rows for expert e start, cursor[e] = 0, and for
 * the experts this rank owns tile_group (local expert per row tile), *num_row_tiles, and
 * meta = -1 on the padding rows. */
typedef struct {
  const int32_t* hist;             /* (world, num_experts) */
  int32_t world, rank, num_experts, tile_rows;
  int64_t capacity_rows;
  int64_t* first_row;              /* [num_experts] */
  int32_t* cursor;                 /* [num_experts] */
  int32_t* tile_group;             /* [capacity_rows / tile_rows] */
  int32_t* num_row_tiles;          /* device scalar */
  int32_t* meta;                   /* this rank's receive-buffer meta, [capacity_rows] */
} b200k_moe_ep_plan_args;
int b200k_moe_ep_plan(const b200k_moe_ep_plan_args* args, b200k_stream stream);

/* Replica i (token i / topk) goes to the rank that owns expert topk_ids[i]: `row_bytes` of
 * src row (i / topk) and, when aux_bytes > 0, `aux_bytes` of aux row (i / topk) (the scale
 * bytes of a quantised row) are stored at row first_row[e] + cursor[e]++ of that rank's
 * buffers, with meta and weight as described above. */
typedef struct {
  const void* topk_ids;
  const float* weights;            /* (num_replicas) routing weights, NULL = 1 */
  int64_t num_replicas;
  int32_t topk, ids_are_int64, num_experts, world, rank;
  const void* src;                 /* (tokens, row_bytes) with row stride src_stride_bytes */
  int64_t src_stride_bytes, row_bytes;
  const void* aux;
  int64_t aux_stride_bytes, aux_bytes;
  const int64_t* first_row;
  int32_t* cursor;
  int64_t capacity_rows;
  void* const* row_peers;          /* (capacity_rows, row_bytes) each */
  void* const* aux_peers;          /* (capacity_rows, aux_bytes) each */
  void* const* meta_peers;         /* (capacity_rows) int32 each */
  void* const* weight_peers;       /* (capacity_rows) fp32 each */
} b200k_moe_ep_dispatch_args;
int b200k_moe_ep_dispatch(const b200k_moe_ep_dispatch_args* args, b200k_stream stream);

/* Barrier between the ranks of one node, as a kernel in stream order: everything the rank
 * stored into peer memory before it is visible to a peer once that peer's barrier has
 * passed.  flag_peers[p] = rank p's flag array (`world` int32, zero before the first call),
 * *epoch_counter a device int32 of this rank (zero before the first call).  Every rank must
 * launch the same sequence of barriers.  A rank that does not hear from a peer within
 * budget_us (0 = two seconds) records role 60 in the status word and goes on.  One GPU per
 * rank: ranks that share a GPU must not use it (their kernels need not run at the same time). */
int b200k_peer_barrier(const void* const* flag_peers, int32_t world, int32_t rank,
                       int32_t* epoch_counter, int32_t budget_us, b200k_stream stream);

/* ---- attention forward ------------------------------------------------
 * Out = softmax(qk_scale * Q K^T + mask) V per (batch, head); replaces fmha_kernel
 * (reference: test/kernels/attention.py:20-128) behind cutile_fmha
 * (samples/AttentionFMHA.py:138-210).  Q (B, Hq, Sq, D), K / V (B, Hkv, Sk, D), Out
 * (B, Hq, Sq, D), all f16 or all bf16, addressed through element strides so that
 * (B, S, H, D) storage works too; the head dimension is contiguous and 64 or 128.
 * `causal` masks key j for query i when j > i + input_pos; query head h reads
 * key/value head h / query_group_size. */
typedef struct {
  const void* q;
  const void* k;
  const void* v;
  void* out;
  int64_t batch, heads_q, heads_kv, seq_q, seq_kv;
  int64_t q_stride_b, q_stride_h, q_stride_s;
  int64_t k_stride_b, k_stride_h, k_stride_s;
  int64_t v_stride_b, v_stride_h, v_stride_s;
  int64_t o_stride_b, o_stride_h, o_stride_s;
  int64_t input_pos;
  int32_t head_dim;
  int32_t dtype;            /* B200K_F16 | B200K_BF16 */
  int32_t query_group_size;
  int32_t causal;
  float qk_scale;
  /* Optional scratch for the split-KV path (see b200k_fmha_workspace_bytes): 16-byte aligned
   * device memory, contents irrelevant before and after the call.  NULL = tensor-core
   * kernels only. */
  void* workspace;
  int64_t workspace_bytes;
} b200k_fmha_args;

int b200k_fmha_fwd(const b200k_fmha_args* args, b200k_stream stream);

/* Bytes of `workspace` with which b200k_fmha_fwd takes the split-KV path on the current
 * device: seq_q * query_group_size <= 8 query rows per key/value head (decode steps; the
 * reference benches q (1, 32, 1, 128) against 1024 keys, test/bench_attention.py:33-44).
 * The keys are split over CTAs that stream K and V once on the CUDA cores; a second kernel
 * merges the partial softmax states.  0 = the path does not apply. */
int64_t b200k_fmha_workspace_bytes(const b200k_fmha_args* args);

#ifdef __cplusplus
}
#endif
#endif /* B200K_H_ */
