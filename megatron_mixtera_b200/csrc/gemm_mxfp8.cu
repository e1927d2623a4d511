// y[M, N] = dequant(xq, x_sf)[M, K] * dequant(wq, w_sf)[N, K]^T (+ bias): MXFP8 GEMM for decode.
//
// Both operands are E4M3 with one E8M0 (power-of-two) scale per 32 elements along K.  The kernel has
// the structure of the bf16 weight-streaming GEMM (128-row weight tile = UMMA M side, tokens = UMMA
// N side, TMA ring, split-K partial sums reduced by a second kernel or by the consumer, shared epilogue) with two differences:
//   * one stage is 128 bytes of K per row (128 elements = four 32-wide scale blocks), and
//   * the MMA is tcgen05.mma kind::mxf8f6f4.block_scale: the scales of a stage (a 512-byte tile per
//     128 rows) arrive by a 1-D bulk copy, are moved to tensor memory with tcgen05.cp and applied by
//     the tensor core; the four MMAs of a stage pick their byte of the scale column through the
//     scale ids of the instruction descriptor.
//
// Scale-factor storage ("tile layout", also what the quantisation kernels write): for a matrix with R
// rows, sf[ceil(R/128)][K/128][512]; inside a tile the scale of (row r, 32-block b) sits at byte
// (r % 32) * 16 + ((r % 128) / 32) * 4 + (b % 4) - i.e. the 32-lane x 16-byte image tensor memory wants.
#include "common.cuh"
#include "quant.cuh"

namespace b200 {
namespace gemm {

constexpr int kFp8TileK = 128;  // bytes = elements of K per stage
constexpr int kSfTileBytes = 512;

template <int BT>
struct Fp8Config {
  static constexpr int kSfTilesX = BT > 128 ? 2 : 1;
  static constexpr int kStageBytesW = kTileN * kFp8TileK;
  static constexpr int kStageBytesX = BT * kFp8TileK;
  static constexpr int kOffX = kStageBytesW;
  static constexpr int kOffSfW = kOffX + kStageBytesX;
  static constexpr int kOffSfX = kOffSfW + kSfTileBytes;
  static constexpr int kTxBytes = kOffSfX + kSfTilesX * kSfTileBytes;
  static constexpr int kStageBytes = (kTxBytes + 1023) / 1024 * 1024;
  static constexpr int kStages = (BT <= 64) ? 4 : (BT <= 128 ? 3 : 2);
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024 + 256;
  static constexpr int kSfCols = 4 + 4 * kSfTilesX;  // tensor-memory columns of one stage's scales
  static constexpr int kTmemNeeded = BT + kStages * kSfCols;
  static constexpr int kTmemCols = kTmemNeeded <= 32 ? 32 : kTmemNeeded <= 64 ? 64 : kTmemNeeded <= 128 ? 128
                                   : kTmemNeeded <= 256 ? 256 : 512;
};

struct Fp8Operands {
  const uint8_t* w_sf;  // tile layout, [n tiles][K/128][512]
  const uint8_t* x_sf;  // tile layout, [ceil(M/128)][K/128][512]
  int k_tiles;          // K / 128
};

template <int BT>
__global__ void __launch_bounds__(kThreads, 1)
gemm_mxfp8_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, Params p,
                  Fp8Operands q) {
  using C = Fp8Config<BT>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + C::kStages * C::kStageBytes);
  uint64_t* empty_bar = full_bar + C::kStages;
  uint64_t* accum_bar = empty_bar + C::kStages;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(accum_bar + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int n_tile = blockIdx.x;
  const int split = blockIdx.y;
  const int m_block = blockIdx.z;
  const int n0 = n_tile * kTileN;
  const int m0 = m_block * BT;
  const int kb_begin = split * p.k_blocks_per_split;
  const int kb_end = min(p.num_k_blocks, kb_begin + p.k_blocks_per_split);
  const int num_kb = kb_end - kb_begin;

  if (tid == 0) {
    for (int s = 0; s < C::kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(accum_bar, 1);
    *abort_flag = 0;
    fence_barrier_init();
    prefetch_tensormap(&map_w);
    prefetch_tensormap(&map_x);
  }
  if (warp == 0) {
    tmem_alloc(tmem_slot, C::kTmemCols);
    tmem_relinquish_alloc_permit();
  }
  tcgen05_fence_before_sync();
  __syncthreads();
  tcgen05_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  // scale tiles of this CTA: weights -> tile row n_tile; tokens -> tile row m0 / 128 (+1 for BT = 256)
  const uint8_t* w_sf = q.w_sf + static_cast<int64_t>(n_tile) * q.k_tiles * kSfTileBytes;
  const uint8_t* x_sf = q.x_sf + static_cast<int64_t>(m0 / 128) * q.k_tiles * kSfTileBytes;

  pdl_launch_dependents();
  if (warp == 0) {
    if (lane == 0) {
      // ---------------- producer ----------------
      auto load_w = [&](int i, int s) {
        uint8_t* stage = smem + s * C::kStageBytes;
        tma_load_2d(stage, &map_w, &full_bar[s], 0, (n_tile * q.k_tiles + kb_begin + i) * kTileN);  // packed tile
        bulk_load_1d(stage + C::kOffSfW, w_sf + static_cast<int64_t>(kb_begin + i) * kSfTileBytes, kSfTileBytes,
                     &full_bar[s]);
      };
      auto load_x = [&](int i, int s) {
        uint8_t* stage = smem + s * C::kStageBytes;
        tma_load_2d(stage + C::kOffX, &map_x, &full_bar[s], (kb_begin + i) * kFp8TileK, m0);
#pragma unroll
        for (int t = 0; t < C::kSfTilesX; ++t)
          bulk_load_1d(stage + C::kOffSfX + t * kSfTileBytes,
                       x_sf + (static_cast<int64_t>(t) * q.k_tiles + kb_begin + i) * kSfTileBytes, kSfTileBytes,
                       &full_bar[s]);
      };
      // weights and their scales are written by no kernel: request them before the programmatic wait
      const int pre = num_kb < C::kStages ? num_kb : C::kStages;
      for (int i = 0; i < pre; ++i) {
        mbar_arrive_expect_tx(&full_bar[i], C::kTxBytes);
        load_w(i, i);
      }
      pdl_wait();
      for (int i = 0; i < pre; ++i) load_x(i, i);
      for (int i = pre; i < num_kb; ++i) {
        const int s = i % C::kStages;
        const uint32_t phase = (i / C::kStages) & 1;
        mbar_wait_bounded(&empty_bar[s], phase ^ 1, abort_flag, kStatusGemmTimeout);
        mbar_arrive_expect_tx(&full_bar[s], C::kTxBytes);
        load_w(i, s);
        load_x(i, s);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0) {
      // ---------------- UMMA issuer ----------------
      constexpr int kN = BT < 16 ? 16 : BT;
      const uint32_t sf_base = tmem_base + BT;                       // scale slots live after the accumulator
      const uint32_t sfb_col_off = static_cast<uint32_t>((m0 % 128) / 32);  // token rows inside their 128-row tile
      for (int i = 0; i < num_kb; ++i) {
        const int s = i % C::kStages;
        const uint32_t phase = (i / C::kStages) & 1;
        mbar_wait_bounded(&full_bar[s], phase, abort_flag, kStatusGemmTimeout);
        tcgen05_fence_after_sync();
        const uint32_t stage_addr = smem_u32(smem + s * C::kStageBytes);
        const uint32_t sfa = sf_base + s * C::kSfCols;
        const uint32_t sfb = sfa + 4;
        tmem_cp_32x128b_warpx4(sfa, umma_desc_sf_tile(stage_addr + C::kOffSfW));
#pragma unroll
        for (int t = 0; t < C::kSfTilesX; ++t)
          tmem_cp_32x128b_warpx4(sfb + 4 * t, umma_desc_sf_tile(stage_addr + C::kOffSfX + t * kSfTileBytes));
        const uint64_t a_desc = umma_desc_k_major_sw128(stage_addr);
        const uint64_t b_desc = umma_desc_k_major_sw128(stage_addr + C::kOffX);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          // 32 elements = 32 bytes per K step inside the 128-byte swizzle row
          umma_mxf8_block_scaled(tmem_base, a_desc + 2 * k, b_desc + 2 * k, umma_idesc_mxf8(kTileN, kN, k, k), sfa,
                                 sfb + sfb_col_off, (i > 0 || k > 0) ? 1u : 0u);
        }
        umma_commit(&empty_bar[s]);
      }
      umma_commit(accum_bar);
    }
    __syncwarp();
  }

  pdl_wait();
  mbar_wait_bounded(accum_bar, 0, abort_flag, kStatusGemmTimeout);
  tcgen05_fence_after_sync();
  epilogue<BT>(p, tmem_base, smem, n_tile, split, m_block);

  tcgen05_fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem_base, C::kTmemCols);
}

template <int BT>
static int launch_mxfp8(const void* xq, const void* x_sf, const void* wq, const void* w_sf, const void* bias, void* y,
                        int64_t ldy, int M, int N, int K, void* workspace, size_t workspace_bytes, cudaStream_t stream,
                        float* partials_out = nullptr, size_t partials_bytes = 0, int* splits_out = nullptr) {
  using C = Fp8Config<BT>;
  // weights: tile-major (see weight_tile_offset) = a [tiles * 128 rows][128 bytes] matrix
  const int n_tiles = (N + kTileN - 1) / kTileN;
  const uint64_t wd[2] = {static_cast<uint64_t>(kFp8TileK), static_cast<uint64_t>(n_tiles) * (K / kFp8TileK) * kTileN};
  const uint64_t wst[1] = {static_cast<uint64_t>(kFp8TileK)};
  const uint64_t ws[1] = {static_cast<uint64_t>(K)};
  const uint32_t wb[2] = {kFp8TileK, kTileN};
  const uint64_t xd[2] = {static_cast<uint64_t>(K), static_cast<uint64_t>(M)};
  const uint32_t xb[2] = {kFp8TileK, BT};
  const CUtensorMap* mw = get_tensor_map(wq, 2, wd, wst, wb, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                         CU_TENSOR_MAP_DATA_TYPE_UINT8);
  const CUtensorMap* mx = get_tensor_map(xq, 2, xd, ws, xb, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                         CU_TENSOR_MAP_DATA_TYPE_UINT8);
  if (!mw || !mx) return B200_ERR_DRIVER;
  const int m_blocks = (M + BT - 1) / BT;
  const int num_kb = K / kFp8TileK;
  const int splits = choose_splits(n_tiles * m_blocks, num_kb);
  Params p;
  p.bias = static_cast<const __nv_bfloat16*>(bias);
  p.y = static_cast<__nv_bfloat16*>(y);
  p.ldy = ldy;
  p.M = M;
  p.N = N;
  p.K = K;
  p.num_k_blocks = num_kb;
  p.k_blocks_per_split = (num_kb + splits - 1) / splits;
  p.num_splits = splits;
  p.partials = nullptr;
  p.keep_partials = partials_out != nullptr;
  p.gated = 0;
  if (partials_out != nullptr) {
    if (partials_bytes < static_cast<size_t>(splits) * M * N * sizeof(float)) return B200_ERR_WORKSPACE;
    p.partials = partials_out;
    *splits_out = splits;
  } else if (splits > 1) {
    const size_t need = static_cast<size_t>(splits) * M * N * sizeof(float);
    if (workspace == nullptr || workspace_bytes < need || !aligned16(workspace)) return B200_ERR_WORKSPACE;
    p.partials = static_cast<float*>(workspace);
  }
  Fp8Operands q;
  q.w_sf = static_cast<const uint8_t*>(w_sf);
  q.x_sf = static_cast<const uint8_t*>(x_sf);
  q.k_tiles = num_kb;
  static std::atomic<uint64_t> smem_attr_done{0};
  if (ensure_dynamic_smem(gemm_mxfp8_kernel<BT>, C::kSmemBytes, smem_attr_done) != B200_OK) return B200_ERR_LAUNCH;
  dim3 grid(n_tiles, splits, m_blocks);
  const int rc = launch_pdl(gemm_mxfp8_kernel<BT>, grid, dim3(kThreads), C::kSmemBytes, stream, *mw, *mx, p, q);
  if (rc != B200_OK || splits == 1 || p.keep_partials) return rc;
  return launch_splitk_reduce(p, stream);
}

// ---------------------------------------------------------------------------------------------
// fc1 + SwiGLU + MXFP8 quantisation in one kernel ("gate / up pair").
//
// w is the gated fc1 weight in the reference's row order [gate ; up] ([2F, K], no re-arrangement).  One CTA
// owns 128 gate features and the 128 matching up features: per K block it loads the two weight tiles and ONE
// token tile and issues two sets of UMMAs into two accumulators, so the token tile - at 128 tokens as many
// bytes as a weight tile - crosses from L2 into the SM once per 256 weight rows instead of once per 128.
// The epilogue holds gate and up of a feature in the same thread: bf16(bf16(silu(bf16 gate)) * bf16 up), the
// rounding points of the unfused path, goes to shared memory, is re-read as 8-feature vectors and written as
// E4M3 + E8M0 scales (the fc2 input) - no [tokens, 2F] bf16 matrix, no activation kernel.  Whole-K units
// only (the caller falls back to GEMM + activation kernel when the grid would be too small without split-K).
// ---------------------------------------------------------------------------------------------
template <int BT>
struct PairConfig {
  static_assert(BT <= 128, "two accumulators of BT columns and the scale slots must fit 512 tensor-memory columns");
  static constexpr int kStageBytesW = kTileN * kFp8TileK;  // one of the two weight tiles
  static constexpr int kStageBytesX = BT * kFp8TileK;
  static constexpr int kOffUp = kStageBytesW;
  static constexpr int kOffX = 2 * kStageBytesW;
  static constexpr int kOffSfGate = kOffX + kStageBytesX;
  static constexpr int kOffSfUp = kOffSfGate + kSfTileBytes;
  static constexpr int kOffSfX = kOffSfUp + kSfTileBytes;
  static constexpr int kTxBytes = kOffSfX + kSfTileBytes;
  static constexpr int kStageBytes = (kTxBytes + 1023) / 1024 * 1024;
  static constexpr int kStages = 4;
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024 + 256;
  static constexpr int kSfCols = 12;  // gate scales, up scales, token scales: 4 columns each
  static constexpr int kTmemNeeded = 2 * BT + kStages * kSfCols;
  static constexpr int kTmemCols = kTmemNeeded <= 128 ? 128 : kTmemNeeded <= 256 ? 256 : 512;
  static_assert(kStages * kStageBytes >= BT * 128 * 2, "the epilogue parks a [BT][128] bf16 tile in the stage memory");
};

struct PairParams {
  uint8_t* q_out;        // [M, F] E4M3
  uint8_t* sf_out;       // E8M0 scales of q_out in the tile layout
  __nv_bfloat16* y_out;  // [M, F] bf16 instead (when q_out is null)
  int64_t ldy;
  const uint8_t* w_sf;
  const uint8_t* x_sf;
  int M, F, k_tiles;     // k_tiles = K / 128
};

constexpr int kPairThreads = 512;  // 16 warps: the SwiGLU epilogue is arithmetic-heavy and is not overlapped with loads

template <int BT>
__global__ void __launch_bounds__(kPairThreads, 1)
gemm_mxfp8_pair_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, PairParams p) {
  using C = PairConfig<BT>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + C::kStages * C::kStageBytes);
  uint64_t* empty_bar = full_bar + C::kStages;
  uint64_t* accum_bar = empty_bar + C::kStages;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(accum_bar + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int pair = blockIdx.x;            // features [pair * 128, pair * 128 + 128)
  const int m_block = blockIdx.z;
  const int m0 = m_block * BT;
  const int gate_tile = pair;
  const int up_tile = p.F / kTileN + pair;
  const int num_kb = p.k_tiles;

  if (tid == 0) {
    for (int s = 0; s < C::kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(accum_bar, 1);
    *abort_flag = 0;
    fence_barrier_init();
    prefetch_tensormap(&map_w);
    prefetch_tensormap(&map_x);
  }

  pdl_launch_dependents();
  const uint8_t* sf_gate = p.w_sf + static_cast<int64_t>(pair) * p.k_tiles * kSfTileBytes;
  const uint8_t* sf_up = p.w_sf + static_cast<int64_t>(p.F / kTileN + pair) * p.k_tiles * kSfTileBytes;
  const uint8_t* sf_x = p.x_sf + static_cast<int64_t>(m0 / 128) * p.k_tiles * kSfTileBytes;
  auto load_w = [&](int i, int s) {
    uint8_t* stage = smem + s * C::kStageBytes;
    tma_load_2d(stage, &map_w, &full_bar[s], 0, (gate_tile * p.k_tiles + i) * kTileN);  // packed tiles
    tma_load_2d(stage + C::kOffUp, &map_w, &full_bar[s], 0, (up_tile * p.k_tiles + i) * kTileN);
    bulk_load_1d(stage + C::kOffSfGate, sf_gate + static_cast<int64_t>(i) * kSfTileBytes, kSfTileBytes, &full_bar[s]);
    bulk_load_1d(stage + C::kOffSfUp, sf_up + static_cast<int64_t>(i) * kSfTileBytes, kSfTileBytes, &full_bar[s]);
  };
  auto load_x = [&](int i, int s) {
    uint8_t* stage = smem + s * C::kStageBytes;
    tma_load_2d(stage + C::kOffX, &map_x, &full_bar[s], i * kFp8TileK, m0);
    bulk_load_1d(stage + C::kOffSfX, sf_x + static_cast<int64_t>(i) * kSfTileBytes, kSfTileBytes, &full_bar[s]);
  };
  const int pre = num_kb < C::kStages ? num_kb : C::kStages;
  if (tid == 0) {
    // The weights are written by no kernel: their first tiles are requested before the programmatic-launch wait
    // and before tensor memory is allocated (a CTA of the preceding kernel on this SM may still hold it).
    for (int i = 0; i < pre; ++i) {
      mbar_arrive_expect_tx(&full_bar[i], C::kTxBytes);
      load_w(i, i);
    }
  }
  if (warp == 2) {
    tmem_alloc(tmem_slot, C::kTmemCols);
    tmem_relinquish_alloc_permit();
  }
  tcgen05_fence_before_sync();
  __syncthreads();
  tcgen05_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0 && lane == 0) {
    // ---------------- producer ----------------
    pdl_wait();
    for (int i = 0; i < pre; ++i) load_x(i, i);
    for (int i = pre; i < num_kb; ++i) {
      const int s = i % C::kStages;
      const uint32_t phase = (i / C::kStages) & 1;
      mbar_wait_bounded(&empty_bar[s], phase ^ 1, abort_flag, kStatusGemmTimeout);
      mbar_arrive_expect_tx(&full_bar[s], C::kTxBytes);
      load_w(i, s);
      load_x(i, s);
    }
  }
  if (warp == 1 && lane == 0) {
    // ---------------- UMMA issuer ----------------
    constexpr int kN = BT < 16 ? 16 : BT;
    const uint32_t sf_base = tmem_base + 2 * BT;
    const uint32_t sfb_col_off = static_cast<uint32_t>((m0 % 128) / 32);
    for (int i = 0; i < num_kb; ++i) {
      const int s = i % C::kStages;
      const uint32_t phase = (i / C::kStages) & 1;
      mbar_wait_bounded(&full_bar[s], phase, abort_flag, kStatusGemmTimeout);
      tcgen05_fence_after_sync();
      const uint32_t stage_addr = smem_u32(smem + s * C::kStageBytes);
      const uint32_t sfa_g = sf_base + s * C::kSfCols;
      const uint32_t sfa_u = sfa_g + 4;
      const uint32_t sfb = sfa_g + 8;
      tmem_cp_32x128b_warpx4(sfa_g, umma_desc_sf_tile(stage_addr + C::kOffSfGate));
      tmem_cp_32x128b_warpx4(sfa_u, umma_desc_sf_tile(stage_addr + C::kOffSfUp));
      tmem_cp_32x128b_warpx4(sfb, umma_desc_sf_tile(stage_addr + C::kOffSfX));
      const uint64_t g_desc = umma_desc_k_major_sw128(stage_addr);
      const uint64_t u_desc = umma_desc_k_major_sw128(stage_addr + C::kOffUp);
      const uint64_t b_desc = umma_desc_k_major_sw128(stage_addr + C::kOffX);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const uint32_t idesc = umma_idesc_mxf8(kTileN, kN, k, k);
        const uint32_t acc = (i > 0 || k > 0) ? 1u : 0u;
        umma_mxf8_block_scaled(tmem_base, g_desc + 2 * k, b_desc + 2 * k, idesc, sfa_g, sfb + sfb_col_off, acc);
        umma_mxf8_block_scaled(tmem_base + BT, u_desc + 2 * k, b_desc + 2 * k, idesc, sfa_u, sfb + sfb_col_off, acc);
      }
      umma_commit(&empty_bar[s]);
    }
    umma_commit(accum_bar);
  }
  __syncwarp();

  // ---------------- epilogue: all sixteen warps ----------------
  pdl_wait();  // the outputs may still be read by the previous kernel until here
  mbar_wait_bounded(accum_bar, 0, abort_flag, kStatusGemmTimeout);
  tcgen05_fence_after_sync();
  {
    // thread = feature (TMEM lane): gate in accumulator 0, up in accumulator 1, same column = same token.  A warp can
    // reach the 32 lanes of quadrant (warp % 4) only; the four warps of a quadrant take 32 tokens each.
    __nv_bfloat16* tile = reinterpret_cast<__nv_bfloat16*>(smem);  // [BT][128] products (every UMMA has completed)
    const int quad = warp & 3;
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16);
    const int f = quad * 32 + lane;
#pragma unroll 1
    for (int c0 = (warp >> 2) * 32; c0 < BT; c0 += (kPairThreads / 128) * 32) {
      uint32_t g[32], u[32];
      tmem_ld_32x32b_x32(lane_addr + c0, g);
      tmem_ld_32x32b_x32(lane_addr + BT + c0, u);
      tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        const float gv = bf16_round(__uint_as_float(g[j]));
        const float uv = bf16_round(__uint_as_float(u[j]));
        const float a = bf16_round(gv / (1.f + expf(-gv)));
        tile[(c0 + j) * 128 + f] = __float2bfloat16_rn(a * uv);
      }
    }
    __syncthreads();
    // 16 vectors of 8 features per token; consecutive lanes take consecutive vectors, so lanes 4j .. 4j+3 hold one
    // 32-feature scale block, as the quantiser expects
    const uint4* tile_v = reinterpret_cast<const uint4*>(tile);
#pragma unroll 1
    for (int v = tid; v < BT * 16; v += kPairThreads) {
      const int m_local = v >> 4;
      const int i = v & 15;
      const int row = m0 + m_local;
      const bool valid = row < p.M;
      const uint4 w4 = tile_v[v];
      const int col0 = pair * kTileN + i * 8;
      if (p.q_out != nullptr) {
        const uint32_t ww[4] = {w4.x, w4.y, w4.z, w4.w};
        float y[8];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          y[2 * k] = bf16_lo(ww[k]);
          y[2 * k + 1] = bf16_hi(ww[k]);
        }
        mx::quantize8(y, valid, row, col0, p.q_out, p.F, p.sf_out, p.F / 128);
      } else if (valid) {
        *reinterpret_cast<uint4*>(p.y_out + static_cast<int64_t>(row) * p.ldy + col0) = w4;
      }
    }
  }

  tcgen05_fence_before_sync();
  __syncthreads();
  if (warp == 2) tmem_dealloc(tmem_base, C::kTmemCols);
}

static int pick_bt_pair(int M) { return M <= 32 ? 32 : (M <= 64 ? 64 : 128); }

template <int BT>
static int launch_mxfp8_pair(const void* xq, const void* x_sf, const void* wq, const void* w_sf, void* q_out, void* sf_out,
                             void* y_out, int64_t ldy, int M, int F, int K, cudaStream_t stream) {
  using C = PairConfig<BT>;
  const uint64_t wd[2] = {static_cast<uint64_t>(kFp8TileK), static_cast<uint64_t>(2 * F / kTileN) * (K / kFp8TileK) * kTileN};
  const uint64_t wst[1] = {static_cast<uint64_t>(kFp8TileK)};
  const uint64_t ws[1] = {static_cast<uint64_t>(K)};
  const uint32_t wb[2] = {kFp8TileK, kTileN};
  const uint64_t xd[2] = {static_cast<uint64_t>(K), static_cast<uint64_t>(M)};
  const uint32_t xb[2] = {kFp8TileK, BT};
  const CUtensorMap* mw = get_tensor_map(wq, 2, wd, wst, wb, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                         CU_TENSOR_MAP_DATA_TYPE_UINT8);
  const CUtensorMap* mx_ = get_tensor_map(xq, 2, xd, ws, xb, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                          CU_TENSOR_MAP_DATA_TYPE_UINT8);
  if (!mw || !mx_) return B200_ERR_DRIVER;
  PairParams p;
  p.q_out = static_cast<uint8_t*>(q_out);
  p.sf_out = static_cast<uint8_t*>(sf_out);
  p.y_out = static_cast<__nv_bfloat16*>(y_out);
  p.ldy = ldy;
  p.w_sf = static_cast<const uint8_t*>(w_sf);
  p.x_sf = static_cast<const uint8_t*>(x_sf);
  p.M = M;
  p.F = F;
  p.k_tiles = K / kFp8TileK;
  static std::atomic<uint64_t> smem_attr_done{0};
  if (ensure_dynamic_smem(gemm_mxfp8_pair_kernel<BT>, C::kSmemBytes, smem_attr_done) != B200_OK) return B200_ERR_LAUNCH;
  dim3 grid(F / kTileN, 1, (M + BT - 1) / BT);
  return launch_pdl(gemm_mxfp8_pair_kernel<BT>, grid, dim3(kPairThreads), C::kSmemBytes, stream, *mw, *mx_, p);
}

}  // namespace gemm
}  // namespace b200

extern "C" {

size_t b200_mxfp8_scale_bytes(int rows, int K) {
  if (rows <= 0 || K <= 0 || K % 128 != 0) return 0;
  // whole 256-row groups, so that a 256-token block of the GEMM can always read two tiles
  return static_cast<size_t>((rows + 255) / 256) * 2 * (K / 128) * b200::gemm::kSfTileBytes;
}

size_t b200_gemm_mxfp8_splitk_bytes(int M, int N, int K) {
  using namespace b200::gemm;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  const int bt = pick_bt(M);
  const int tiles = ((N + kTileN - 1) / kTileN) * ((M + bt - 1) / bt);
  return static_cast<size_t>(choose_splits(tiles, K / kFp8TileK)) * M * N * sizeof(float);
}

int b200_gemm_mxfp8_splitk(const void* xq, const void* x_sf, const void* wq, const void* w_sf, int M, int N, int K,
                           float* partials, size_t partials_bytes, int* num_splits, b200_stream_t stream) {
  using namespace b200;
  if (!xq || !x_sf || !wq || !w_sf || !partials || !num_splits || M <= 0 || N <= 0 || K <= 0)
    return B200_ERR_INVALID_ARGUMENT;
  if (K % 128 != 0) return B200_ERR_ALIGNMENT;
  if (!aligned16(xq) || !aligned16(wq) || !aligned16(x_sf) || !aligned16(w_sf) || !aligned16(partials))
    return B200_ERR_ALIGNMENT;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  switch (gemm::pick_bt(M)) {
    case 32: return gemm::launch_mxfp8<32>(xq, x_sf, wq, w_sf, nullptr, nullptr, N, M, N, K, nullptr, 0, s, partials, partials_bytes, num_splits);
    case 64: return gemm::launch_mxfp8<64>(xq, x_sf, wq, w_sf, nullptr, nullptr, N, M, N, K, nullptr, 0, s, partials, partials_bytes, num_splits);
    case 128: return gemm::launch_mxfp8<128>(xq, x_sf, wq, w_sf, nullptr, nullptr, N, M, N, K, nullptr, 0, s, partials, partials_bytes, num_splits);
    default: return gemm::launch_mxfp8<256>(xq, x_sf, wq, w_sf, nullptr, nullptr, N, M, N, K, nullptr, 0, s, partials, partials_bytes, num_splits);
  }
}

size_t b200_gemm_mxfp8_workspace_bytes(int M, int N, int K) {
  using namespace b200::gemm;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  const int bt = pick_bt(M);
  const int tiles = ((N + kTileN - 1) / kTileN) * ((M + bt - 1) / bt);
  const int splits = choose_splits(tiles, K / kFp8TileK);
  if (splits == 1) return 0;
  return static_cast<size_t>(splits) * static_cast<size_t>(M) * N * sizeof(float);
}

int b200_gemm_mxfp8(const void* xq, const void* x_sf, const void* wq, const void* w_sf, const void* bias, void* y,
                    int64_t ldy, int M, int N, int K, void* workspace, size_t workspace_bytes, b200_stream_t stream) {
  using namespace b200;
  if (!xq || !x_sf || !wq || !w_sf || !y || M <= 0 || N <= 0 || K <= 0) return B200_ERR_INVALID_ARGUMENT;
  if (K % 128 != 0 || ldy < N) return B200_ERR_ALIGNMENT;
  if (!aligned16(xq) || !aligned16(wq) || !aligned16(x_sf) || !aligned16(w_sf)) return B200_ERR_ALIGNMENT;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  switch (gemm::pick_bt(M)) {
    case 32: return gemm::launch_mxfp8<32>(xq, x_sf, wq, w_sf, bias, y, ldy, M, N, K, workspace, workspace_bytes, s);
    case 64: return gemm::launch_mxfp8<64>(xq, x_sf, wq, w_sf, bias, y, ldy, M, N, K, workspace, workspace_bytes, s);
    case 128: return gemm::launch_mxfp8<128>(xq, x_sf, wq, w_sf, bias, y, ldy, M, N, K, workspace, workspace_bytes, s);
    default: return gemm::launch_mxfp8<256>(xq, x_sf, wq, w_sf, bias, y, ldy, M, N, K, workspace, workspace_bytes, s);
  }
}

int b200_gemm_mxfp8_swiglu(const void* xq, const void* x_sf, const void* wq, const void* w_sf, void* q_out, void* sf_out,
                           void* y_out, int64_t ldy, int M, int F, int K, b200_stream_t stream) {
  using namespace b200;
  if (!xq || !x_sf || !wq || !w_sf || M <= 0 || F <= 0 || K <= 0) return B200_ERR_INVALID_ARGUMENT;
  if ((q_out == nullptr) == (y_out == nullptr) || (q_out != nullptr) != (sf_out != nullptr)) return B200_ERR_INVALID_ARGUMENT;
  if (K % 128 != 0 || F % 128 != 0 || (y_out && (ldy < F || ldy % 8 != 0))) return B200_ERR_ALIGNMENT;
  if (!aligned16(xq) || !aligned16(wq) || !aligned16(x_sf) || !aligned16(w_sf) || (q_out && !aligned16(q_out)) ||
      (sf_out && !aligned16(sf_out)) || (y_out && !aligned16(y_out)))
    return B200_ERR_ALIGNMENT;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  switch (gemm::pick_bt_pair(M)) {
    case 32: return gemm::launch_mxfp8_pair<32>(xq, x_sf, wq, w_sf, q_out, sf_out, y_out, ldy, M, F, K, s);
    case 64: return gemm::launch_mxfp8_pair<64>(xq, x_sf, wq, w_sf, q_out, sf_out, y_out, ldy, M, F, K, s);
    default: return gemm::launch_mxfp8_pair<128>(xq, x_sf, wq, w_sf, q_out, sf_out, y_out, ldy, M, F, K, s);
  }
}

}  // extern "C"
