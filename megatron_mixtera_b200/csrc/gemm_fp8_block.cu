// y[M, N] = dequant(xq, x_scale)[M, K] * dequant(wq, w_scale)[N, K]^T (+ bias): block-scaled FP8 GEMM
// with fp32 scales - one per 128 x 128 weight block and one per token per 128 elements of K.
//
// fp32 scales cannot ride along inside the tensor core (the block-scaled UMMA takes power-of-two E8M0
// scales only), so each 128-wide K block is multiplied on its own and promoted in registers:
//
//   warp 4 / lane 0 : producer  - per stage (= one K block): weight tile [128 x 128 B], token tile
//                                 [BT x 128 B] (TMA, 128-byte swizzle) and the BT token scales (bulk copy)
//   warp 5 / lane 0 : UMMA      - 4 x tcgen05.mma kind::f8f6f4 into one of two TMEM accumulators
//   warps 0-3       : promoters - tcgen05.ld the finished block accumulator, total += acc * (w_scale *
//                                 x_scale[token]) in registers, hand the accumulator back
// (producer and UMMA issuer are warps of their own: the promoters release the stages and accumulators
// they wait for, so they must not share a thread with them)
//
// The MMA of block i+1 runs while block i is promoted.  At the end the totals go back to tensor memory
// and the shared epilogue (bf16 store or split-K partial store) takes over.
#include "common.cuh"

namespace b200 {
namespace gemm {

constexpr int kBlkThreads = 192;

template <int BT>
struct BlkConfig {
  static_assert(BT <= 128, "the promoted totals live in registers: at most 128 tokens per CTA");
  static constexpr int kStageBytesW = kTileN * 128;
  static constexpr int kStageBytesX = BT * 128;
  static constexpr int kOffX = kStageBytesW;
  static constexpr int kOffScale = kOffX + kStageBytesX;
  static constexpr int kStageBytes = (kOffScale + BT * 4 + 1023) / 1024 * 1024;
  static constexpr int kStages = (BT <= 64) ? 4 : 3;
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024 + 256;
  static constexpr int kTmemCols = 2 * BT < 32 ? 32 : 2 * BT;  // two block accumulators (64 / 128 / 256)
};

struct BlkOperands {
  const float* w_scale;  // [ceil(N/128)][K/128]
  const float* x_scale;  // [K/128][m_pad]
  int k_tiles;
  int m_pad;
};

__device__ __forceinline__ void tmem_st_32x32b_x32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
      "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]),
      "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]),
      "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// kind::f8f6f4, E4M3 x E4M3 -> fp32, both operands K-major
__host__ __device__ constexpr uint32_t umma_idesc_f8(int m, int n) {
  return (1u << 4) | (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(m >> 4) << 24);
}
__device__ __forceinline__ void umma_f8(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                        uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(tmem_d),
      "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}

template <int BT>
__global__ void __launch_bounds__(kBlkThreads, 1)
gemm_fp8_block_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, Params p,
                      BlkOperands q) {
  using C = BlkConfig<BT>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + C::kStages * C::kStageBytes);
  uint64_t* empty_bar = full_bar + C::kStages;
  uint64_t* acc_full = empty_bar + C::kStages;
  uint64_t* acc_empty = acc_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
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
  // token scales of this CTA's rows that exist (a multiple of 4 floats = 16 bytes by construction of m_pad)
  const int scale_floats = min(BT, q.m_pad - m0);
  const uint32_t tx_bytes = C::kOffScale + scale_floats * 4;

  if (tid == 0) {
    for (int s = 0; s < C::kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1 + 4);  // the UMMA commit + the four promoter warps (they read the scales)
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], 4);
    }
    *abort_flag = 0;
    fence_barrier_init();
    prefetch_tensormap(&map_w);
    prefetch_tensormap(&map_x);
  }
  if (warp == 4) {
    tmem_alloc(tmem_slot, C::kTmemCols);
    tmem_relinquish_alloc_permit();
  }
  tcgen05_fence_before_sync();
  __syncthreads();
  tcgen05_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  pdl_launch_dependents();
  if (warp == 4) {
   if (lane == 0) {
    // ---------------- producer ----------------
    auto load_x = [&](int i, int s) {
      uint8_t* stage = smem + s * C::kStageBytes;
      tma_load_2d(stage + C::kOffX, &map_x, &full_bar[s], (kb_begin + i) * 128, m0);
      bulk_load_1d(stage + C::kOffScale, q.x_scale + static_cast<int64_t>(kb_begin + i) * q.m_pad + m0,
                   scale_floats * 4, &full_bar[s]);
    };
    const int pre = num_kb < C::kStages ? num_kb : C::kStages;
    for (int i = 0; i < pre; ++i) {  // weights are written by no kernel: request them before the wait
      mbar_arrive_expect_tx(&full_bar[i], tx_bytes);
      tma_load_2d(smem + i * C::kStageBytes, &map_w, &full_bar[i], 0, (n_tile * q.k_tiles + kb_begin + i) * kTileN);
    }
    pdl_wait();
    for (int i = 0; i < pre; ++i) load_x(i, i);
    for (int i = pre; i < num_kb; ++i) {
      const int s = i % C::kStages;
      const uint32_t phase = (i / C::kStages) & 1;
      mbar_wait_bounded(&empty_bar[s], phase ^ 1, abort_flag, kStatusGemmTimeout);
      mbar_arrive_expect_tx(&full_bar[s], tx_bytes);
      tma_load_2d(smem + s * C::kStageBytes, &map_w, &full_bar[s], 0, (n_tile * q.k_tiles + kb_begin + i) * kTileN);
      load_x(i, s);
    }
   }
  } else if (warp == 5) {
   if (lane == 0) {
    // ---------------- UMMA issuer ----------------
    constexpr uint32_t idesc = umma_idesc_f8(kTileN, BT < 16 ? 16 : BT);
    for (int i = 0; i < num_kb; ++i) {
      const int s = i % C::kStages;
      const int b = i & 1;
      mbar_wait_bounded(&full_bar[s], (i / C::kStages) & 1, abort_flag, kStatusGemmTimeout);
      mbar_wait_bounded(&acc_empty[b], ((i >> 1) & 1) ^ 1, abort_flag, kStatusGemmTimeout);
      tcgen05_fence_after_sync();
      const uint32_t stage_addr = smem_u32(smem + s * C::kStageBytes);
      const uint64_t a_desc = umma_desc_k_major_sw128(stage_addr);
      const uint64_t b_desc = umma_desc_k_major_sw128(stage_addr + C::kOffX);
#pragma unroll
      for (int k = 0; k < 4; ++k) umma_f8(tmem_base + b * BT, a_desc + 2 * k, b_desc + 2 * k, idesc, k > 0 ? 1u : 0u);
      umma_commit(&empty_bar[s]);
      umma_commit(&acc_full[b]);
    }
   }
  } else {
  // ---------------- promoters: warps 0-3 ----------------
  pdl_wait();
  float total[BT];
#pragma unroll
  for (int j = 0; j < BT; ++j) total[j] = 0.f;
  const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(warp * 32) << 16);
  const float* w_scale = q.w_scale + static_cast<int64_t>(n_tile) * q.k_tiles + kb_begin;
  float sw_next = num_kb > 0 ? __ldg(w_scale) : 0.f;
  for (int i = 0; i < num_kb; ++i) {
    const int s = i % C::kStages;
    const int b = i & 1;
    const float sw = sw_next;
    if (i + 1 < num_kb) sw_next = __ldg(w_scale + i + 1);
    mbar_wait_bounded(&acc_full[b], (i >> 1) & 1, abort_flag, kStatusGemmTimeout);
    tcgen05_fence_after_sync();
    const float* xs = reinterpret_cast<const float*>(smem + s * C::kStageBytes + C::kOffScale);
#pragma unroll
    for (int c0 = 0; c0 < BT; c0 += 32) {
      uint32_t r[32];
      tmem_ld_32x32b_x32(lane_addr + b * BT + c0, r);
      tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < 32; j += 4) {
        const float4 sx = *reinterpret_cast<const float4*>(xs + c0 + j);  // same address for the whole warp
        total[c0 + j] = fmaf(__uint_as_float(r[j]), sw * sx.x, total[c0 + j]);
        total[c0 + j + 1] = fmaf(__uint_as_float(r[j + 1]), sw * sx.y, total[c0 + j + 1]);
        total[c0 + j + 2] = fmaf(__uint_as_float(r[j + 2]), sw * sx.z, total[c0 + j + 2]);
        total[c0 + j + 3] = fmaf(__uint_as_float(r[j + 3]), sw * sx.w, total[c0 + j + 3]);
      }
    }
    tcgen05_fence_before_sync();
    __syncwarp();
    if (lane == 0) {
      mbar_arrive(&acc_empty[b]);  // the accumulator may be overwritten
      mbar_arrive(&empty_bar[s]);  // the stage's scales have been read
    }
  }
  // totals -> tensor memory (accumulator 0; each warp only ever touches its own 32 lanes), then the
  // common epilogue
#pragma unroll
  for (int c0 = 0; c0 < BT; c0 += 32) {
    uint32_t r[32];
#pragma unroll
    for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(total[c0 + j]);
    tmem_st_32x32b_x32(lane_addr + c0, r);
  }
  tmem_st_wait();
  epilogue<BT>(p, tmem_base, smem, n_tile, split, m_block);
  }

  tcgen05_fence_before_sync();
  __syncthreads();
  if (warp == 4) tmem_dealloc(tmem_base, C::kTmemCols);
}

template <int BT>
static int launch_fp8_block(const void* xq, const float* x_scale, int m_pad, const void* wq, const float* w_scale,
                            const void* bias, void* y, int64_t ldy, int M, int N, int K, void* workspace,
                            size_t workspace_bytes, cudaStream_t stream, float* partials_out = nullptr,
                            size_t partials_bytes = 0, int* splits_out = nullptr) {
  using C = BlkConfig<BT>;
  // weights: tile-major (see weight_tile_offset in quant.cuh) = a [tiles * 128 rows][128 bytes] matrix
  const uint64_t wd[2] = {128, static_cast<uint64_t>((N + kTileN - 1) / kTileN) * (K / 128) * kTileN};
  const uint64_t wst[1] = {128};
  const uint64_t ws[1] = {static_cast<uint64_t>(K)};
  const uint32_t wb[2] = {128, kTileN};
  const uint64_t xd[2] = {static_cast<uint64_t>(K), static_cast<uint64_t>(M)};
  const uint32_t xb[2] = {128, BT};
  const CUtensorMap* mw = get_tensor_map(wq, 2, wd, wst, wb, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                         CU_TENSOR_MAP_DATA_TYPE_UINT8);
  const CUtensorMap* mx = get_tensor_map(xq, 2, xd, ws, xb, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                         CU_TENSOR_MAP_DATA_TYPE_UINT8);
  if (!mw || !mx) return B200_ERR_DRIVER;
  const int n_tiles = (N + kTileN - 1) / kTileN;
  const int m_blocks = (M + BT - 1) / BT;
  const int num_kb = K / 128;
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
  BlkOperands q;
  q.w_scale = w_scale;
  q.x_scale = x_scale;
  q.k_tiles = num_kb;
  q.m_pad = m_pad;
  static std::atomic<uint64_t> smem_attr_done{0};
  if (ensure_dynamic_smem(gemm_fp8_block_kernel<BT>, C::kSmemBytes, smem_attr_done) != B200_OK) return B200_ERR_LAUNCH;
  dim3 grid(n_tiles, splits, m_blocks);
  const int rc = launch_pdl(gemm_fp8_block_kernel<BT>, grid, dim3(kBlkThreads), C::kSmemBytes, stream, *mw, *mx, p, q);
  if (rc != B200_OK || splits == 1 || p.keep_partials) return rc;
  return launch_splitk_reduce(p, stream);
}

// Token block per CTA: up to 64 tokens the weight-major kernel above; 128 and 256 tokens the token-major kernel of
// gemm_fp8_block_tok.cu.
static int pick_bt_block(int M) { return M <= 32 ? 32 : (M <= 64 ? 64 : (M <= 128 ? 128 : 256)); }

}  // namespace gemm
}  // namespace b200

#include "gemm_fp8_block_tok.cu"
#include "gemm_fp8_block_pair.cu"

extern "C" {

int b200_set_fp8_block_cta_pairs(int enable) {
  b200::gemm::g_fp8_block_cta_pairs.store(enable != 0 ? 1 : 0, std::memory_order_relaxed);
  return B200_OK;
}

size_t b200_gemm_fp8_block_splitk_bytes(int M, int N, int K) {
  using namespace b200::gemm;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  const int bt = pick_bt_block(M);
  const int tiles = ((N + kTileN - 1) / kTileN) * ((M + bt - 1) / bt);
  return static_cast<size_t>(choose_splits(tiles, K / 128, bt >= 128 ? 1 : 0)) * M * N * sizeof(float);
}

int b200_gemm_fp8_block_splitk(const void* xq, const float* x_scale, int m_pad, const void* wq, const float* w_scale,
                               int M, int N, int K, float* partials, size_t partials_bytes, int* num_splits,
                               b200_stream_t stream) {
  using namespace b200;
  if (!xq || !x_scale || !wq || !w_scale || !partials || !num_splits || M <= 0 || N <= 0 || K <= 0)
    return B200_ERR_INVALID_ARGUMENT;
  if (K % 128 != 0 || m_pad < M || m_pad % 4 != 0) return B200_ERR_ALIGNMENT;
  if (!aligned16(xq) || !aligned16(wq) || !aligned16(x_scale) || !aligned16(partials)) return B200_ERR_ALIGNMENT;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (gemm::fp8_block_pair_applicable(M, N))
    return gemm::launch_fp8_block_pair(xq, x_scale, m_pad, wq, w_scale, nullptr, nullptr, N, M, N, K, nullptr, 0, s, partials,
                                       partials_bytes, num_splits);
  switch (gemm::pick_bt_block(M)) {
    case 32:
      return gemm::launch_fp8_block<32>(xq, x_scale, m_pad, wq, w_scale, nullptr, nullptr, N, M, N, K, nullptr, 0, s, partials, partials_bytes, num_splits);
    case 64:
      return gemm::launch_fp8_block<64>(xq, x_scale, m_pad, wq, w_scale, nullptr, nullptr, N, M, N, K, nullptr, 0, s, partials, partials_bytes, num_splits);
    case 128:
      return gemm::launch_fp8_block_tok<1>(xq, x_scale, m_pad, wq, w_scale, nullptr, nullptr, N, M, N, K, nullptr, 0, s, partials, partials_bytes, num_splits);
    default:
      return gemm::launch_fp8_block_tok<2>(xq, x_scale, m_pad, wq, w_scale, nullptr, nullptr, N, M, N, K, nullptr, 0, s, partials, partials_bytes, num_splits);
  }
}

size_t b200_gemm_fp8_block_workspace_bytes(int M, int N, int K) {
  using namespace b200::gemm;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  const int bt = pick_bt_block(M);
  const int tiles = ((N + kTileN - 1) / kTileN) * ((M + bt - 1) / bt);
  const int splits = choose_splits(tiles, K / 128, bt >= 128 ? 1 : 0);
  if (splits == 1) return 0;
  return static_cast<size_t>(splits) * static_cast<size_t>(M) * N * sizeof(float);
}

int b200_gemm_fp8_block(const void* xq, const float* x_scale, int m_pad, const void* wq, const float* w_scale,
                        const void* bias, void* y, int64_t ldy, int M, int N, int K, void* workspace,
                        size_t workspace_bytes, b200_stream_t stream) {
  using namespace b200;
  if (!xq || !x_scale || !wq || !w_scale || !y || M <= 0 || N <= 0 || K <= 0) return B200_ERR_INVALID_ARGUMENT;
  if (K % 128 != 0 || ldy < N || m_pad < M || m_pad % 4 != 0) return B200_ERR_ALIGNMENT;
  if (!aligned16(xq) || !aligned16(wq) || !aligned16(x_scale)) return B200_ERR_ALIGNMENT;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (gemm::fp8_block_pair_applicable(M, N))
    return gemm::launch_fp8_block_pair(xq, x_scale, m_pad, wq, w_scale, bias, y, ldy, M, N, K, workspace, workspace_bytes, s,
                                       nullptr, 0, nullptr);
  switch (gemm::pick_bt_block(M)) {
    case 32:
      return gemm::launch_fp8_block<32>(xq, x_scale, m_pad, wq, w_scale, bias, y, ldy, M, N, K, workspace, workspace_bytes, s);
    case 64:
      return gemm::launch_fp8_block<64>(xq, x_scale, m_pad, wq, w_scale, bias, y, ldy, M, N, K, workspace, workspace_bytes, s);
    case 128:
      return gemm::launch_fp8_block_tok<1>(xq, x_scale, m_pad, wq, w_scale, bias, y, ldy, M, N, K, workspace, workspace_bytes, s, nullptr, 0, nullptr);
    default:
      return gemm::launch_fp8_block_tok<2>(xq, x_scale, m_pad, wq, w_scale, bias, y, ldy, M, N, K, workspace, workspace_bytes, s, nullptr, 0, nullptr);
  }
}

}  // extern "C"
