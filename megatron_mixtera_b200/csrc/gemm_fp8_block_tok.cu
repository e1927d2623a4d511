// Block-scaled FP8 GEMM (fp32 scales: 128 x 128 weight blocks, 1 x 128 token blocks) for token blocks of 128 and 256:
// the 70B configuration's batch.  Same arithmetic as gemm_fp8_block.cu, other orientation.
//
// Here the TOKENS are the UMMA "M" side (one TMEM lane per token, 128 per MMA, two MMAs for 256 tokens) and the 128
// weight rows of the CTA's tile are the "N" side (one TMEM column per output feature).  What that buys:
//   * a promoter thread owns ONE token, so the token scale of a K block is one scalar per thread and the promotion is
//     one FFMA per accumulator element (the weight-major form needs a multiply and a shared-memory read per element
//     on top, and was 5 x off the weight-streaming time at 256 tokens);
//   * a thread ends up with 128 consecutive output features of its token: the epilogue stores 16-byte vectors
//     straight from registers, no tensor-memory write-back, no transposition;
//   * 256 tokens share every weight tile: each weight byte crosses from HBM once per 256 tokens.
//
//   warps 0 .. 4H-1 : promoters (H = 1 or 2 halves of 128 tokens; warp w: lane quadrant w % 4 of half w / 4)
//   warp 4H, lane 0 : producer - per stage (= one K block) the token tile [H * 128 x 128 B], the weight tile
//                     [128 x 128 B, tile-major] (TMA, 128-byte swizzle) and the tokens' scales (bulk copy)
//   warp 4H+1, lane 0 : UMMA   - 4 x tcgen05.mma kind::f8f6f4 per half into one of two accumulator buffers
#include "common.cuh"

namespace b200 {
namespace gemm {

__device__ __forceinline__ void tmem_ld_32x32b_x16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}

template <int H>
struct TokConfig {
  static constexpr int kTokens = H * 128;
  static constexpr int kPromoterWarps = 4 * H;
  static constexpr int kThreads = (kPromoterWarps + 2) * 32;
  static constexpr int kStageBytesX = kTokens * 128;
  static constexpr int kOffW = kStageBytesX;
  static constexpr int kOffScale = kOffW + kTileN * 128;
  static constexpr int kStageBytes = (kOffScale + kTokens * 4 + 1023) / 1024 * 1024;
  static constexpr int kStages = 4;
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024 + 256;
  static constexpr int kTmemCols = 2 * H * 128;  // two buffers of H accumulators, 128 feature columns each
};

template <int H>
__global__ void __launch_bounds__(TokConfig<H>::kThreads, 1)
gemm_fp8_block_tok_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, Params p,
                          BlkOperands q) {
  using C = TokConfig<H>;
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
  const int m0 = m_block * C::kTokens;
  const int kb_begin = split * p.k_blocks_per_split;
  const int kb_end = min(p.num_k_blocks, kb_begin + p.k_blocks_per_split);
  const int num_kb = kb_end - kb_begin;
  // token scales of this CTA's rows that exist (a multiple of 4 floats = 16 bytes by construction of m_pad)
  const int scale_floats = min(C::kTokens, q.m_pad - m0);
  const uint32_t tx_bytes = C::kOffScale + scale_floats * 4;
  constexpr int kProducerWarp = C::kPromoterWarps, kMmaWarp = C::kPromoterWarps + 1;

  if (tid == 0) {
    for (int s = 0; s < C::kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1 + C::kPromoterWarps);  // the UMMA commit + the promoter warps (they read the scales)
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], C::kPromoterWarps);
    }
    *abort_flag = 0;
    fence_barrier_init();
    prefetch_tensormap(&map_w);
    prefetch_tensormap(&map_x);
  }
  if (warp == kProducerWarp) {
    tmem_alloc(tmem_slot, C::kTmemCols);
    tmem_relinquish_alloc_permit();
  }
  tcgen05_fence_before_sync();
  __syncthreads();
  tcgen05_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  pdl_launch_dependents();
  if (warp == kProducerWarp) {
    if (lane == 0) {
      // ---------------- producer ----------------
      auto load_w = [&](int i, int s) {  // weights are tile-major: tile (n_tile, k block) is 128 consecutive rows
        tma_load_2d(smem + s * C::kStageBytes + C::kOffW, &map_w, &full_bar[s], 0, (n_tile * q.k_tiles + kb_begin + i) * kTileN);
      };
      auto load_x = [&](int i, int s) {
        uint8_t* stage = smem + s * C::kStageBytes;
        tma_load_2d(stage, &map_x, &full_bar[s], (kb_begin + i) * 128, m0);
        bulk_load_1d(stage + C::kOffScale, q.x_scale + static_cast<int64_t>(kb_begin + i) * q.m_pad + m0, scale_floats * 4,
                     &full_bar[s]);
      };
      const int pre = num_kb < C::kStages ? num_kb : C::kStages;
      for (int i = 0; i < pre; ++i) {  // weights are written by no kernel: request them before the wait
        mbar_arrive_expect_tx(&full_bar[i], tx_bytes);
        load_w(i, i);
      }
      pdl_wait();
      for (int i = 0; i < pre; ++i) load_x(i, i);
      for (int i = pre; i < num_kb; ++i) {
        const int s = i % C::kStages;
        const uint32_t phase = (i / C::kStages) & 1;
        mbar_wait_bounded(&empty_bar[s], phase ^ 1, abort_flag, kStatusGemmTimeout);
        mbar_arrive_expect_tx(&full_bar[s], tx_bytes);
        load_w(i, s);
        load_x(i, s);
      }
    }
  } else if (warp == kMmaWarp) {
    if (lane == 0) {
      // ---------------- UMMA issuer: D[token, feature] = X[token, k] * W[feature, k]^T ----------------
      constexpr uint32_t idesc = umma_idesc_f8(128, kTileN);
      for (int i = 0; i < num_kb; ++i) {
        const int s = i % C::kStages;
        const int b = i & 1;
        mbar_wait_bounded(&full_bar[s], (i / C::kStages) & 1, abort_flag, kStatusGemmTimeout);
        mbar_wait_bounded(&acc_empty[b], ((i >> 1) & 1) ^ 1, abort_flag, kStatusGemmTimeout);
        tcgen05_fence_after_sync();
        const uint32_t stage_addr = smem_u32(smem + s * C::kStageBytes);
        const uint64_t w_desc = umma_desc_k_major_sw128(stage_addr + C::kOffW);
#pragma unroll
        for (int h = 0; h < H; ++h) {
          const uint64_t x_desc = umma_desc_k_major_sw128(stage_addr + h * 128 * 128);
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_f8(tmem_base + (b * H + h) * 128, x_desc + 2 * k, w_desc + 2 * k, idesc, k > 0 ? 1u : 0u);
        }
        umma_commit(&empty_bar[s]);
        umma_commit(&acc_full[b]);
      }
    }
  } else {
    // ---------------- promoters: one token per thread, 128 feature totals in registers ----------------
    pdl_wait();
    const int half = warp >> 2;
    const int tok = half * 128 + (warp & 3) * 32 + lane;  // token of this thread inside the CTA's block
    float total[kTileN];
#pragma unroll
    for (int j = 0; j < kTileN; ++j) total[j] = 0.f;
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>((warp & 3) * 32) << 16) + half * 128;
    const float* w_scale = q.w_scale + static_cast<int64_t>(n_tile) * q.k_tiles + kb_begin;
    float sw_next = num_kb > 0 ? __ldg(w_scale) : 0.f;
    for (int i = 0; i < num_kb; ++i) {
      const int s = i % C::kStages;
      const int b = i & 1;
      const float sw = sw_next;
      if (i + 1 < num_kb) sw_next = __ldg(w_scale + i + 1);
      mbar_wait_bounded(&acc_full[b], (i >> 1) & 1, abort_flag, kStatusGemmTimeout);
      tcgen05_fence_after_sync();
      // rows past the last token have no scale in the stage (and no output): any finite factor will do
      const float sx = tok < scale_floats ? reinterpret_cast<const float*>(smem + s * C::kStageBytes + C::kOffScale)[tok] : 0.f;
      const float sc = sw * sx;
      // 16 columns at a time, software-pipelined: the load of the next 16 is in flight while these are added
      const uint32_t acc_addr = lane_addr + b * (H * 128);
      uint32_t ra[16], rb[16];
      tmem_ld_32x32b_x16(acc_addr, ra);
      tmem_ld_wait();
#pragma unroll
      for (int c0 = 0; c0 < kTileN; c0 += 32) {
        tmem_ld_32x32b_x16(acc_addr + c0 + 16, rb);
#pragma unroll
        for (int j = 0; j < 16; ++j) total[c0 + j] = fmaf(__uint_as_float(ra[j]), sc, total[c0 + j]);
        tmem_ld_wait();
        if (c0 + 32 < kTileN) tmem_ld_32x32b_x16(acc_addr + c0 + 32, ra);
#pragma unroll
        for (int j = 0; j < 16; ++j) total[c0 + 16 + j] = fmaf(__uint_as_float(rb[j]), sc, total[c0 + 16 + j]);
        if (c0 + 32 < kTileN) tmem_ld_wait();
      }
      tcgen05_fence_before_sync();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&acc_empty[b]);  // the accumulator may be overwritten
        mbar_arrive(&empty_bar[s]);  // the stage's scales have been read
      }
    }

    // ---------------- epilogue: the thread's token row, 128 consecutive features, straight from registers ----------------
    const int m = m0 + tok;
    if (m < p.M) {
      const bool full_tile = n0 + kTileN <= p.N;
      if (p.num_splits == 1 && !p.keep_partials) {
        __nv_bfloat16* dst = p.y + static_cast<int64_t>(m) * p.ldy + n0;
        const bool vec = full_tile && (p.ldy & 7) == 0 && (reinterpret_cast<uintptr_t>(p.y) & 15) == 0;
#pragma unroll
        for (int j = 0; j < kTileN; j += 8) {
          float v[8];
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            v[k] = total[j + k];
            // bias is added to the bf16-rounded product, as `matmul(x, w.t()) + bias` does
            if (p.bias != nullptr && n0 + j + k < p.N) v[k] = bf16_round(v[k]) + __bfloat162float(p.bias[n0 + j + k]);
          }
          if (vec) {
            *reinterpret_cast<uint4*>(dst + j) = make_uint4(pack_bf16x2(v[0], v[1]), pack_bf16x2(v[2], v[3]),
                                                            pack_bf16x2(v[4], v[5]), pack_bf16x2(v[6], v[7]));
          } else {
#pragma unroll
            for (int k = 0; k < 8; ++k)
              if (n0 + j + k < p.N) dst[j + k] = __float2bfloat16_rn(v[k]);
          }
        }
      } else {
        float* dst = p.partials + (static_cast<int64_t>(split) * p.M + m) * p.N + n0;
        const bool vec = full_tile && (p.N & 3) == 0;
#pragma unroll
        for (int j = 0; j < kTileN; j += 4) {
          if (vec) {
            __stcg(reinterpret_cast<float4*>(dst + j), make_float4(total[j], total[j + 1], total[j + 2], total[j + 3]));
          } else {
#pragma unroll
            for (int k = 0; k < 4; ++k)
              if (n0 + j + k < p.N) __stcg(dst + j + k, total[j + k]);
          }
        }
      }
    }
  }

  tcgen05_fence_before_sync();
  __syncthreads();
  if (warp == kProducerWarp) tmem_dealloc(tmem_base, C::kTmemCols);
}

template <int H>
static int launch_fp8_block_tok(const void* xq, const float* x_scale, int m_pad, const void* wq, const float* w_scale,
                                const void* bias, void* y, int64_t ldy, int M, int N, int K, void* workspace,
                                size_t workspace_bytes, cudaStream_t stream, float* partials_out, size_t partials_bytes,
                                int* splits_out) {
  using C = TokConfig<H>;
  const int n_tiles = (N + kTileN - 1) / kTileN;
  const uint64_t wd[2] = {128, static_cast<uint64_t>(n_tiles) * (K / 128) * kTileN};
  const uint64_t wst[1] = {128};
  const uint64_t xs[1] = {static_cast<uint64_t>(K)};
  const uint32_t wb[2] = {128, kTileN};
  const uint64_t xd[2] = {static_cast<uint64_t>(K), static_cast<uint64_t>(M)};
  const uint32_t xb[2] = {128, static_cast<uint32_t>(C::kTokens)};
  const CUtensorMap* mw = get_tensor_map(wq, 2, wd, wst, wb, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                         CU_TENSOR_MAP_DATA_TYPE_UINT8);
  const CUtensorMap* mx_ = get_tensor_map(xq, 2, xd, xs, xb, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                          CU_TENSOR_MAP_DATA_TYPE_UINT8);
  if (!mw || !mx_) return B200_ERR_DRIVER;
  const int m_blocks = (M + C::kTokens - 1) / C::kTokens;
  const int num_kb = K / 128;
  const int splits = choose_splits(n_tiles * m_blocks, num_kb, 1);  // 200 KiB of stages / 512 TMEM columns: one CTA per SM
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
  if (ensure_dynamic_smem(gemm_fp8_block_tok_kernel<H>, C::kSmemBytes, smem_attr_done) != B200_OK) return B200_ERR_LAUNCH;
  dim3 grid(n_tiles, splits, m_blocks);
  const int rc = launch_pdl(gemm_fp8_block_tok_kernel<H>, grid, dim3(C::kThreads), C::kSmemBytes, stream, *mw, *mx_, p, q);
  if (rc != B200_OK || splits == 1 || p.keep_partials) return rc;
  return launch_splitk_reduce(p, stream);
}

}  // namespace gemm
}  // namespace b200
