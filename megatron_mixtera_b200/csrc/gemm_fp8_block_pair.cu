// Block-scaled FP8 GEMM (fp32 scales: 128 x 128 weight blocks, 1 x 128 token blocks) for a 256-token block, as a PAIR
// of CTAs on two SMs that issue one tcgen05.mma.cta_group::2 per K step.
//
// Why: the single-CTA kernel (gemm_fp8_block_tok.cu, 256 tokens x 128 weight rows per CTA) stages 32 KB of tokens and
// 16 KB of weights per K block, so the SMs take in three times the weight bytes - and an SM takes in only ~60 GB/s.
// Here the output tile is 256 tokens x 256 weight rows per CTA pair:
//   CTA r of the pair stages ITS 128 tokens (A operand, 16 KB per K block) and ITS 128 of the 256 weight rows (its half
//   of the B operand, 16 KB); the pair's MMA (M = 256, N = 256, K = 32) reads A from each CTA's own shared memory and B
//   from both, and leaves the 128 x 256 fp32 accumulator of CTA r's tokens in CTA r's tensor memory.
// Per CTA that is 32 KB per K block for 128 x 256 outputs instead of 48 KB for 256 x 128: two times the weight bytes
// through the L2 -> SM path instead of three, and no multicast load is needed for it.
//
//   warps 0 .. 7 : promoters - one token per thread (lane quadrant w % 4), 128 of the 256 features (column half w / 4):
//                  tcgen05.ld the K block's accumulator, total += acc * (w_scale * x_scale[token]) - one FFMA per element
//   warp 8, lane 0 : producer - per stage the CTA's token tile and weight tile (TMA, 128-byte swizzle); both CTAs'
//                    copies complete on the LEADER's (cluster rank 0) full barrier, which expects the bytes of both
//   warp 9, lane 0, leader only : 4 x tcgen05.mma.cta_group::2 kind::f8f6f4 per K block into one of two accumulator
//                    buffers (2 x 256 columns = all of tensor memory), then commits to the stage's empty barrier and the
//                    buffer's full barrier of BOTH CTAs
// The promoters of both CTAs release an accumulator buffer by arriving on the leader's barrier (remote arrive from the
// peer).  Token scales are read from global memory by the promoters (one float per thread per K block, a K block ahead).
// Every wait is bounded; the two CTAs meet at a cluster barrier after set-up and before tensor memory is freed, so
// neither leaves while the other can still touch its shared or tensor memory.
#include "common.cuh"

namespace b200 {
namespace gemm {

__device__ __forceinline__ uint32_t cluster_cta_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_barrier() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared::cluster address of the same shared-memory location in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t cluster_addr_of(const void* smem_ptr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_u32(smem_ptr)), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// TMA tile load of one CTA of a pair whose completion bytes are counted on a barrier given by its shared::cluster
// address (the leader's).  No multicast: the tile lands in the executing CTA's shared memory only.
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* m, uint32_t bar_cluster_addr, int32_t x,
                                                 int32_t y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar_cluster_addr), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* slot, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(slot)), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish_alloc_permit_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void umma_f8_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                             uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(tmem_d),
      "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// arrive (once the pair's MMAs issued so far have completed) on the barrier at a shared::cluster address
__device__ __forceinline__ void umma_commit_pair(uint32_t bar_cluster_addr) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_cluster_addr) : "memory");
}

struct PairTileConfig {
  static constexpr int kTokensPerCta = 128;
  static constexpr int kPromoterWarps = 8;
  static constexpr int kThreads = (kPromoterWarps + 2) * 32;
  static constexpr int kStageBytesX = kTokensPerCta * 128;
  static constexpr int kOffW = kStageBytesX;
  static constexpr int kStageBytes = kStageBytesX + kTileN * 128;  // 32 KB
  static constexpr int kStages = 6;
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024 + 256;
  static constexpr int kTmemCols = 512;  // two buffers of 256 feature columns
};

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(PairTileConfig::kThreads, 1)
gemm_fp8_block_pair_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, Params p,
                           BlkOperands q) {
  using C = PairTileConfig;
  extern __shared__ uint8_t smem_raw[];
  // (the dynamic shared memory of both CTAs starts at the same offset, so every carve-up below is at the same offset in
  // both: the pair's MMA and the remote arrives rely on that)
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + C::kStages * C::kStageBytes);  // used in the leader only
  uint64_t* empty_bar = full_bar + C::kStages;
  uint64_t* acc_full = empty_bar + C::kStages;
  uint64_t* acc_empty = acc_full + 2;                                                    // used in the leader only
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const uint32_t rank = cluster_cta_rank();          // 0 = leader
  const int n_tile = blockIdx.x;                      // this CTA's weight tile: 2 * pair + rank
  const int split = blockIdx.y;
  const int m0 = blockIdx.z * 256 + static_cast<int>(rank) * C::kTokensPerCta;  // this CTA's first token
  const int kb_begin = split * p.k_blocks_per_split;
  const int kb_end = min(p.num_k_blocks, kb_begin + p.k_blocks_per_split);
  const int num_kb = kb_end - kb_begin;
  constexpr int kProducerWarp = C::kPromoterWarps, kMmaWarp = C::kPromoterWarps + 1;

  if (tid == 0) {
    for (int s = 0; s < C::kStages; ++s) {
      mbar_init(&full_bar[s], 1);   // the leader's producer (it expects the bytes of both CTAs)
      mbar_init(&empty_bar[s], 1);  // the MMA commit
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);                           // the MMA commit
      mbar_init(&acc_empty[b], 2 * C::kPromoterWarps);      // the promoter warps of both CTAs
    }
    *abort_flag = 0;
    fence_barrier_init();
    prefetch_tensormap(&map_w);
    prefetch_tensormap(&map_x);
  }
  if (warp == kProducerWarp) {
    tmem_alloc_pair(tmem_slot, C::kTmemCols);
    tmem_relinquish_alloc_permit_pair();
  }
  tcgen05_fence_before_sync();
  __syncthreads();
  cluster_barrier();  // both CTAs' barriers are initialised and both allocations made before anything crosses over
  tcgen05_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  pdl_launch_dependents();
  if (warp == kProducerWarp) {
    if (lane == 0) {
      // ---------------- producer (both CTAs) ----------------
      uint32_t leader_full[C::kStages];
#pragma unroll
      for (int s = 0; s < C::kStages; ++s) leader_full[s] = cluster_addr_of(&full_bar[s], 0);
      auto load_w = [&](int i, int s) {  // weights are tile-major: tile (n_tile, k block) is 128 consecutive rows
        tma_load_2d_pair(smem + s * C::kStageBytes + C::kOffW, &map_w, leader_full[s], 0,
                         (n_tile * q.k_tiles + kb_begin + i) * kTileN);
      };
      auto load_x = [&](int i, int s) {
        tma_load_2d_pair(smem + s * C::kStageBytes, &map_x, leader_full[s], (kb_begin + i) * 128, m0);
      };
      const int pre = num_kb < C::kStages ? num_kb : C::kStages;
      for (int i = 0; i < pre; ++i) {  // weights are written by no kernel: request them before the wait
        if (rank == 0) mbar_arrive_expect_tx(&full_bar[i], 2 * C::kStageBytes);
        load_w(i, i);
      }
      pdl_wait();
      for (int i = 0; i < pre; ++i) load_x(i, i);
      for (int i = pre; i < num_kb; ++i) {
        const int s = i % C::kStages;
        const uint32_t phase = (i / C::kStages) & 1;
        mbar_wait_bounded(&empty_bar[s], phase ^ 1, abort_flag, kStatusGemmTimeout);
        if (rank == 0) mbar_arrive_expect_tx(&full_bar[s], 2 * C::kStageBytes);
        load_w(i, s);
        load_x(i, s);
      }
    }
  } else if (warp == kMmaWarp) {
    if (lane == 0 && rank == 0) {
      // ------- UMMA issuer (leader): D[token, feature] = X[token, k] * W[feature, k]^T, 256 x 256 per pair -------
      constexpr uint32_t idesc = umma_idesc_f8(256, 256);
      uint32_t peer_empty[C::kStages], peer_acc_full[2];
#pragma unroll
      for (int s = 0; s < C::kStages; ++s) peer_empty[s] = cluster_addr_of(&empty_bar[s], 1);
      peer_acc_full[0] = cluster_addr_of(&acc_full[0], 1);
      peer_acc_full[1] = cluster_addr_of(&acc_full[1], 1);
      for (int i = 0; i < num_kb; ++i) {
        const int s = i % C::kStages;
        const int b = i & 1;
        mbar_wait_bounded(&full_bar[s], (i / C::kStages) & 1, abort_flag, kStatusGemmTimeout);
        mbar_wait_bounded(&acc_empty[b], ((i >> 1) & 1) ^ 1, abort_flag, kStatusGemmTimeout);
        tcgen05_fence_after_sync();
        const uint32_t stage_addr = smem_u32(smem + s * C::kStageBytes);
        const uint64_t x_desc = umma_desc_k_major_sw128(stage_addr);
        const uint64_t w_desc = umma_desc_k_major_sw128(stage_addr + C::kOffW);
#pragma unroll
        for (int k = 0; k < 4; ++k)
          umma_f8_pair(tmem_base + b * 256, x_desc + 2 * k, w_desc + 2 * k, idesc, k > 0 ? 1u : 0u);
        umma_commit_pair(smem_u32(&empty_bar[s]));
        umma_commit_pair(peer_empty[s]);
        umma_commit_pair(smem_u32(&acc_full[b]));
        umma_commit_pair(peer_acc_full[b]);
      }
    }
  } else {
    // ---------------- promoters: one token per thread, 128 of the pair's 256 feature totals in registers ----------------
    pdl_wait();
    const int quad = warp & 3;
    const int col_half = warp >> 2;
    const int tile_of_cols = (n_tile & ~1) + col_half;  // the weight tile whose features these columns are
    const int m = m0 + quad * 32 + lane;                // this thread's token
    const bool m_ok = m < p.M;
    float total[kTileN];
#pragma unroll
    for (int j = 0; j < kTileN; ++j) total[j] = 0.f;
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + col_half * 128;
    const uint32_t leader_acc_empty[2] = {cluster_addr_of(&acc_empty[0], 0), cluster_addr_of(&acc_empty[1], 0)};
    const float* w_scale = q.w_scale + static_cast<int64_t>(tile_of_cols) * q.k_tiles + kb_begin;
    const float* x_scale = q.x_scale + static_cast<int64_t>(kb_begin) * q.m_pad + m;
    float sw_next = num_kb > 0 ? __ldg(w_scale) : 0.f;
    float sx_next = (num_kb > 0 && m_ok) ? __ldcg(x_scale) : 0.f;
    for (int i = 0; i < num_kb; ++i) {
      const int b = i & 1;
      const float sc = sw_next * sx_next;
      if (i + 1 < num_kb) {
        sw_next = __ldg(w_scale + i + 1);
        sx_next = m_ok ? __ldcg(x_scale + static_cast<int64_t>(i + 1) * q.m_pad) : 0.f;
      }
      mbar_wait_bounded(&acc_full[b], (i >> 1) & 1, abort_flag, kStatusGemmTimeout);
      tcgen05_fence_after_sync();
      // 16 columns at a time, software-pipelined: the load of the next 16 is in flight while these are added
      const uint32_t acc_addr = lane_addr + b * 256;
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
      if (lane == 0) mbar_arrive_cluster(leader_acc_empty[b]);  // the accumulator half may be overwritten
    }

    // ---------------- epilogue: the thread's token row, 128 consecutive features, straight from registers ----------------
    const int n0 = tile_of_cols * kTileN;
    if (m_ok) {
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

  // Neither CTA may leave (or free tensor memory) while the other's MMA, copies or arrives can still reach it.
  tcgen05_fence_before_sync();
  __syncthreads();
  cluster_barrier();
  if (warp == kProducerWarp) tmem_dealloc_pair(tmem_base, C::kTmemCols);
}

// Whether the pair kernel takes this shape: a whole number of weight-tile pairs and more than 128 tokens.
static std::atomic<int> g_fp8_block_cta_pairs{0};

static bool fp8_block_pair_applicable(int M, int N) {
  return g_fp8_block_cta_pairs.load(std::memory_order_relaxed) != 0 && M > 128 && M <= 256 && N % (2 * kTileN) == 0;
}

static int launch_fp8_block_pair(const void* xq, const float* x_scale, int m_pad, const void* wq, const float* w_scale,
                                 const void* bias, void* y, int64_t ldy, int M, int N, int K, void* workspace,
                                 size_t workspace_bytes, cudaStream_t stream, float* partials_out, size_t partials_bytes,
                                 int* splits_out) {
  using C = PairTileConfig;
  const int n_tiles = N / kTileN;
  const uint64_t wd[2] = {128, static_cast<uint64_t>(n_tiles) * (K / 128) * kTileN};
  const uint64_t wst[1] = {128};
  const uint64_t xs[1] = {static_cast<uint64_t>(K)};
  const uint32_t wb[2] = {128, kTileN};
  const uint64_t xd[2] = {static_cast<uint64_t>(K), static_cast<uint64_t>(M)};
  const uint32_t xb[2] = {128, static_cast<uint32_t>(C::kTokensPerCta)};
  const CUtensorMap* mw = get_tensor_map(wq, 2, wd, wst, wb, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                         CU_TENSOR_MAP_DATA_TYPE_UINT8);
  const CUtensorMap* mx_ = get_tensor_map(xq, 2, xd, xs, xb, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                          CU_TENSOR_MAP_DATA_TYPE_UINT8);
  if (!mw || !mx_) return B200_ERR_DRIVER;
  const int num_kb = K / 128;
  // the same split rule as the single-CTA kernel (one CTA per weight tile and 256-token block, one CTA per SM), so the
  // *_bytes queries size the workspace for either kernel
  const int splits = choose_splits(n_tiles, num_kb, 1);
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
  if (ensure_dynamic_smem(gemm_fp8_block_pair_kernel, C::kSmemBytes, smem_attr_done) != B200_OK) return B200_ERR_LAUNCH;
  dim3 grid(n_tiles, splits, 1);  // x: weight tiles, two consecutive ones form a cluster
  const int rc = launch_pdl(gemm_fp8_block_pair_kernel, grid, dim3(C::kThreads), C::kSmemBytes, stream, *mw, *mx_, p, q);
  if (rc != B200_OK || splits == 1 || p.keep_partials) return rc;
  return launch_splitk_reduce(p, stream);
}

}  // namespace gemm
}  // namespace b200
