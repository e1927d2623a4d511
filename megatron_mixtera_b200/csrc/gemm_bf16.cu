// y[M, N] = x[M, K] * w[N, K]^T (+ bias): weight-streaming GEMM for decode on tcgen05 / TMEM.
//
// Decode has few tokens (M = 8 ... 256) and large weights, so the kernel is bound by streaming w
// from HBM once.  The roles of the two operands are swapped with respect to the usual GEMM: a tile
// of 128 weight rows is the UMMA "M" side (one TMEM lane per output feature) and the tokens are the
// UMMA "N" side (one TMEM column per token, 32 ... 256).  Each CTA owns one (128-feature tile,
// token block, K range) unit:
//
//   warp 0 / lane 0 : TMA producer  - w tile [128 x 64] and x tile [BT x 64] per stage, 128B swizzle;
//                                     the first w tiles are requested before the programmatic-launch
//                                     wait, so weight streaming overlaps the previous kernel's tail
//   warp 1 / lane 0 : UMMA issuer   - 4 x tcgen05.mma (K = 16 each) per stage, fp32 accumulate in TMEM
//   warps 0-3       : epilogue      - tcgen05.ld, then either bf16 store or split-K partial store
//
// Small N (e.g. out-proj, 32 tiles) cannot fill 148 SMs with whole-K units, so K is split across
// CTAs.  Partials go to an fp32 workspace and a second, fully parallel kernel sums them in split
// order (deterministic) and writes bf16.  (A "last CTA to arrive reduces its tile" scheme was tried
// first: correct, but the single reducing CTA cost 3 - 6 us per GEMM.)
#include "common.cuh"

namespace b200 {
namespace gemm {

constexpr int kTileN = 128;   // weight rows per CTA (UMMA M)
constexpr int kTileK = 64;    // bf16 elements per stage along K = one 128-byte swizzle row
constexpr int kUmmaK = 16;
constexpr int kThreads = 128;
constexpr int kMaxSplits = 32;

template <int BT>
struct Config {
  static constexpr int kStageBytesW = kTileN * kTileK * 2;
  static constexpr int kStageBytesX = BT * kTileK * 2;
  static constexpr int kStageBytes = kStageBytesW + kStageBytesX;
  // ~96 KiB of tiles per CTA so that two CTAs are resident per SM.
  static constexpr int kStages = (BT <= 64) ? 4 : (BT <= 128 ? 3 : 2);
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024 /*alignment slack*/ + 256 /*barriers*/;
  static constexpr int kTmemCols = BT < 32 ? 32 : BT;
};

struct Params {
  const __nv_bfloat16* bias;
  __nv_bfloat16* y;
  float* partials;      // [splits][M][N] fp32 (split-K only)
  int64_t ldy;
  int M, N, K;
  int num_k_blocks;     // ceil(K / 64)
  int k_blocks_per_split;
  int num_splits;
  int keep_partials;    // 1: fp32 partial sums are the result (even for one split); a fused consumer reduces them
  int gated;            // 1: rows 0-63 of every 128-row weight tile are gate features, rows 64-127 the matching up
                        //    features; y[M, N/2] = bf16(bf16(silu(gate)) * up) (whole-K units only)
};

// Sum of the split-K partial tiles: y[m, n] = bf16(sum_s partial[s][m][n]) (+ bias), splits added in order
// (deterministic).  One thread per four consecutive features; all CTAs of the grid work in parallel, which
// is what a single "last arriver" CTA cannot offer.
__global__ void __launch_bounds__(256)
splitk_reduce_kernel(const float* __restrict__ partials, int splits, int M, int N, const __nv_bfloat16* __restrict__ bias,
                     __nv_bfloat16* __restrict__ y, int64_t ldy) {
  pdl_launch_dependents();
  pdl_wait();
  const int64_t split_stride = static_cast<int64_t>(M) * N;
  if ((N & 3) == 0) {
    const int nq = N >> 2;
    const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx >= static_cast<int64_t>(M) * nq) return;
    const int m = static_cast<int>(idx / nq);
    const int n = static_cast<int>(idx - static_cast<int64_t>(m) * nq) * 4;
    const float* src = partials + static_cast<int64_t>(m) * N + n;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 4
    for (int s = 0; s < splits; ++s) {
      const float4 v = __ldcg(reinterpret_cast<const float4*>(src + s * split_stride));
      acc.x += v.x;
      acc.y += v.y;
      acc.z += v.z;
      acc.w += v.w;
    }
    if (bias != nullptr) {  // bias is added to the bf16-rounded product, as `matmul(x, w.t()) + bias` does
      acc.x = bf16_round(acc.x) + __bfloat162float(bias[n]);
      acc.y = bf16_round(acc.y) + __bfloat162float(bias[n + 1]);
      acc.z = bf16_round(acc.z) + __bfloat162float(bias[n + 2]);
      acc.w = bf16_round(acc.w) + __bfloat162float(bias[n + 3]);
    }
    __nv_bfloat16* dst = y + static_cast<int64_t>(m) * ldy + n;
    if ((ldy & 3) == 0) {
      *reinterpret_cast<uint2*>(dst) = make_uint2(pack_bf16x2(acc.x, acc.y), pack_bf16x2(acc.z, acc.w));
    } else {
      dst[0] = __float2bfloat16_rn(acc.x);
      dst[1] = __float2bfloat16_rn(acc.y);
      dst[2] = __float2bfloat16_rn(acc.z);
      dst[3] = __float2bfloat16_rn(acc.w);
    }
  } else {
    const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx >= split_stride) return;
    const int m = static_cast<int>(idx / N);
    const int n = static_cast<int>(idx - static_cast<int64_t>(m) * N);
    float acc = 0.f;
    for (int s = 0; s < splits; ++s) acc += __ldcg(partials + s * split_stride + idx);
    if (bias != nullptr) acc = bf16_round(acc) + __bfloat162float(bias[n]);
    y[static_cast<int64_t>(m) * ldy + n] = __float2bfloat16_rn(acc);
  }
}

static int launch_splitk_reduce(const Params& p, cudaStream_t stream) {
  const int64_t work = (p.N & 3) == 0 ? static_cast<int64_t>(p.M) * (p.N >> 2) : static_cast<int64_t>(p.M) * p.N;
  const unsigned blocks = static_cast<unsigned>((work + 255) / 256);
  return launch_pdl(splitk_reduce_kernel, dim3(blocks), dim3(256), 0, stream, static_cast<const float*>(p.partials),
                    p.num_splits, p.M, p.N, p.bias, p.y, p.ldy);
}

// Barrier over the 128 threads that run the epilogue (warps 0-3 in every GEMM kernel; some kernels have more warps).
__device__ __forceinline__ void epilogue_barrier() { asm volatile("bar.sync 2, 128;" ::: "memory"); }

// Accumulator -> output.  TMEM lane = output feature, TMEM column = token.  Either rounds to bf16 and
// stores (whole-K units), or stores the fp32 partial tile for splitk_reduce_kernel.
template <int BT>
__device__ __forceinline__ void epilogue(const Params& p, uint32_t tmem_base, uint8_t* stage_smem, int n_tile, int split,
                                         int m_block) {
  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int n0 = n_tile * kTileN;
  const int m0 = m_block * BT;
  const int n = n0 + warp * 32 + lane;          // output feature held by this thread (TMEM lane)
  const bool n_ok = n < p.N;
  const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(warp * 32) << 16);

  if (p.gated) {
    // SwiGLU in the epilogue.  Warps 0-1 hold gate features, warps 2-3 the matching up features (same lane).  Of
    // every 32 tokens the gate warps finish the first 16 and the up warps the last 16: each side parks the half it
    // does not finish in shared memory (the pipeline stages are free, every UMMA has completed).  Rounding points as
    // in the unfused path: GEMM output to bf16, silu to bf16, product to bf16.
    float* xch = reinterpret_cast<float*>(stage_smem);  // [BT tokens][64 features]
    const int f = (warp & 1) * 32 + lane;               // feature inside the 64-wide half
    const int out_col = n_tile * 64 + f;
    const bool col_ok = out_col < (p.N >> 1);
    const bool is_gate = warp < 2;
    const int own0 = is_gate ? 0 : 16;                  // tokens of the chunk this thread finishes
#pragma unroll 1
    for (int c0 = 0; c0 < BT; c0 += 32) {
      uint32_t r[32];
      tmem_ld_32x32b_x32(lane_addr + c0, r);
      tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const int jj = is_gate ? j + 16 : j;            // the other side's tokens
        xch[(c0 + jj) * 64 + f] = bf16_round(__uint_as_float(is_gate ? r[j + 16] : r[j]));
      }
      __syncthreads();
      if (col_ok) {
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const int m = m0 + c0 + own0 + j;
          if (m < p.M) {
            const float mine = bf16_round(__uint_as_float(is_gate ? r[j] : r[j + 16]));
            const float other = xch[(c0 + own0 + j) * 64 + f];
            const float g = is_gate ? mine : other;
            const float u = is_gate ? other : mine;
            const float a = bf16_round(g / (1.f + expf(-g)));
            p.y[static_cast<int64_t>(m) * p.ldy + out_col] = __float2bfloat16_rn(a * u);
          }
        }
      }
      __syncthreads();
    }
  } else if (p.num_splits == 1 && !p.keep_partials) {
    const float b = (p.bias != nullptr && n_ok) ? __bfloat162float(p.bias[n]) : 0.f;
    if (n0 + kTileN <= p.N && (p.ldy & 7) == 0 && (reinterpret_cast<uintptr_t>(p.y) & 15) == 0) {
      // Whole tile, 16-byte aligned rows: transpose through shared memory (the pipeline stages are free, every UMMA
      // has completed) so that the tile leaves as 16-byte vectors along the features - one store instruction per 8
      // outputs instead of one per output.
      __nv_bfloat16* tile = reinterpret_cast<__nv_bfloat16*>(stage_smem);  // [<= 128 tokens][128 features]
      constexpr int kRows = BT < 128 ? BT : 128;
#pragma unroll 1
      for (int h0 = 0; h0 < BT; h0 += kRows) {
#pragma unroll 1
        for (int c0 = 0; c0 < kRows; c0 += 32) {
          uint32_t r[32];
          tmem_ld_32x32b_x32(lane_addr + h0 + c0, r);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            float v = __uint_as_float(r[j]);
            if (p.bias != nullptr) v = bf16_round(v) + b;  // bias is added to the bf16-rounded product
            tile[(c0 + j) * kTileN + warp * 32 + lane] = __float2bfloat16_rn(v);
          }
        }
        epilogue_barrier();
        const uint4* tile_v = reinterpret_cast<const uint4*>(tile);
#pragma unroll 1
        for (int v = tid; v < kRows * 16; v += kThreads) {
          const int m = m0 + h0 + (v >> 4);
          if (m < p.M) *reinterpret_cast<uint4*>(p.y + static_cast<int64_t>(m) * p.ldy + n0 + (v & 15) * 8) = tile_v[v];
        }
        if (h0 + kRows < BT) epilogue_barrier();
      }
    } else {
#pragma unroll 1
      for (int c0 = 0; c0 < BT; c0 += 32) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(lane_addr + c0, r);
        tmem_ld_wait();
        if (n_ok) {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const int m = m0 + c0 + j;
            if (m < p.M) {
              float v = __uint_as_float(r[j]);
              // bias is added to the bf16-rounded product, as `matmul(x, w.t()) + bias` does
              if (p.bias != nullptr) v = bf16_round(v) + b;
              p.y[static_cast<int64_t>(m) * p.ldy + n] = __float2bfloat16_rn(v);
            }
          }
        }
      }
    }
  } else {
    float* part = p.partials + static_cast<int64_t>(split) * p.M * p.N;
    if (n0 + kTileN <= p.N && (p.N & 3) == 0) {
      // the same transposition for the fp32 partial tile: float4 stores along the features
      float* tile = reinterpret_cast<float*>(stage_smem);  // [<= 64 tokens][128 features]
      constexpr int kRows = BT < 64 ? BT : 64;
#pragma unroll 1
      for (int h0 = 0; h0 < BT; h0 += kRows) {
#pragma unroll 1
        for (int c0 = 0; c0 < kRows; c0 += 32) {
          uint32_t r[32];
          tmem_ld_32x32b_x32(lane_addr + h0 + c0, r);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) tile[(c0 + j) * kTileN + warp * 32 + lane] = __uint_as_float(r[j]);
        }
        epilogue_barrier();
        const float4* tile_v = reinterpret_cast<const float4*>(tile);
#pragma unroll 1
        for (int v = tid; v < kRows * 32; v += kThreads) {
          const int m = m0 + h0 + (v >> 5);
          if (m < p.M) __stcg(reinterpret_cast<float4*>(part + static_cast<int64_t>(m) * p.N + n0) + (v & 31), tile_v[v]);
        }
        if (h0 + kRows < BT) epilogue_barrier();
      }
    } else {
#pragma unroll 1
      for (int c0 = 0; c0 < BT; c0 += 32) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(lane_addr + c0, r);
        tmem_ld_wait();
        if (n_ok) {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const int m = m0 + c0 + j;
            if (m < p.M) __stcg(&part[static_cast<int64_t>(m) * p.N + n], __uint_as_float(r[j]));
          }
        }
      }
    }
    // The partial tile is complete once this kernel ends; a second kernel (splitk_reduce_kernel, or the fused consumer)
    // sums the splits of every output element in split order.
  }
}

template <int BT>
__global__ void __launch_bounds__(kThreads, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, Params p) {
  using C = Config<BT>;
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

  pdl_launch_dependents();
  if (warp == 0) {
    if (lane == 0) {
      // ---------------- TMA producer ----------------
      // The weights are written by no kernel, so their first tiles are requested before waiting
      // for the previous kernel on the stream; the activations (its output) only afterwards.
      const int pre = num_kb < C::kStages ? num_kb : C::kStages;
      for (int i = 0; i < pre; ++i) {
        mbar_arrive_expect_tx(&full_bar[i], C::kStageBytes);
        tma_load_2d(smem + i * C::kStageBytes, &map_w, &full_bar[i], (kb_begin + i) * kTileK, n0);
      }
      pdl_wait();
      for (int i = 0; i < pre; ++i)
        tma_load_2d(smem + i * C::kStageBytes + C::kStageBytesW, &map_x, &full_bar[i], (kb_begin + i) * kTileK, m0);
      for (int i = pre; i < num_kb; ++i) {
        const int s = i % C::kStages;
        const uint32_t phase = (i / C::kStages) & 1;
        mbar_wait_bounded(&empty_bar[s], phase ^ 1, abort_flag, kStatusGemmTimeout);
        uint8_t* stage = smem + s * C::kStageBytes;
        mbar_arrive_expect_tx(&full_bar[s], C::kStageBytes);
        const int k0 = (kb_begin + i) * kTileK;
        tma_load_2d(stage, &map_w, &full_bar[s], k0, n0);
        tma_load_2d(stage + C::kStageBytesW, &map_x, &full_bar[s], k0, m0);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0) {
      // ---------------- UMMA issuer ----------------
      constexpr uint32_t idesc = umma_idesc_bf16(kTileN, BT < 16 ? 16 : BT);
      for (int i = 0; i < num_kb; ++i) {
        const int s = i % C::kStages;
        const uint32_t phase = (i / C::kStages) & 1;
        mbar_wait_bounded(&full_bar[s], phase, abort_flag, kStatusGemmTimeout);
        tcgen05_fence_after_sync();
        const uint32_t a_addr = smem_u32(smem + s * C::kStageBytes);
        const uint32_t b_addr = a_addr + C::kStageBytesW;
        const uint64_t a_desc = umma_desc_k_major_sw128(a_addr);
        const uint64_t b_desc = umma_desc_k_major_sw128(b_addr);
#pragma unroll
        for (int k = 0; k < kTileK / kUmmaK; ++k) {
          // 32 bytes per K step inside the 128-byte swizzle row -> +2 in the encoded start address
          umma_f16(tmem_base, a_desc + 2 * k, b_desc + 2 * k, idesc, (i > 0 || k > 0) ? 1u : 0u);
        }
        umma_commit(&empty_bar[s]);  // frees the stage when these UMMAs have read it
      }
      umma_commit(accum_bar);        // accumulator complete
    }
    __syncwarp();
  }

  // ---------------- epilogue: all four warps ----------------
  pdl_wait();  // outputs and partial sums may still be in use by the previous kernel until here
  mbar_wait_bounded(accum_bar, 0, abort_flag, kStatusGemmTimeout);
  tcgen05_fence_after_sync();

  epilogue<BT>(p, tmem_base, smem, n_tile, split, m_block);

  tcgen05_fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem_base, C::kTmemCols);
}

// Number of K splits: fill `ctas_per_sm` CTAs per SM when there are too few output tiles, keep at least
// `min_k_blocks` K blocks per split, never more than `max_splits`.  The three numbers are a tuning policy that
// the host may change (b200_set_gemm_split_policy); it must not change between a b200_gemm_*_bytes query and the
// launch it sizes.
static std::atomic<int> g_split_ctas_per_sm{2}, g_split_min_k_blocks{4}, g_split_max{kMaxSplits};

// `resident_ctas_per_sm`: 0 = the policy's value; a kernel of which only one CTA fits an SM passes 1.
static int choose_splits(int tiles, int num_k_blocks, int resident_ctas_per_sm = 0) {
  const int per_sm = resident_ctas_per_sm > 0 ? resident_ctas_per_sm : g_split_ctas_per_sm.load(std::memory_order_relaxed);
  const int slots = per_sm * sm_count();
  const int min_kb = g_split_min_k_blocks.load(std::memory_order_relaxed);
  if (tiles * 2 > slots) return 1;
  int s = slots / tiles;
  const int cap = g_split_max.load(std::memory_order_relaxed);
  if (s > cap) s = cap;
  if (s > num_k_blocks / min_kb) s = num_k_blocks / min_kb;
  if (s < 1) s = 1;
  // drop empty trailing splits
  const int per = (num_k_blocks + s - 1) / s;
  s = (num_k_blocks + per - 1) / per;
  return s;
}

static int pick_bt(int M) {
  if (M <= 32) return 32;
  if (M <= 64) return 64;
  if (M <= 128) return 128;
  return 256;
}

template <int BT>
static int launch(const void* x, int64_t ldx, const void* w, const void* bias, void* y, int64_t ldy, int M, int N,
                  int K, void* workspace, size_t workspace_bytes, cudaStream_t stream, bool cache_maps = true,
                  float* partials_out = nullptr, size_t partials_bytes = 0, int* splits_out = nullptr,
                  bool gated = false) {
  using C = Config<BT>;
  const uint64_t wd[2] = {static_cast<uint64_t>(K), static_cast<uint64_t>(N)};
  const uint64_t ws[1] = {static_cast<uint64_t>(K) * 2};
  const uint32_t wb[2] = {kTileK, kTileN};
  const uint64_t xd[2] = {static_cast<uint64_t>(K), static_cast<uint64_t>(M)};
  const uint64_t xs[1] = {static_cast<uint64_t>(ldx) * 2};
  const uint32_t xb[2] = {kTileK, BT};
  CUtensorMap local_w, local_x;  // used when the descriptor cache (a host allocation) must be avoided
  const CUtensorMap* mw = &local_w;
  const CUtensorMap* mx = &local_x;
  if (cache_maps) {
    mw = get_tensor_map(w, 2, wd, ws, wb, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B);
    mx = get_tensor_map(x, 2, xd, xs, xb, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B);
    if (!mw || !mx) return B200_ERR_DRIVER;
  } else if (!encode_tensor_map(&local_w, w, 2, wd, ws, wb, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B) ||
             !encode_tensor_map(&local_x, x, 2, xd, xs, xb, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B)) {
    return B200_ERR_DRIVER;
  }

  const int n_tiles = (N + kTileN - 1) / kTileN;
  const int m_blocks = (M + BT - 1) / BT;
  const int num_kb = (K + kTileK - 1) / kTileK;
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
  p.gated = gated ? 1 : 0;
  if (gated && (splits != 1 || partials_out != nullptr)) return B200_ERR_INVALID_ARGUMENT;
  if (partials_out != nullptr) {
    if (partials_bytes < static_cast<size_t>(splits) * M * N * sizeof(float)) return B200_ERR_WORKSPACE;
    p.partials = partials_out;
    *splits_out = splits;
  } else if (splits > 1) {
    const size_t need = static_cast<size_t>(splits) * M * N * sizeof(float);
    if (workspace == nullptr || workspace_bytes < need || !aligned16(workspace)) return B200_ERR_WORKSPACE;
    p.partials = static_cast<float*>(workspace);
  }
  static std::atomic<uint64_t> smem_attr_done{0};
  if (ensure_dynamic_smem(gemm_bf16_kernel<BT>, C::kSmemBytes, smem_attr_done) != B200_OK) return B200_ERR_LAUNCH;
  dim3 grid(n_tiles, splits, m_blocks);
  const int rc = launch_pdl(gemm_bf16_kernel<BT>, grid, dim3(kThreads), C::kSmemBytes, stream, *mw, *mx, p);
  if (rc != B200_OK || splits == 1 || p.keep_partials) return rc;
  return launch_splitk_reduce(p, stream);
}

}  // namespace gemm
}  // namespace b200

extern "C" {

int b200_set_gemm_split_policy(int ctas_per_sm, int min_k_blocks_per_split, int max_splits) {
  using namespace b200::gemm;
  if (ctas_per_sm < 1 || ctas_per_sm > 4 || min_k_blocks_per_split < 1 || max_splits < 1 || max_splits > kMaxSplits)
    return B200_ERR_INVALID_ARGUMENT;
  g_split_ctas_per_sm.store(ctas_per_sm, std::memory_order_relaxed);
  g_split_min_k_blocks.store(min_k_blocks_per_split, std::memory_order_relaxed);
  g_split_max.store(max_splits, std::memory_order_relaxed);
  return B200_OK;
}

int b200_gemm_bf16_swiglu_supported(int M, int N, int K) {
  using namespace b200::gemm;
  if (M <= 0 || N <= 0 || K <= 0 || N % 128 != 0 || K % 8 != 0) return 0;
  const int bt = pick_bt(M);
  const int tiles = (N / kTileN) * ((M + bt - 1) / bt);
  return choose_splits(tiles, (K + kTileK - 1) / kTileK) == 1 ? 1 : 0;
}

int b200_gemm_bf16_swiglu(const void* x, int64_t ldx, const void* w, void* y, int64_t ldy, int M, int N, int K,
                          b200_stream_t stream) {
  using namespace b200;
  if (!x || !w || !y || M <= 0 || N <= 0 || K <= 0) return B200_ERR_INVALID_ARGUMENT;
  if (K % 8 != 0 || ldx % 8 != 0 || ldx < K || N % 128 != 0 || ldy < N / 2) return B200_ERR_ALIGNMENT;
  if (!aligned16(x) || !aligned16(w)) return B200_ERR_ALIGNMENT;
  if (!b200_gemm_bf16_swiglu_supported(M, N, K)) return B200_ERR_INVALID_ARGUMENT;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  switch (gemm::pick_bt(M)) {
    case 32: return gemm::launch<32>(x, ldx, w, nullptr, y, ldy, M, N, K, nullptr, 0, s, true, nullptr, 0, nullptr, true);
    case 64: return gemm::launch<64>(x, ldx, w, nullptr, y, ldy, M, N, K, nullptr, 0, s, true, nullptr, 0, nullptr, true);
    case 128: return gemm::launch<128>(x, ldx, w, nullptr, y, ldy, M, N, K, nullptr, 0, s, true, nullptr, 0, nullptr, true);
    default: return gemm::launch<256>(x, ldx, w, nullptr, y, ldy, M, N, K, nullptr, 0, s, true, nullptr, 0, nullptr, true);
  }
}

size_t b200_gemm_bf16_splitk_bytes(int M, int N, int K) {
  using namespace b200::gemm;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  const int bt = pick_bt(M);
  const int tiles = ((N + kTileN - 1) / kTileN) * ((M + bt - 1) / bt);
  return static_cast<size_t>(choose_splits(tiles, (K + kTileK - 1) / kTileK)) * M * N * sizeof(float);
}

int b200_gemm_bf16_splitk(const void* x, int64_t ldx, const void* w, int M, int N, int K, float* partials,
                          size_t partials_bytes, int* num_splits, b200_stream_t stream) {
  using namespace b200;
  if (!x || !w || !partials || !num_splits || M <= 0 || N <= 0 || K <= 0) return B200_ERR_INVALID_ARGUMENT;
  if (K % 8 != 0 || ldx % 8 != 0 || ldx < K) return B200_ERR_ALIGNMENT;
  if (!aligned16(x) || !aligned16(w) || !aligned16(partials)) return B200_ERR_ALIGNMENT;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  switch (gemm::pick_bt(M)) {
    case 32: return gemm::launch<32>(x, ldx, w, nullptr, nullptr, N, M, N, K, nullptr, 0, s, true, partials, partials_bytes, num_splits);
    case 64: return gemm::launch<64>(x, ldx, w, nullptr, nullptr, N, M, N, K, nullptr, 0, s, true, partials, partials_bytes, num_splits);
    case 128: return gemm::launch<128>(x, ldx, w, nullptr, nullptr, N, M, N, K, nullptr, 0, s, true, partials, partials_bytes, num_splits);
    default: return gemm::launch<256>(x, ldx, w, nullptr, nullptr, N, M, N, K, nullptr, 0, s, true, partials, partials_bytes, num_splits);
  }
}

size_t b200_gemm_bf16_workspace_bytes(int M, int N, int K) {
  using namespace b200::gemm;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  const int bt = pick_bt(M);
  const int tiles = ((N + kTileN - 1) / kTileN) * ((M + bt - 1) / bt);
  const int splits = choose_splits(tiles, (K + kTileK - 1) / kTileK);
  if (splits == 1) return 0;
  return static_cast<size_t>(splits) * static_cast<size_t>(M) * N * sizeof(float);
}

int b200_gemm_bf16(const void* x, int64_t ldx, const void* w, const void* bias, void* y, int64_t ldy, int M, int N,
                   int K, void* workspace, size_t workspace_bytes, b200_stream_t stream) {
  using namespace b200;
  if (!x || !w || !y || M <= 0 || N <= 0 || K <= 0) return B200_ERR_INVALID_ARGUMENT;
  if (K % 8 != 0 || ldx % 8 != 0 || ldx < K || ldy < N) return B200_ERR_ALIGNMENT;
  if (!aligned16(x) || !aligned16(w)) return B200_ERR_ALIGNMENT;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  switch (gemm::pick_bt(M)) {
    case 32: return gemm::launch<32>(x, ldx, w, bias, y, ldy, M, N, K, workspace, workspace_bytes, s);
    case 64: return gemm::launch<64>(x, ldx, w, bias, y, ldy, M, N, K, workspace, workspace_bytes, s);
    case 128: return gemm::launch<128>(x, ldx, w, bias, y, ldy, M, N, K, workspace, workspace_bytes, s);
    default: return gemm::launch<256>(x, ldx, w, bias, y, ldy, M, N, K, workspace, workspace_bytes, s);
  }
}

}  // extern "C"

// =============================================================================================
// GEMM for callers that must not allocate device memory.
//
// Some hosts of this library cannot call cudaMalloc at the point where they need a GEMM: a
// latency-critical serving loop that must not take the allocator's locks or its implicit
// synchronisation, a server that has handed the whole device to a memory pool of its own, or a
// plugin that only receives input and output pointers from its framework.  For them the split-K scratch (the fp32 partial sums)
// lives in the fixed array below instead of a caller workspace.  Every GPU that loads the library
// pays for the array once, until the process exits.
// =============================================================================================
namespace b200 {
namespace gemm {

constexpr size_t kStaticScratchBytes = 16u << 20;  // 16 MiB of partial sums
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

// `g_static_scratch` is a device symbol: in host code its name is only a handle, so the device
// address is looked up once per device (with that device current) and cached.
// Two host threads that make the first call on a device at the same time both look the address up and
// store the same value (the slots are atomic), so no ordering is needed between them.
static void* static_scratch_address() {
  static std::atomic<void*> addr[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  void* p = addr[dev].load(std::memory_order_acquire);
  if (p == nullptr) {
    if (cudaGetSymbolAddress(&p, g_static_scratch) != cudaSuccess) {
      (void)cudaGetLastError();
      return nullptr;
    }
    addr[dev].store(p, std::memory_order_release);
  }
  return p;
}

}  // namespace gemm
}  // namespace b200

extern "C" {

size_t b200_gemm_bf16_static_scratch_limit(void) { return b200::gemm::kStaticScratchBytes; }

int b200_gemm_bf16_static_scratch(const void* x, int64_t ldx, const void* w, const void* bias, void* y, int64_t ldy,
                                  int M, int N, int K, b200_stream_t stream) {
  using namespace b200;
  if (!x || !w || !y || M <= 0 || N <= 0 || K <= 0) return B200_ERR_INVALID_ARGUMENT;
  if (K % 8 != 0 || ldx % 8 != 0 || ldx < K || ldy < N) return B200_ERR_ALIGNMENT;
  if (!aligned16(x) || !aligned16(w)) return B200_ERR_ALIGNMENT;
  const size_t need = b200_gemm_bf16_workspace_bytes(M, N, K);
  if (need > gemm::kStaticScratchBytes) return B200_ERR_SCRATCH_LIMIT;
  void* scratch = gemm::static_scratch_address();
  if (scratch == nullptr) return B200_ERR_LAUNCH;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  // Nothing in the array has to start at zero: the partial sums of a call are completely written by the
  // GEMM kernel before the reduction kernel of the same call reads them.
  const size_t bytes = gemm::kStaticScratchBytes;
  switch (gemm::pick_bt(M)) {
    case 32: return gemm::launch<32>(x, ldx, w, bias, y, ldy, M, N, K, scratch, bytes, s, false);
    case 64: return gemm::launch<64>(x, ldx, w, bias, y, ldy, M, N, K, scratch, bytes, s, false);
    case 128: return gemm::launch<128>(x, ldx, w, bias, y, ldy, M, N, K, scratch, bytes, s, false);
    default: return gemm::launch<256>(x, ldx, w, bias, y, ldy, M, N, K, scratch, bytes, s, false);
  }
}

}  // extern "C"
