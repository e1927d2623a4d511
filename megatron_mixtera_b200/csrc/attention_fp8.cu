// Paged decode attention over an FP8 (E4M3) KV pool with one fp32 scale per KV head (head dim 128).
//
// Nothing is converted: both products run on the fp8 tensor-core path (mma.sync m16n8k32 e4m3 x e4m3 -> f32).
//   S = Q K^T : the queries are split into two E4M3 terms (hi + lo, ~7 significant bits, one power-of-two scale
//               per query head) and the key bytes are the B operand exactly as ldmatrix delivers them.
//   O = P V   : P * 256 is split the same way; the B operand needs, per thread, four consecutive bytes of one
//               head dimension over four tokens, so the value pool is stored transposed inside a chunk,
//               [chunk][head][dim][token position], and within every 32 tokens the positions are permuted
//               (v_position below) to the order in which the S accumulators of a thread hold the tokens:
//               the P fragment is then built from the thread's own registers, without shuffles.
// One CTA = (row, KV head, context split) as in the 16-bit kernel; a tile is 128 tokens (K 16 KB + V^T 16 KB),
// every consumer warp takes 32 of them.  The per-tile chain ldmatrix -> mma -> softmax -> pack -> ldmatrix -> mma of the
// eight consumer warps an SM holds is latency bound, so what counts is the number of mma and exp2 per tile: with the two
// terms as separate instructions the kernel read E4M3 bytes at ~4 TB/s; stacked in one 16-row operand (kMode 2 below)
// it reads them at 6.3-6.4 TB/s, the measured HBM copy rate (32 requests x 68 k tokens, 16 context splits), twice the
// tokens per second of the 16-bit kernel.  (Two stages and three CTAs per SM were tried: registers spill, no gain.)
#include <cuda_fp8.h>

#include "common.cuh"

namespace b200 {
namespace attn8 {

constexpr int D = 128;
constexpr int kTile = 128;  // tokens per tile
constexpr int kConsumerWarps = 4;
constexpr int kConsumerThreads = kConsumerWarps * 32;
constexpr int kThreads = kConsumerThreads + 32;
constexpr int kStages = 3;
constexpr int kTileBytes = kTile * D;       // K tile [token][dim]; V tile [dim][position]: 16 KB each
constexpr int kStageBytes = 2 * kTileBytes;
constexpr int kQStride16 = D + 8;           // bf16 staging of the rotated queries
constexpr int kQ16Bytes = 16 * kQStride16 * 2;
constexpr int kQ8Stride = D + 4;            // byte rows of the E4M3 query terms, padded against bank conflicts
constexpr int kQ8Bytes = 2 * 16 * kQ8Stride + 64;
constexpr int kMergeBytes = kConsumerWarps * 16 * (D + 2) * 4;
static_assert(kMergeBytes <= kStages * kStageBytes, "merge buffers reuse the tile ring");
constexpr int kSmemBytes = kStages * kStageBytes + kQ16Bytes + 256 + kQ8Bytes + 1024;
constexpr float kPScale = 256.f;            // P is multiplied by this before the E4M3 split

// Position inside a chunk at which token `tok`'s value bytes are stored (a permutation of every 32 tokens).
// Slot 4t+e of a 16-token half holds token [2t, 2t+1, 8+2t, 9+2t][e]: what lane (., t) owns after S = Q K^T.
__host__ __device__ __forceinline__ int v_position(int tok) {
  const int v = tok & 15;
  const int slot = v < 8 ? ((v >> 1) << 2) + (v & 1) : (((v - 8) >> 1) << 2) + 2 + (v & 1);
  return (tok & ~15) + slot;
}

__device__ __forceinline__ void mma_e4m3_16832(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.f32.e4m3.e4m3.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%0, %1, %2, %3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint8_t to_e4m3(float x) {
  return static_cast<uint8_t>(__nv_cvt_float_to_fp8(x, __NV_SATFINITE, __NV_E4M3));
}
__device__ __forceinline__ float from_e4m3(uint8_t b) {
  const __half_raw h = __nv_cvt_fp8_to_halfraw(b, __NV_E4M3);
  return __half2float(*reinterpret_cast<const __half*>(&h));
}
// four floats -> four E4M3 bytes (a in the lowest byte)
__device__ __forceinline__ uint32_t pack_e4m3x4(float a, float b, float c, float d) {
  const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
  const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, __NV_E4M3);
  return lo | (hi << 16);
}
// x rounded to the four significant bits E4M3 keeps (exact for E4M3's normal range; below it the result is
// finer than E4M3, which only makes the low-order term of a split vanish there)
__device__ __forceinline__ float round_to_e4m3_bits(float x) {
  return __uint_as_float((__float_as_uint(x) + 0x00080000u) & 0xfff00000u);
}

__device__ __forceinline__ int split_length(int kv_len, int num_splits, int min_split) {
  int per = (kv_len + num_splits - 1) / num_splits;
  per = ((per + kTile - 1) / kTile) * kTile;
  return per < min_split ? min_split : per;
}
__device__ __forceinline__ void rope_pair(float x1, float x2, float c, float s, float& o1, float& o2) {
  o1 = bf16_round(bf16_round(x1 * c) + bf16_round(-x2 * s));
  o2 = bf16_round(bf16_round(x2 * c) + bf16_round(x1 * s));
}
__device__ __forceinline__ void consumer_barrier() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

using attn::Params;

// kMode 1, 2: queries and probabilities as hi + lo E4M3 terms (the kernel then adds nothing measurable to the
// pool's own quantisation error: 1.3e-3 against 4e-2 relative); kMode 0: one term each (the usual FP8-attention
// trade: total error 5.2e-2 instead of 4.0e-2).
// kMode 2 ("stacked", groups of at most 8 query heads - every Llama shape): the hi terms of the group's heads are rows
// 0..7 of the 16-row A operand and the lo terms of the same heads rows 8..15, so ONE mma yields both partial products
// and the thread that owns row g also owns row g + 8: S = S_hi + S_lo and O = O_hi + O_lo are register adds.  Two
// terms then cost the tensor-core work of one, and the softmax runs on one row per thread instead of two.
// kMode 1 (groups of 9..16 heads): the terms as separate mma instructions into the same accumulators.
// kMode 3: one term for groups of at most 8 heads - rows 8..15 are padding, so their softmax is skipped.
template <int kMode>
__global__ void __launch_bounds__(kThreads, 2)
paged_attention_fp8_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v, Params p) {
  constexpr bool kTwoTerms = kMode == 1 || kMode == 2;
  constexpr bool kStacked = kMode == 2;
  constexpr bool kLowerRowsOnly = kMode == 3;
  constexpr int kRows = (kStacked || kLowerRowsOnly) ? 1 : 2;  // accumulator rows (g, g + 8) with a softmax state of their own
  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;

  pdl_launch_dependents();
  const int unit = blockIdx.x;
  const int split = unit % p.num_splits;
  const int h = (unit / p.num_splits) % p.nkv;
  const int t_slot = unit / (p.num_splits * p.nkv);
  const int t = p.row_order ? p.row_order[t_slot] : t_slot;
  // (every CTA waits for the preceding grid before it exits, early exits included: see attention.cu)
  if (static_cast<unsigned>(t) >= static_cast<unsigned>(p.T)) {
    pdl_wait();
    return;
  }
  const int G = p.G;
  const int kv_len = p.kv_len[t];
  if (kv_len <= 0) {  // padding row: zeros
    pdl_wait();
    if (p.num_splits == 1) {
      __shared__ float red0[4];
      if (tid < kConsumerThreads)
        for (int i = tid; i < G * D; i += kConsumerThreads)
          attn::store_output<D>(p, t, h * G + i / D, i % D, 0.f, red0, attn::consumer_barrier);
    }
    return;
  }
  const int L = split_length(kv_len, p.num_splits, p.min_split);
  const int start = split * L;
  if (start >= kv_len) {
    pdl_wait();
    return;
  }
  const int end = min(kv_len, start + L);
  const int n_tiles = (end - start + kTile - 1) / kTile;
  const int row = p.row_of_token ? p.row_of_token[t] : t;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __nv_bfloat16* q16 = reinterpret_cast<__nv_bfloat16*>(smem + kStages * kStageBytes);
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + kStages * kStageBytes + kQ16Bytes);
  uint64_t* empty_bar = full_bar + kStages;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(empty_bar + kStages);
  uint8_t* q8_hi = smem + kStages * kStageBytes + kQ16Bytes + 256;
  uint8_t* q8_lo = q8_hi + 16 * kQ8Stride;
  float* q_scale = reinterpret_cast<float*>(q8_lo + 16 * kQ8Stride);  // one power of two per query row

  if (tid == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], kConsumerWarps);
    }
    *abort_flag = 0;
    fence_barrier_init();
    prefetch_tensormap(&map_k);
    prefetch_tensormap(&map_v);
  }
  __syncthreads();

  if (warp == kConsumerWarps) {
    // ------------------------------- producer warp -------------------------------
    if (lane == 0) {
      if (!p.fused) pdl_wait();  // prefill steps: the append kernel before us writes the pool
      const int32_t* bt_row = p.block_table + static_cast<int64_t>(row) * p.max_chunks;
      int cur_c = -1, cur_id = 0;
      for (int i = 0; i < n_tiles; ++i) {
        const int s = i % kStages;
        const uint32_t phase = (i / kStages) & 1;
        const int tok0 = start + i * kTile;
        const int c = tok0 / p.chunk;
        if (c != cur_c) {
          cur_c = c;
          cur_id = bt_row[c];
        }
        const int in_chunk = tok0 - c * p.chunk;
        mbar_wait_bounded(&empty_bar[s], phase ^ 1, abort_flag, kStatusAttnTimeout);
        uint8_t* kdst = smem + s * kStageBytes;
        mbar_arrive_expect_tx(&full_bar[s], kStageBytes);
        tma_load_3d(kdst, &map_k, &full_bar[s], 0, h, cur_id * p.chunk + in_chunk);           // [token][dim]
        tma_load_3d(kdst + kTileBytes, &map_v, &full_bar[s], in_chunk, 0, cur_id * p.nkv + h);  // [dim][position]
      }
    }
    return;
  }

  // --------------------------------- consumer warps ---------------------------------
  const int gid = lane >> 2;
  const int tig = lane & 3;
  const __nv_bfloat16* qkv_t = p.qkv + (static_cast<int64_t>(t) * p.nkv + h) * (G + 2) * D;

  pdl_wait();  // qkv is the previous kernel's output
  // Rotated queries as bf16 (the reference's rounding point), then per head: power-of-two scale and two E4M3 terms.
  {
    const bool rope = p.cos != nullptr;
    const int64_t pq = rope ? p.pos_q[t] : 0;
    const __nv_bfloat16* cs = p.cos + pq * (D / 2);
    const __nv_bfloat16* sn = p.sin + pq * (D / 2);
    for (int i = tid; i < G * (D / 2); i += kConsumerThreads) {
      const int g = i / (D / 2);
      const int j = i - g * (D / 2);
      float x1 = __bfloat162float(qkv_t[g * D + j]);
      float x2 = __bfloat162float(qkv_t[g * D + j + D / 2]);
      if (rope) rope_pair(x1, x2, __bfloat162float(cs[j]), __bfloat162float(sn[j]), x1, x2);
      q16[g * kQStride16 + j] = __float2bfloat16_rn(x1);
      q16[g * kQStride16 + j + D / 2] = __float2bfloat16_rn(x2);
    }
  }
  consumer_barrier();
  for (int r = warp; r < 16; r += kConsumerWarps) {  // one warp per query row, four elements per lane
    float x[4] = {0.f, 0.f, 0.f, 0.f};
    if (r < G) {
#pragma unroll
      for (int e = 0; e < 4; ++e) x[e] = __bfloat162float(q16[r * kQStride16 + lane * 4 + e]);
    }
    float amax = fmaxf(fmaxf(fabsf(x[0]), fabsf(x[1])), fmaxf(fabsf(x[2]), fabsf(x[3])));
    amax = warp_max(amax);
    // smallest power of two s with amax / s <= 256: the high term keeps clear of E4M3's 448 limit
    const float s = amax > 0.f ? exp2f(ceilf(log2f(amax * (1.f / 256.f)))) : 1.f;
    const float inv = 1.f / s;
    uint32_t hi = 0, lo = 0;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float v = x[e] * inv;
      const uint8_t bh = to_e4m3(v);
      const uint8_t bl = to_e4m3(v - from_e4m3(bh));
      hi |= static_cast<uint32_t>(bh) << (8 * e);
      lo |= static_cast<uint32_t>(bl) << (8 * e);
    }
    *reinterpret_cast<uint32_t*>(q8_hi + r * kQ8Stride + lane * 4) = hi;
    *reinterpret_cast<uint32_t*>(q8_lo + r * kQ8Stride + lane * 4) = lo;
    if (lane == 0) q_scale[r] = s;
  }
  consumer_barrier();

  // A fragments of the two query terms: k-step s covers dims 32s .. 32s+31
  uint32_t qh[4][4], ql[4][4];
#pragma unroll
  for (int s = 0; s < 4; ++s) {
    const int c0 = s * 32 + tig * 4;
    qh[s][0] = *reinterpret_cast<const uint32_t*>(q8_hi + gid * kQ8Stride + c0);
    qh[s][1] = *reinterpret_cast<const uint32_t*>(q8_hi + (gid + 8) * kQ8Stride + c0);
    qh[s][2] = *reinterpret_cast<const uint32_t*>(q8_hi + gid * kQ8Stride + c0 + 16);
    qh[s][3] = *reinterpret_cast<const uint32_t*>(q8_hi + (gid + 8) * kQ8Stride + c0 + 16);
    ql[s][0] = *reinterpret_cast<const uint32_t*>(q8_lo + gid * kQ8Stride + c0);
    ql[s][1] = *reinterpret_cast<const uint32_t*>(q8_lo + (gid + 8) * kQ8Stride + c0);
    ql[s][2] = *reinterpret_cast<const uint32_t*>(q8_lo + gid * kQ8Stride + c0 + 16);
    ql[s][3] = *reinterpret_cast<const uint32_t*>(q8_lo + (gid + 8) * kQ8Stride + c0 + 16);
    if constexpr (kStacked) {  // rows 8..15 of the A operand = the lo terms of rows 0..7
      qh[s][1] = ql[s][0];
      qh[s][3] = ql[s][2];
    }
  }
  // logits in the log2 domain: acc * (query scale * key scale * softmax scale * log2 e), per row
  const float row_scale[2] = {q_scale[gid] * p.k_scale[h] * p.scale_log2, q_scale[gid + 8] * p.k_scale[h] * p.scale_log2};
  const float out_scale = p.v_scale[h] * (1.f / kPScale);

  float oacc[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) oacc[i][0] = oacc[i][1] = oacc[i][2] = oacc[i][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY};
  float l_run[2] = {0.f, 0.f};
  const int new_pos = kv_len - 1;
  const bool owns_new = p.fused && new_pos >= start && new_pos < end;
  const int r0 = warp * 32;  // this warp's token slice inside a tile
  const int mi = lane >> 3;  // ldmatrix: which of the four 8 x 16-byte matrices this lane addresses
  const int mr = lane & 7;

  for (int i = 0; i < n_tiles; ++i) {
    const int s = i % kStages;
    const uint32_t phase = (i / kStages) & 1;
    const int tok0 = start + i * kTile;
    mbar_wait_bounded(&full_bar[s], phase, abort_flag, kStatusAttnTimeout);
    uint8_t* ktile = smem + s * kStageBytes;
    uint8_t* vtile = ktile + kTileBytes;

    if (owns_new && new_pos >= tok0 + r0 && new_pos < tok0 + r0 + 32) {
      // This warp's slice holds the new token: rotate and quantise k, quantise v, store both to the pool and patch
      // them into the tiles (key row `rr`; value column v_position(rr) of every dim row).
      const int rr = new_pos - tok0;
      const int vcol = v_position(rr);
      const __nv_bfloat16* kn = qkv_t + G * D;
      const __nv_bfloat16* vn = kn + D;
      const int64_t ci = p.chunk_idx[t];
      const int lp = static_cast<int>(p.local_pos[t]);
      uint8_t* kg = reinterpret_cast<uint8_t*>(p.k_cache) + ((ci * p.chunk + lp) * p.nkv + h) * D;
      uint8_t* vg = reinterpret_cast<uint8_t*>(p.v_cache) + (ci * p.nkv + h) * static_cast<int64_t>(D) * p.chunk + v_position(lp);
      const bool rope = p.cos != nullptr;
      const int64_t pk = rope ? p.pos_k[t] : 0;
      const float ks = p.k_scale[h], vs = p.v_scale[h];
      for (int j = lane * 2; j < D / 2; j += 64) {
        float a1 = __bfloat162float(kn[j]), a2 = __bfloat162float(kn[j + D / 2]);
        float b1 = __bfloat162float(kn[j + 1]), b2 = __bfloat162float(kn[j + 1 + D / 2]);
        if (rope) {
          const __nv_bfloat16* cs = p.cos + pk * (D / 2);
          const __nv_bfloat16* sn = p.sin + pk * (D / 2);
          rope_pair(a1, a2, __bfloat162float(cs[j]), __bfloat162float(sn[j]), a1, a2);
          rope_pair(b1, b2, __bfloat162float(cs[j + 1]), __bfloat162float(sn[j + 1]), b1, b2);
        }
        const int dd[4] = {j, j + 1, j + D / 2, j + 1 + D / 2};
        const uint8_t kb[4] = {to_e4m3(a1 / ks), to_e4m3(b1 / ks), to_e4m3(a2 / ks), to_e4m3(b2 / ks)};
        const uint8_t vb[4] = {to_e4m3(__bfloat162float(vn[j]) / vs), to_e4m3(__bfloat162float(vn[j + 1]) / vs),
                               to_e4m3(__bfloat162float(vn[j + D / 2]) / vs), to_e4m3(__bfloat162float(vn[j + 1 + D / 2]) / vs)};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int d = dd[e];
          kg[d] = kb[e];
          vg[static_cast<int64_t>(d) * p.chunk] = vb[e];
          ktile[rr * 128 + ((((d >> 4) ^ (rr & 7)) << 4) | (d & 15))] = kb[e];
          vtile[d * 128 + ((((vcol >> 4) ^ (d & 7)) << 4) | (vcol & 15))] = vb[e];
        }
      }
      __syncwarp();
    }

    if (tok0 + r0 < end) {
      // ---- S = Q K^T: 16 rows x 32 tokens (n-tiles of 8 tokens), hi and lo query terms ----
      float sacc[4][4];
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) sacc[nt][0] = sacc[nt][1] = sacc[nt][2] = sacc[nt][3] = 0.f;
      const uint32_t kbase = smem_u32(ktile);
#pragma unroll
      for (int ks = 0; ks < 4; ++ks) {
#pragma unroll
        for (int pair = 0; pair < 2; ++pair) {
          // matrices: (tokens +0..7, bytes 32ks..+15), (tokens +0..7, bytes +16..+31), (tokens +8..15, ...) x 2
          const int trow = r0 + pair * 16 + ((mi >> 1) << 3) + mr;
          const int c16 = ks * 2 + (mi & 1);
          uint32_t b0, b1, b2, b3;
          ldmatrix_x4(kbase + trow * 128 + ((c16 ^ (trow & 7)) << 4), b0, b1, b2, b3);
          mma_e4m3_16832(sacc[pair * 2], qh[ks], b0, b1);
          if constexpr (kTwoTerms && !kStacked) mma_e4m3_16832(sacc[pair * 2], ql[ks], b0, b1);
          mma_e4m3_16832(sacc[pair * 2 + 1], qh[ks], b2, b3);
          if constexpr (kTwoTerms && !kStacked) mma_e4m3_16832(sacc[pair * 2 + 1], ql[ks], b2, b3);
        }
      }
      // ---- online softmax (log2 domain) ----
      float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) {
#pragma unroll
        for (int c = 0; c < 2 * kRows; ++c) {
          const int tok = tok0 + r0 + nt * 8 + tig * 2 + (c & 1);
          float v = kStacked ? (sacc[nt][c] + sacc[nt][c + 2]) * row_scale[0] : sacc[nt][c] * row_scale[c >> 1];
          if (tok >= end) v = -INFINITY;
          sacc[nt][c] = v;
          mx[c >> 1] = fmaxf(mx[c >> 1], v);
        }
      }
      float alpha[2], m_use[2];
#pragma unroll
      for (int r = 0; r < kRows; ++r) {
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
        const float m_new = fmaxf(m_run[r], mx[r]);
        m_use[r] = (m_new == -INFINITY) ? 0.f : m_new;
        alpha[r] = exp2f(m_run[r] - m_use[r]);
        m_run[r] = m_new;
        l_run[r] *= alpha[r];
      }
      // P * 256 as two E4M3 terms.  k-slot 4*tig+e of a 16-token half is token [2tig, 2tig+1, 8+2tig, 9+2tig][e]:
      // the tokens this thread holds in n-tiles (0, 1) resp. (2, 3) - the order the value pool is stored in.
      uint32_t ph[4], pl[4];
      {
        float hi[4][4], lo[4][4];
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
#pragma unroll
          for (int c = 0; c < 2 * kRows; ++c) {
            const float pv = exp2f(sacc[nt][c] - m_use[c >> 1]);
            l_run[c >> 1] += pv;
            const float ps = pv * kPScale;
            hi[nt][c] = round_to_e4m3_bits(ps);
            lo[nt][c] = ps - hi[nt][c];
          }
        }
        ph[0] = pack_e4m3x4(hi[0][0], hi[0][1], hi[1][0], hi[1][1]);
        ph[2] = pack_e4m3x4(hi[2][0], hi[2][1], hi[3][0], hi[3][1]);
        pl[0] = pack_e4m3x4(lo[0][0], lo[0][1], lo[1][0], lo[1][1]);
        pl[2] = pack_e4m3x4(lo[2][0], lo[2][1], lo[3][0], lo[3][1]);
        if constexpr (kStacked) {  // rows 8..15 of the A operand = the lo terms of rows 0..7
          ph[1] = pl[0];
          ph[3] = pl[2];
        } else if constexpr (kLowerRowsOnly) {
          ph[1] = ph[3] = 0u;
        } else {
          ph[1] = pack_e4m3x4(hi[0][2], hi[0][3], hi[1][2], hi[1][3]);
          ph[3] = pack_e4m3x4(hi[2][2], hi[2][3], hi[3][2], hi[3][3]);
          pl[1] = pack_e4m3x4(lo[0][2], lo[0][3], lo[1][2], lo[1][3]);
          pl[3] = pack_e4m3x4(lo[2][2], lo[2][3], lo[3][2], lo[3][3]);
        }
      }
      if constexpr (kRows == 1) alpha[1] = alpha[0];  // stacked: the O_lo rows follow their head's running maximum
#pragma unroll
      for (int i2 = 0; i2 < D / 8; ++i2) {
        oacc[i2][0] *= alpha[0];
        oacc[i2][1] *= alpha[0];
        oacc[i2][2] *= alpha[1];
        oacc[i2][3] *= alpha[1];
      }
      // ---- O += P V: B operand = rows of the transposed value tile ----
      const uint32_t vbase = smem_u32(vtile);
#pragma unroll
      for (int dn = 0; dn < D / 16; ++dn) {
        // matrices: (dims +0..7, positions r0..r0+15), (dims +0..7, positions +16..+31), (dims +8..15, ...) x 2
        const int drow = dn * 16 + ((mi >> 1) << 3) + mr;
        const int c16 = warp * 2 + (mi & 1);
        uint32_t b0, b1, b2, b3;
        ldmatrix_x4(vbase + drow * 128 + ((c16 ^ (drow & 7)) << 4), b0, b1, b2, b3);
        mma_e4m3_16832(oacc[dn * 2], ph, b0, b1);
        if constexpr (kTwoTerms && !kStacked) mma_e4m3_16832(oacc[dn * 2], pl, b0, b1);
        mma_e4m3_16832(oacc[dn * 2 + 1], ph, b2, b3);
        if constexpr (kTwoTerms && !kStacked) mma_e4m3_16832(oacc[dn * 2 + 1], pl, b2, b3);
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&empty_bar[s]);
  }

  // ------------------------------ merge the four warps ------------------------------
#pragma unroll
  for (int r = 0; r < kRows; ++r) {
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
  }
  consumer_barrier();  // every warp is done with the tile ring; reuse it
  float* mo = reinterpret_cast<float*>(smem);  // [warp][16][D]
  float* mm = mo + kConsumerWarps * 16 * D;    // [warp][16]
  float* ml = mm + kConsumerWarps * 16;        // [warp][16]
#pragma unroll
  for (int i2 = 0; i2 < D / 8; ++i2) {
    const int col = i2 * 8 + tig * 2;
    float* o0 = mo + (warp * 16 + gid) * D + col;
    float* o1 = mo + (warp * 16 + gid + 8) * D + col;
    if constexpr (kStacked) {  // O = O_hi + O_lo; rows 8..15 are not heads
      o0[0] = oacc[i2][0] + oacc[i2][2];
      o0[1] = oacc[i2][1] + oacc[i2][3];
    } else {
      o0[0] = oacc[i2][0];
      o0[1] = oacc[i2][1];
      if constexpr (!kLowerRowsOnly) {
        o1[0] = oacc[i2][2];
        o1[1] = oacc[i2][3];
      }
    }
  }
  if (tig == 0) {
    mm[warp * 16 + gid] = m_run[0];
    ml[warp * 16 + gid] = l_run[0];
    if constexpr (kRows == 2) {
      mm[warp * 16 + gid + 8] = m_run[1];
      ml[warp * 16 + gid + 8] = l_run[1];
    }
  }
  consumer_barrier();
  for (int i = tid; i < G * D; i += kConsumerThreads) {
    const int g = i / D;
    const int d = i - g * D;
    float m = -INFINITY;
#pragma unroll
    for (int w = 0; w < kConsumerWarps; ++w) m = fmaxf(m, mm[w * 16 + g]);
    float acc = 0.f, lsum = 0.f;
    if (m != -INFINITY) {
#pragma unroll
      for (int w = 0; w < kConsumerWarps; ++w) {
        const float sc = exp2f(mm[w * 16 + g] - m);
        acc += mo[(w * 16 + g) * D + d] * sc;
        lsum += ml[w * 16 + g] * sc;
      }
    }
    const float o = lsum > 0.f ? acc / lsum * out_scale : 0.f;
    const int64_t qh_idx = static_cast<int64_t>(t) * p.nq + h * G + g;
    if (p.num_splits == 1) {
      attn::store_output<D>(p, t, h * G + g, d, o, ml + kConsumerWarps * 16, attn::consumer_barrier);
    } else {
      p.ws_o[(qh_idx * p.num_splits + split) * D + d] = o;
      if (d == 0) p.ws_lse[qh_idx * p.num_splits + split] = lsum > 0.f ? m + log2f(lsum) : -INFINITY;
    }
  }
}

// Merge of the context splits (same as the 16-bit kernel's, with this kernel's split length).
__global__ void __launch_bounds__(D) combine_fp8_kernel(Params p) {
  pdl_launch_dependents();
  pdl_wait();
  const int qh = blockIdx.x;
  const int t = qh / p.nq;
  const int d = threadIdx.x;
  const int kv_len = p.kv_len[t];
  float o = 0.f;
  if (kv_len > 0) {
    const int L = split_length(kv_len, p.num_splits, p.min_split);
    const int n_act = (kv_len + L - 1) / L;
    const float* lse = p.ws_lse + static_cast<int64_t>(qh) * p.num_splits;
    float mx = -INFINITY;
    for (int s = 0; s < n_act; ++s) mx = fmaxf(mx, lse[s]);
    if (mx != -INFINITY) {
      float acc = 0.f, wsum = 0.f;
      for (int s = 0; s < n_act; ++s) {
        const float w = exp2f(lse[s] - mx);
        acc += w * p.ws_o[(static_cast<int64_t>(qh) * p.num_splits + s) * D + d];
        wsum += w;
      }
      o = acc / wsum;
    }
  }
  __shared__ float red[4];
  attn::store_output<D>(p, t, qh - t * p.nq, d, o, red, [] { __syncthreads(); });
}

// Prefill / mixed steps: rotate k, quantise, scatter k (row layout) and v (transposed, permuted layout).
__global__ void __launch_bounds__(128) rope_append_fp8_kernel(Params p) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int G = p.G;
  const bool rope = p.cos != nullptr;
  const int64_t pk = rope ? p.pos_k[t] : 0;
  const int64_t ci = p.chunk_idx[t];
  const int lp = static_cast<int>(p.local_pos[t]);
  uint8_t* kc = reinterpret_cast<uint8_t*>(p.k_cache);
  uint8_t* vc = reinterpret_cast<uint8_t*>(p.v_cache);
  for (int i = threadIdx.x; i < p.nkv * (D / 2); i += blockDim.x) {
    const int h = i / (D / 2);
    const int j = i - h * (D / 2);
    const __nv_bfloat16* kn = p.qkv + (static_cast<int64_t>(t) * p.nkv + h) * (G + 2) * D + G * D;
    const __nv_bfloat16* vn = kn + D;
    float x1 = __bfloat162float(kn[j]);
    float x2 = __bfloat162float(kn[j + D / 2]);
    if (rope)
      rope_pair(x1, x2, __bfloat162float(p.cos[pk * (D / 2) + j]), __bfloat162float(p.sin[pk * (D / 2) + j]), x1, x2);
    const float ks = p.k_scale[h], vs = p.v_scale[h];
    uint8_t* kg = kc + ((ci * p.chunk + lp) * p.nkv + h) * D;
    uint8_t* vg = vc + (ci * p.nkv + h) * static_cast<int64_t>(D) * p.chunk + v_position(lp);
    kg[j] = to_e4m3(x1 / ks);
    kg[j + D / 2] = to_e4m3(x2 / ks);
    vg[static_cast<int64_t>(j) * p.chunk] = to_e4m3(__bfloat162float(vn[j]) / vs);
    vg[static_cast<int64_t>(j + D / 2) * p.chunk] = to_e4m3(__bfloat162float(vn[j + D / 2]) / vs);
  }
}

static int launch_attention_fp8(Params& p, bool two_terms, cudaStream_t stream) {
  if (p.chunk % kTile != 0) return B200_ERR_INVALID_ARGUMENT;  // a tile never straddles two chunks
  // keys: [token][head][dim] bytes; values: [chunk * head][dim][position] bytes
  const uint64_t kdims[3] = {static_cast<uint64_t>(D), static_cast<uint64_t>(p.nkv), static_cast<uint64_t>(p.num_chunks) * p.chunk};
  const uint64_t kstr[2] = {static_cast<uint64_t>(D), static_cast<uint64_t>(p.nkv) * D};
  const uint32_t kbox[3] = {128u, 1, kTile};
  const uint64_t vdims[3] = {static_cast<uint64_t>(p.chunk), static_cast<uint64_t>(D), static_cast<uint64_t>(p.num_chunks) * p.nkv};
  const uint64_t vstr[2] = {static_cast<uint64_t>(p.chunk), static_cast<uint64_t>(p.chunk) * D};
  const uint32_t vbox[3] = {128u, static_cast<uint32_t>(D), 1};
  const CUtensorMap* mk = get_tensor_map(p.k_cache, 3, kdims, kstr, kbox, CU_TENSOR_MAP_SWIZZLE_128B,
                                         CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_DATA_TYPE_UINT8);
  const CUtensorMap* mv = get_tensor_map(p.v_cache, 3, vdims, vstr, vbox, CU_TENSOR_MAP_SWIZZLE_128B,
                                         CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_DATA_TYPE_UINT8);
  if (!mk || !mv) return B200_ERR_DRIVER;
  static std::atomic<uint64_t> smem_attr_done0{0}, smem_attr_done1{0}, smem_attr_done2{0}, smem_attr_done3{0};
  if (ensure_dynamic_smem(paged_attention_fp8_kernel<0>, kSmemBytes, smem_attr_done0) != B200_OK ||
      ensure_dynamic_smem(paged_attention_fp8_kernel<1>, kSmemBytes, smem_attr_done1) != B200_OK ||
      ensure_dynamic_smem(paged_attention_fp8_kernel<2>, kSmemBytes, smem_attr_done2) != B200_OK ||
      ensure_dynamic_smem(paged_attention_fp8_kernel<3>, kSmemBytes, smem_attr_done3) != B200_OK)
    return B200_ERR_LAUNCH;
  const int64_t units = static_cast<int64_t>(p.T) * p.nkv * p.num_splits;
  if (units > 0x7fffffff) return B200_ERR_INVALID_ARGUMENT;
  const int mode = two_terms ? (p.G <= 8 ? 2 : 1) : (p.G <= 8 ? 3 : 0);
  const dim3 grid(static_cast<unsigned>(units)), block(kThreads);
  int rc = mode == 0   ? launch_pdl(paged_attention_fp8_kernel<0>, grid, block, kSmemBytes, stream, *mk, *mv, p)
           : mode == 1 ? launch_pdl(paged_attention_fp8_kernel<1>, grid, block, kSmemBytes, stream, *mk, *mv, p)
           : mode == 2 ? launch_pdl(paged_attention_fp8_kernel<2>, grid, block, kSmemBytes, stream, *mk, *mv, p)
                       : launch_pdl(paged_attention_fp8_kernel<3>, grid, block, kSmemBytes, stream, *mk, *mv, p);
  if (rc != B200_OK) return rc;
  if (p.num_splits > 1) rc = launch_pdl(combine_fp8_kernel, dim3(p.T * p.nq), dim3(D), 0, stream, p);
  return rc;
}

}  // namespace attn8
}  // namespace b200

extern "C" {

int b200_fp8_value_position(int token_in_chunk) { return b200::attn8::v_position(token_in_chunk); }

}  // extern "C"
