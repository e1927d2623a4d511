// Paged-KV attention for the dynamic inference context (GQA, bf16 KV pool, head dim 64 / 128; the E4M3 pool has
// kernels of its own in attention_fp8.cu).
//
// One CTA works on one (token row, KV head, context split) unit:
//   * a producer warp walks the row's block table and streams 64-token K and V tiles of that KV
//     head from the chunked pool into a 3-stage shared-memory ring with TMA (3-D tensor map
//     {d, head, token}, 128-byte swizzle), completion on mbarriers;
//   * four consumer warps each take a 16-token slice of every tile: S = Q K^T with mma.sync
//     (the M side is the group's 4-8 query heads padded to 16), online softmax with warp shuffles
//     in the exp2 domain, O += P V (P as hi + lo bf16 terms); per-warp (max, sum, O) states are
//     merged through shared memory at the end.
// RoPE of the query heads is applied while staging Q.  In decode steps (fuse_rope_append) the unit
// whose range contains the new token also rotates the new key, writes key and value into the pool
// and patches them into its shared-memory tile, so no separate append kernel runs.
// With num_splits > 1 every unit writes a normalised partial output and its log-sum-exp; a small
// second kernel merges the splits of a row (flash-decoding).
//
// The kernel is bound by reading the K/V pool once from HBM: algorithmic bytes per launch are
// sum_rows kv_len * 2 * nkv * d * 2.
#include "common.cuh"
#include "quant.cuh"

namespace b200 {
namespace attn {

constexpr int kTile = 64;            // tokens per K/V tile
constexpr int kConsumerWarps = 4;
constexpr int kConsumerThreads = kConsumerWarps * 32;
constexpr int kThreads = kConsumerThreads + 32;
constexpr int kStages = 3;
constexpr int kMaxSplits = 64;

template <int D>
struct Cfg {
  static constexpr int kSub = D / 64;                 // 128-byte swizzle rows hold 64 bf16 values
  static constexpr int kSubBytes = kTile * 128;       // one [64 tokens x 64 dims] sub-tile
  static constexpr int kTileBytes = kSub * kSubBytes; // K or V tile in the ring
  static constexpr int kStageBytes = 2 * kTileBytes;
  static constexpr int kQStride = D + 8;              // bf16 elements, padded against bank conflicts
  static constexpr int kQBytes = 16 * kQStride * 2;
  static constexpr int kQkvBytes = 18 * D * 2;        // (G + 2) <= 18 head vectors of this unit, when they are summed
                                                      // here from the QKV GEMM's split-K partial sums
  static constexpr int kMergeBytes = kConsumerWarps * 16 * (D + 2) * 4;
  static_assert(kMergeBytes <= kStages * kStageBytes, "merge buffers reuse the tile ring");
  static constexpr int kSmemBytes = kStages * kStageBytes + kQBytes + 256 + kQkvBytes + 1024;
};

struct Params {
  const __nv_bfloat16* qkv;
  const float* qkv_partials;  // [qkv_splits][T][nkv * (G + 2) * D] fp32: split-K partial sums of the QKV GEMM, used
  int qkv_splits;             // instead of qkv when non-null (decode kernel only)
  __nv_bfloat16* k_cache;
  __nv_bfloat16* v_cache;
  const int32_t* block_table;
  const int32_t* kv_len;
  const int32_t* row_of_token;
  const int32_t* row_order;
  const int64_t* pos_q;
  const int64_t* pos_k;
  const int64_t* chunk_idx;
  const int64_t* local_pos;
  const __nv_bfloat16* cos;
  const __nv_bfloat16* sin;
  __nv_bfloat16* out;
  // Quantised output (the out-projection's FP8 input) instead of `out`: E4M3 bytes [T][nq * D] + scales, written by the
  // kernel that finishes an output row (decode kernels only).  out_q_mode: mx::kQuantMx (E8M0 per 32, tile layout) or
  // mx::kQuantBlock128 (fp32 per token per 128 = per head, scale[nq][out_m_pad]; head_dim 128 only).
  uint8_t* out_q;
  void* out_sf;
  int out_q_mode, out_m_pad;
  const float* k_scale;  // E4M3 pool (attention_fp8.cu): one scale per KV head; nullptr otherwise
  const float* v_scale;
  float* ws_o;    // [T][nq][splits][D]
  float* ws_lse;  // [T][nq][splits]   (log2 domain)
  int T, nq, nkv, G, chunk, num_chunks, max_chunks, num_splits, fused, min_split;
  float scale_log2;  // softmax scale * log2(e)
};

// Tokens per split for a row of kv_len tokens: equal shares rounded up to whole tiles, never
// smaller than min_split.  The combine kernel uses the same formula.
__device__ __forceinline__ int split_length(int kv_len, int num_splits, int min_split) {
  int per = (kv_len + num_splits - 1) / num_splits;
  per = ((per + kTile - 1) / kTile) * kTile;
  return per < min_split ? min_split : per;
}

// out = bf16(bf16(x1 * c) - bf16(x2 * s)), bf16(bf16(x2 * c) + bf16(x1 * s)): the rounding points of
// `t * cos + rotate_half(t) * sin` evaluated in bf16.
__device__ __forceinline__ void rope_pair(float x1, float x2, float c, float s, float& o1, float& o2) {
  o1 = bf16_round(bf16_round(x1 * c) + bf16_round(-x2 * s));
  o2 = bf16_round(bf16_round(x2 * c) + bf16_round(x1 * s));
}

__device__ __forceinline__ void consumer_barrier() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

// One finished output element o of (token t, query head `head`, dim d).  Plain mode: bf16 store.  Quantised mode: the
// bf16-rounded value (what a stand-alone quantiser would read) goes out as E4M3 with the scale of its block.  The 32
// lanes of a warp hold 32 consecutive dims of one head (all call sites), which is one MXFP8 scale block; the 128-block
// recipe needs the maximum over the whole head (D == 128 = four warps): `red` is a 4-float shared array and
// `block_sync` the barrier over exactly the threads that take part.  Every thread of the warp / block must call it.
template <int D, typename Sync>
__device__ __forceinline__ void store_output(const Params& p, int t, int head, int d, float o, float* red, Sync block_sync) {
  if (p.out_q == nullptr) {
    p.out[(static_cast<int64_t>(t) * p.nq + head) * D + d] = __float2bfloat16_rn(o);
    return;
  }
  const float ob = bf16_round(o);
  const int64_t ldq = static_cast<int64_t>(p.nq) * D;
  const int col = head * D + d;
  float amax = warp_max(fabsf(ob));
  if (p.out_q_mode == mx::kQuantMx) {
    const uint32_t e = mx::e8m0_scale_byte(amax);
    const float inv = scalbnf(1.0f, 127 - static_cast<int>(e));
    p.out_q[t * ldq + col] = static_cast<uint8_t>(__nv_cvt_float_to_fp8(ob * inv, __NV_SATFINITE, __NV_E4M3));
    if ((threadIdx.x & 31) == 0)
      static_cast<uint8_t*>(p.out_sf)[mx::sf_offset(t, col >> 5, static_cast<int>(ldq >> 7))] = static_cast<uint8_t>(e);
  } else {
    const int w = (d >> 5) & 3;
    if ((threadIdx.x & 31) == 0) red[w] = amax;
    block_sync();
    amax = fmaxf(fmaxf(red[0], red[1]), fmaxf(red[2], red[3]));
    block_sync();  // `red` may be rewritten by the next call
    const float sc = fmaxf(amax / 448.0f, 1e-30f);
    p.out_q[t * ldq + col] = static_cast<uint8_t>(__nv_cvt_float_to_fp8(ob / sc, __NV_SATFINITE, __NV_E4M3));
    if (d == 0) static_cast<float*>(p.out_sf)[static_cast<int64_t>(head) * p.out_m_pad + t] = sc;
  }
}

template <int D>
__global__ void __launch_bounds__(kThreads, 2)
paged_attention_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v, Params p) {
  using C = Cfg<D>;
  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;

  pdl_launch_dependents();
  const int unit = blockIdx.x;
  const int split = unit % p.num_splits;
  const int h = (unit / p.num_splits) % p.nkv;
  const int t_slot = unit / (p.num_splits * p.nkv);
  const int t = p.row_order ? p.row_order[t_slot] : t_slot;
  // Every CTA waits for the preceding grid before it exits, also on the early exits below: programmatic
  // launch ordering is only transitive (this grid's successors may assume that its predecessors are done)
  // if no grid can complete before the one in front of it.
  if (static_cast<unsigned>(t) >= static_cast<unsigned>(p.T)) {  // not a permutation: skip, never index with it
    pdl_wait();
    return;
  }
  const int G = p.G;
  const int kv_len = p.kv_len[t];

  if (kv_len <= 0) {  // padding row: flash-attn returns zeros for it
    pdl_wait();
    if (p.num_splits == 1) {
      __shared__ float red0[4];
      if (tid < kConsumerThreads)
        for (int i = tid; i < G * D; i += kConsumerThreads) store_output<D>(p, t, h * G + i / D, i % D, 0.f, red0, consumer_barrier);
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
  __nv_bfloat16* q_smem = reinterpret_cast<__nv_bfloat16*>(smem + kStages * C::kStageBytes);
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + kStages * C::kStageBytes + C::kQBytes);
  uint64_t* empty_bar = full_bar + kStages;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(empty_bar + kStages);
  __nv_bfloat16* qkv_smem = reinterpret_cast<__nv_bfloat16*>(smem + kStages * C::kStageBytes + C::kQBytes + 256);

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
      // Decode steps: the pool holds only what earlier steps wrote (this step's key/value is patched
      // in by the consumers), so K/V streaming starts without waiting for the QKV GEMM before us.
      // Prefill steps: the append kernel right before us writes the pool, so wait for it.
      if (!p.fused) pdl_wait();
      const int32_t* bt_row = p.block_table + static_cast<int64_t>(row) * p.max_chunks;
      int cur_c = -1;
      int cur_id = 0;
      for (int i = 0; i < n_tiles; ++i) {
        const int s = i % kStages;
        const uint32_t phase = (i / kStages) & 1;
        const int tok0 = start + i * kTile;
        const int c = tok0 / p.chunk;
        if (c != cur_c) {
          cur_c = c;
          cur_id = bt_row[c];
        }
        const int tok_row = cur_id * p.chunk + (tok0 - c * p.chunk);
        mbar_wait_bounded(&empty_bar[s], phase ^ 1, abort_flag, kStatusAttnTimeout);
        uint8_t* kdst = smem + s * C::kStageBytes;
        uint8_t* vdst = kdst + C::kTileBytes;
        mbar_arrive_expect_tx(&full_bar[s], C::kStageBytes);
#pragma unroll
        for (int sub = 0; sub < C::kSub; ++sub) {
          tma_load_3d(kdst + sub * C::kSubBytes, &map_k, &full_bar[s], sub * 64, h, tok_row);
          tma_load_3d(vdst + sub * C::kSubBytes, &map_v, &full_bar[s], sub * 64, h, tok_row);
        }
      }
    }
    return;
  }

  // --------------------------------- consumer warps ---------------------------------
  const int gid = lane >> 2;
  const int tig = lane & 3;
  const __nv_bfloat16* qkv_t = p.qkv + (static_cast<int64_t>(t) * p.nkv + h) * (G + 2) * D;

  pdl_wait();  // qkv is the previous kernel's output
  if (p.qkv_partials != nullptr) {
    // The QKV GEMM left fp32 split-K partial sums: reduce this unit's (G + 2) head vectors here (split order, one
    // bf16 rounding - what the GEMM's own reduction kernel would have written) and read them from shared memory.
    const int width = (G + 2) * D;
    const int64_t row_elems = static_cast<int64_t>(p.nkv) * width;
    const float* src = p.qkv_partials + static_cast<int64_t>(t) * row_elems + static_cast<int64_t>(h) * width;
    const int64_t split_stride = static_cast<int64_t>(p.T) * row_elems;
    for (int i = tid * 4; i < width; i += kConsumerThreads * 4) {
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int sp = 0; sp < p.qkv_splits; ++sp) {
        const float4 v = __ldcg(reinterpret_cast<const float4*>(src + sp * split_stride + i));
        acc.x += v.x;
        acc.y += v.y;
        acc.z += v.z;
        acc.w += v.w;
      }
      *reinterpret_cast<uint2*>(qkv_smem + i) = make_uint2(pack_bf16x2(acc.x, acc.y), pack_bf16x2(acc.z, acc.w));
    }
    consumer_barrier();
    qkv_t = qkv_smem;
  }
  // Stage Q (with RoPE) as a zero-padded [16][D] tile.
  for (int i = tid; i < 16 * C::kQStride / 2; i += kConsumerThreads)
    reinterpret_cast<uint32_t*>(q_smem)[i] = 0u;
  consumer_barrier();
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
      q_smem[g * C::kQStride + j] = __float2bfloat16_rn(x1);
      q_smem[g * C::kQStride + j + D / 2] = __float2bfloat16_rn(x2);
    }
  }
  consumer_barrier();

  uint32_t qf[D / 16][4];
#pragma unroll
  for (int ks = 0; ks < D / 16; ++ks) {
    const int col = ks * 16 + tig * 2;
    qf[ks][0] = *reinterpret_cast<const uint32_t*>(&q_smem[gid * C::kQStride + col]);
    qf[ks][1] = *reinterpret_cast<const uint32_t*>(&q_smem[(gid + 8) * C::kQStride + col]);
    qf[ks][2] = *reinterpret_cast<const uint32_t*>(&q_smem[gid * C::kQStride + col + 8]);
    qf[ks][3] = *reinterpret_cast<const uint32_t*>(&q_smem[(gid + 8) * C::kQStride + col + 8]);
  }

  float oacc[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) oacc[i][0] = oacc[i][1] = oacc[i][2] = oacc[i][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY};
  float l_run[2] = {0.f, 0.f};  // per-thread partial row sums (reduced over the quad at the end)

  // FP8 pool: K and V are bytes * per-head scale; the scales factor out of both products
  const float scale_log2 = p.scale_log2;
  const int new_pos = kv_len - 1;  // position of this step's token (decode)
  const bool owns_new = p.fused && new_pos >= start && new_pos < end;
  const int r0 = warp * 16;        // this warp's token slice inside a tile

  for (int i = 0; i < n_tiles; ++i) {
    const int s = i % kStages;
    const uint32_t phase = (i / kStages) & 1;
    const int tok0 = start + i * kTile;
    mbar_wait_bounded(&full_bar[s], phase, abort_flag, kStatusAttnTimeout);
    uint8_t* ktile = smem + s * C::kStageBytes;
    uint8_t* vtile = ktile + C::kTileBytes;

    if (owns_new && new_pos >= tok0 + r0 && new_pos < tok0 + r0 + 16) {
      // This warp's slice contains the new token: rotate k, store k and v to the pool and patch the tile.
      const int rr = new_pos - tok0;
      const __nv_bfloat16* kn = qkv_t + G * D;
      const __nv_bfloat16* vn = kn + D;
      const int64_t slot = (p.chunk_idx[t] * p.chunk + p.local_pos[t]) * p.nkv + h;
      const bool rope = p.cos != nullptr;
      const int64_t pk = rope ? p.pos_k[t] : 0;
      for (int j = lane * 2; j < D / 2; j += 64) {
        float a1 = __bfloat162float(kn[j]), a2 = __bfloat162float(kn[j + D / 2]);
        float b1 = __bfloat162float(kn[j + 1]), b2 = __bfloat162float(kn[j + 1 + D / 2]);
        if (rope) {
          const __nv_bfloat16* cs = p.cos + pk * (D / 2);
          const __nv_bfloat16* sn = p.sin + pk * (D / 2);
          rope_pair(a1, a2, __bfloat162float(cs[j]), __bfloat162float(sn[j]), a1, a2);
          rope_pair(b1, b2, __bfloat162float(cs[j + 1]), __bfloat162float(sn[j + 1]), b1, b2);
        }
        // elements (j, j+1) and (j+D/2, j+1+D/2) of the rotated key and of the value
        __nv_bfloat16* kg = p.k_cache + slot * D;
        __nv_bfloat16* vg = p.v_cache + slot * D;
        const uint32_t lo = pack_bf16x2(a1, b1);
        const uint32_t hi = pack_bf16x2(a2, b2);
        const uint32_t vlo = *reinterpret_cast<const uint32_t*>(&vn[j]);
        const uint32_t vhi = *reinterpret_cast<const uint32_t*>(&vn[j + D / 2]);
        *reinterpret_cast<uint32_t*>(&kg[j]) = lo;
        *reinterpret_cast<uint32_t*>(&kg[j + D / 2]) = hi;
        *reinterpret_cast<uint32_t*>(&vg[j]) = vlo;
        *reinterpret_cast<uint32_t*>(&vg[j + D / 2]) = vhi;
        const int e[2] = {j, j + D / 2};
        const uint32_t kv[2] = {lo, hi};
        const uint32_t vv[2] = {vlo, vhi};
#pragma unroll
        for (int q = 0; q < 2; ++q) {
          const int sub = e[q] >> 6;
          const int byte = (e[q] & 63) * 2;
          const int off = sub * C::kSubBytes + rr * 128 + ((((byte >> 4) ^ (rr & 7)) << 4) | (byte & 15));
          *reinterpret_cast<uint32_t*>(ktile + off) = kv[q];
          *reinterpret_cast<uint32_t*>(vtile + off) = vv[q];
        }
      }
      __syncwarp();
    }

    if (tok0 + r0 < end) {
      // ---- S = Q K^T for this warp's 16 tokens ----
      float sacc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
      const int ld_row = r0 + ((lane >> 4) << 3) + (lane & 7);  // token row this lane addresses
      const int ld_kh = (lane >> 3) & 1;
      const uint32_t kbase = smem_u32(ktile) + ld_row * 128;
#pragma unroll
      for (int ks = 0; ks < D / 16; ++ks) {
        const int chunk16 = (ks * 2 + ld_kh) & 7;
        const int sub = (ks * 2) >> 3;
        uint32_t b0, b1, b2, b3;
        ldmatrix_x4(kbase + sub * C::kSubBytes + ((chunk16 ^ (ld_row & 7)) << 4), b0, b1, b2, b3);
        mma_bf16_16816(sacc[0], qf[ks], b0, b1);
        mma_bf16_16816(sacc[1], qf[ks], b2, b3);
      }
      // ---- online softmax (log2 domain) ----
      float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const int tok = tok0 + r0 + nt * 8 + tig * 2 + (c & 1);
          float v = sacc[nt][c] * scale_log2;
          if (tok >= end) v = -INFINITY;
          sacc[nt][c] = v;
          mx[c >> 1] = fmaxf(mx[c >> 1], v);
        }
      }
      float alpha[2], m_use[2];
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
        const float m_new = fmaxf(m_run[r], mx[r]);
        m_use[r] = (m_new == -INFINITY) ? 0.f : m_new;
        alpha[r] = exp2f(m_run[r] - m_use[r]);
        m_run[r] = m_new;
        l_run[r] *= alpha[r];
      }
      // P is fed to the tensor cores as hi + lo bf16 terms (two MMAs per V fragment): the bf16 rounding
      // of P alone would cost ~2e-3 relative accuracy per output; the pair keeps 16 bits (~2e-4 after the
      // output rounding).  A third term was measured: +5 us per launch for no visible gain downstream.
      uint32_t pf[4], pl[4];
      {
        float pv[2][4], pr[2][4];
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            pv[nt][c] = exp2f(sacc[nt][c] - m_use[c >> 1]);
            l_run[c >> 1] += pv[nt][c];
            pr[nt][c] = pv[nt][c] - bf16_round(pv[nt][c]);
          }
        }
        pf[0] = pack_bf16x2(pv[0][0], pv[0][1]);
        pf[1] = pack_bf16x2(pv[0][2], pv[0][3]);
        pf[2] = pack_bf16x2(pv[1][0], pv[1][1]);
        pf[3] = pack_bf16x2(pv[1][2], pv[1][3]);
        pl[0] = pack_bf16x2(pr[0][0], pr[0][1]);
        pl[1] = pack_bf16x2(pr[0][2], pr[0][3]);
        pl[2] = pack_bf16x2(pr[1][0], pr[1][1]);
        pl[3] = pack_bf16x2(pr[1][2], pr[1][3]);
      }
#pragma unroll
      for (int i2 = 0; i2 < D / 8; ++i2) {
        oacc[i2][0] *= alpha[0];
        oacc[i2][1] *= alpha[0];
        oacc[i2][2] *= alpha[1];
        oacc[i2][3] *= alpha[1];
      }
      // ---- O += P V ----
      const int v_row = r0 + (((lane >> 3) & 1) << 3) + (lane & 7);
      const int v_dh = lane >> 4;
      const uint32_t vbase = smem_u32(vtile) + v_row * 128;
#pragma unroll
      for (int dn = 0; dn < D / 16; ++dn) {
        const int chunk16 = (dn * 2 + v_dh) & 7;
        const int sub = (dn * 2) >> 3;
        uint32_t b0, b1, b2, b3;
        ldmatrix_x4_trans(vbase + sub * C::kSubBytes + ((chunk16 ^ (v_row & 7)) << 4), b0, b1, b2, b3);
        mma_bf16_16816(oacc[dn * 2], pf, b0, b1);
        mma_bf16_16816(oacc[dn * 2], pl, b0, b1);
        mma_bf16_16816(oacc[dn * 2 + 1], pf, b2, b3);
        mma_bf16_16816(oacc[dn * 2 + 1], pl, b2, b3);
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&empty_bar[s]);
  }

  // ------------------------------ merge the four warps ------------------------------
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
  }
  consumer_barrier();  // every warp is done with the tile ring; reuse it
  float* mo = reinterpret_cast<float*>(smem);                 // [warp][16][D]
  float* mm = mo + kConsumerWarps * 16 * D;                   // [warp][16]
  float* ml = mm + kConsumerWarps * 16;                       // [warp][16]
#pragma unroll
  for (int i2 = 0; i2 < D / 8; ++i2) {
    const int col = i2 * 8 + tig * 2;
    float* o0 = mo + (warp * 16 + gid) * D + col;
    float* o1 = mo + (warp * 16 + gid + 8) * D + col;
    o0[0] = oacc[i2][0];
    o0[1] = oacc[i2][1];
    o1[0] = oacc[i2][2];
    o1[1] = oacc[i2][3];
  }
  if (tig == 0) {
    mm[warp * 16 + gid] = m_run[0];
    mm[warp * 16 + gid + 8] = m_run[1];
    ml[warp * 16 + gid] = l_run[0];
    ml[warp * 16 + gid + 8] = l_run[1];
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
    const float o = lsum > 0.f ? acc / lsum : 0.f;
    const int64_t qh = static_cast<int64_t>(t) * p.nq + h * G + g;
    if (p.num_splits == 1) {
      store_output<D>(p, t, h * G + g, d, o, ml + kConsumerWarps * 16, consumer_barrier);
    } else {
      p.ws_o[(qh * p.num_splits + split) * D + d] = o;
      if (d == 0) p.ws_lse[qh * p.num_splits + split] = lsum > 0.f ? m + log2f(lsum) : -INFINITY;
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Prefill / mixed steps: a block of consecutive query tokens of one request shares every K/V tile.
//
// One CTA = (unit, KV head); a unit is (block-table row, first token, number of tokens <= 64 / G) from a
// list the host builds per step.  The 64 MMA rows are (token j, group head g) pairs, row = j * G + g, so
// each of the four consumer warps owns 16 rows and the whole 64-token tile: S = Q K^T (8 n-tiles), per-row
// causal limit kv_seq_lengths[token], online softmax, O += P V - no cross-warp merge.  Compared with one
// CTA per token (the decode kernel used row-wise) a K/V tile is read once per 64 / G tokens instead of
// once per token.  Keys and values are already in the pool (b200_rope_append ran before); the queries are
// rotated here, in registers.  bf16 pool only.
// ---------------------------------------------------------------------------------------------
template <int D>
__global__ void __launch_bounds__(kThreads, 2)
paged_prefill_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v, Params p,
                     const int32_t* __restrict__ units) {
  using C = Cfg<D>;
  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;

  pdl_launch_dependents();
  const int h = blockIdx.x % p.nkv;
  const int32_t* unit = units + 4 * (blockIdx.x / p.nkv);
  const int row = unit[0];
  const int t0 = unit[1];
  const int n_tok = unit[2];
  const int G = p.G;
  const int qb = 64 / G;  // tokens per unit
  if (n_tok <= 0 || n_tok > qb || t0 < 0 || t0 + n_tok > p.T) {  // padding entry (or a malformed one)
    pdl_wait();
    return;
  }
  int max_kv = 0;
  for (int j = 0; j < n_tok; ++j) max_kv = max(max_kv, p.kv_len[t0 + j]);
  const int n_tiles = (max_kv + kTile - 1) / kTile;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + kStages * C::kStageBytes);
  uint64_t* empty_bar = full_bar + kStages;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(empty_bar + kStages);

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
    if (lane == 0) {
      pdl_wait();  // the append kernel before us writes the pool
      const int32_t* bt_row = p.block_table + static_cast<int64_t>(row) * p.max_chunks;
      int cur_c = -1, cur_id = 0;
      for (int i = 0; i < n_tiles; ++i) {
        const int s = i % kStages;
        const uint32_t phase = (i / kStages) & 1;
        const int tok0 = i * kTile;
        const int c = tok0 / p.chunk;
        if (c != cur_c) {
          cur_c = c;
          cur_id = bt_row[c];
        }
        const int tok_row = cur_id * p.chunk + (tok0 - c * p.chunk);
        mbar_wait_bounded(&empty_bar[s], phase ^ 1, abort_flag, kStatusAttnTimeout);
        uint8_t* kdst = smem + s * C::kStageBytes;
        uint8_t* vdst = kdst + C::kTileBytes;
        mbar_arrive_expect_tx(&full_bar[s], C::kStageBytes);
#pragma unroll
        for (int sub = 0; sub < C::kSub; ++sub) {
          tma_load_3d(kdst + sub * C::kSubBytes, &map_k, &full_bar[s], sub * 64, h, tok_row);
          tma_load_3d(vdst + sub * C::kSubBytes, &map_v, &full_bar[s], sub * 64, h, tok_row);
        }
      }
    }
    return;
  }

  // --------------------------------- consumer warps ---------------------------------
  const int gid = lane >> 2;
  const int tig = lane & 3;
  pdl_wait();  // qkv is an earlier kernel's output

  // This thread's two MMA rows: (token, head) and the keys the token may see.
  int tok_r[2], head_r[2], kv_r[2];
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int rho = warp * 16 + gid + r * 8;
    const int j = rho / G;
    head_r[r] = rho - j * G;
    tok_r[r] = j < n_tok ? t0 + j : -1;
    kv_r[r] = j < n_tok ? p.kv_len[t0 + j] : 0;
  }
  // Q fragments straight from global memory, rotated in registers: the thread that holds columns
  // (c, c+1) of a row also holds (c + D/2, c + 1 + D/2), the RoPE partners.
  uint32_t qf[D / 16][4];
#pragma unroll
  for (int ks = 0; ks < D / 16; ++ks) qf[ks][0] = qf[ks][1] = qf[ks][2] = qf[ks][3] = 0u;
  {
    const bool rope = p.cos != nullptr;
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      if (tok_r[r] < 0) continue;
      const __nv_bfloat16* q = p.qkv + (static_cast<int64_t>(tok_r[r]) * p.nkv + h) * (G + 2) * D + head_r[r] * D;
      const int64_t pq = rope ? p.pos_q[tok_r[r]] : 0;
      const __nv_bfloat16* cs = p.cos + pq * (D / 2);
      const __nv_bfloat16* sn = p.sin + pq * (D / 2);
#pragma unroll
      for (int ks = 0; ks < D / 32; ++ks) {
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          const int j = ks * 16 + tig * 2 + half * 8;
          const uint32_t lo = *reinterpret_cast<const uint32_t*>(q + j);
          const uint32_t hi = *reinterpret_cast<const uint32_t*>(q + j + D / 2);
          float a1 = bf16_lo(lo), b1 = bf16_hi(lo), a2 = bf16_lo(hi), b2 = bf16_hi(hi);
          if (rope) {
            const uint32_t c2 = *reinterpret_cast<const uint32_t*>(cs + j);
            const uint32_t s2 = *reinterpret_cast<const uint32_t*>(sn + j);
            rope_pair(a1, a2, bf16_lo(c2), bf16_lo(s2), a1, a2);
            rope_pair(b1, b2, bf16_hi(c2), bf16_hi(s2), b1, b2);
          }
          qf[ks][r + 2 * half] = pack_bf16x2(a1, b1);
          qf[ks + D / 32][r + 2 * half] = pack_bf16x2(a2, b2);
        }
      }
    }
  }

  float oacc[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) oacc[i][0] = oacc[i][1] = oacc[i][2] = oacc[i][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY};
  float l_run[2] = {0.f, 0.f};
  const float scale_log2 = p.scale_log2;
  // keys this warp's rows can see at most (warp-uniform): later tiles are skipped
  int warp_kv = max(kv_r[0], kv_r[1]);
#pragma unroll
  for (int o = 4; o < 32; o <<= 1) warp_kv = max(warp_kv, __shfl_xor_sync(0xffffffffu, warp_kv, o));

  for (int i = 0; i < n_tiles; ++i) {
    const int s = i % kStages;
    const uint32_t phase = (i / kStages) & 1;
    const int tok0 = i * kTile;
    mbar_wait_bounded(&full_bar[s], phase, abort_flag, kStatusAttnTimeout);
    uint8_t* ktile = smem + s * C::kStageBytes;
    uint8_t* vtile = ktile + C::kTileBytes;
    if (tok0 < warp_kv) {
      // ---- S = Q K^T: 16 rows x 64 tokens ----
      float sacc[8][4];
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) sacc[nt][0] = sacc[nt][1] = sacc[nt][2] = sacc[nt][3] = 0.f;
      const int ld_sub = ((lane >> 4) << 3) + (lane & 7);  // token row inside a 16-token slab
      const int ld_kh = (lane >> 3) & 1;
#pragma unroll
      for (int ks = 0; ks < D / 16; ++ks) {
        const int chunk16 = (ks * 2 + ld_kh) & 7;
        const int sub = (ks * 2) >> 3;
#pragma unroll
        for (int slab = 0; slab < 4; ++slab) {
          const int ld_row = slab * 16 + ld_sub;
          uint32_t b0, b1, b2, b3;
          ldmatrix_x4(smem_u32(ktile) + sub * C::kSubBytes + ld_row * 128 + ((chunk16 ^ (ld_row & 7)) << 4), b0, b1, b2, b3);
          mma_bf16_16816(sacc[slab * 2], qf[ks], b0, b1);
          mma_bf16_16816(sacc[slab * 2 + 1], qf[ks], b2, b3);
        }
      }
      // ---- causal mask + online softmax (log2 domain) ----
      float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const int tok = tok0 + nt * 8 + tig * 2 + (c & 1);
          float v = sacc[nt][c] * scale_log2;
          if (tok >= kv_r[c >> 1]) v = -INFINITY;
          sacc[nt][c] = v;
          mx[c >> 1] = fmaxf(mx[c >> 1], v);
        }
      }
      float alpha[2], m_use[2];
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
        const float m_new = fmaxf(m_run[r], mx[r]);
        m_use[r] = (m_new == -INFINITY) ? 0.f : m_new;
        alpha[r] = exp2f(m_run[r] - m_use[r]);
        m_run[r] = m_new;
        l_run[r] *= alpha[r];
      }
#pragma unroll
      for (int i2 = 0; i2 < D / 8; ++i2) {
        oacc[i2][0] *= alpha[0];
        oacc[i2][1] *= alpha[0];
        oacc[i2][2] *= alpha[1];
        oacc[i2][3] *= alpha[1];
      }
      // ---- O += P V, one 16-token slab at a time (P as hi + lo bf16 terms, like the decode kernel) ----
      const int v_sub = (((lane >> 3) & 1) << 3) + (lane & 7);
      const int v_dh = lane >> 4;
#pragma unroll
      for (int slab = 0; slab < 4; ++slab) {
        uint32_t pf[4], pl[4];
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
          float pv[4], pr[4];
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            pv[c] = exp2f(sacc[slab * 2 + nt][c] - m_use[c >> 1]);
            l_run[c >> 1] += pv[c];
            pr[c] = pv[c] - bf16_round(pv[c]);
          }
          pf[nt * 2] = pack_bf16x2(pv[0], pv[1]);
          pf[nt * 2 + 1] = pack_bf16x2(pv[2], pv[3]);
          pl[nt * 2] = pack_bf16x2(pr[0], pr[1]);
          pl[nt * 2 + 1] = pack_bf16x2(pr[2], pr[3]);
        }
        const int v_row = slab * 16 + v_sub;
        const uint32_t vbase = smem_u32(vtile) + v_row * 128;
#pragma unroll
        for (int dn = 0; dn < D / 16; ++dn) {
          const int chunk16 = (dn * 2 + v_dh) & 7;
          const int sub = (dn * 2) >> 3;
          uint32_t b0, b1, b2, b3;
          ldmatrix_x4_trans(vbase + sub * C::kSubBytes + ((chunk16 ^ (v_row & 7)) << 4), b0, b1, b2, b3);
          mma_bf16_16816(oacc[dn * 2], pf, b0, b1);
          mma_bf16_16816(oacc[dn * 2], pl, b0, b1);
          mma_bf16_16816(oacc[dn * 2 + 1], pf, b2, b3);
          mma_bf16_16816(oacc[dn * 2 + 1], pl, b2, b3);
        }
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&empty_bar[s]);
  }

  // ------------------------------ normalise and store ------------------------------
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
    if (tok_r[r] < 0) continue;
    const float inv = l_run[r] > 0.f ? 1.f / l_run[r] : 0.f;  // a token that sees no key gets zeros, as flash-attn does
    __nv_bfloat16* o = p.out + (static_cast<int64_t>(tok_r[r]) * p.nq + h * G + head_r[r]) * D;
#pragma unroll
    for (int i2 = 0; i2 < D / 8; ++i2) {
      const int col = i2 * 8 + tig * 2;
      *reinterpret_cast<uint32_t*>(o + col) = pack_bf16x2(oacc[i2][2 * r] * inv, oacc[i2][2 * r + 1] * inv);
    }
  }
}

// Merge the splits of each (token, query head): out = sum_s 2^(lse_s - max) O_s / sum_s 2^(lse_s - max).
template <int D>
__global__ void __launch_bounds__(D) combine_kernel(Params p) {
  pdl_launch_dependents();
  pdl_wait();
  const int qh = blockIdx.x;  // t * nq + head
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
  store_output<D>(p, t, qh - t * p.nq, d, o, red, [] { __syncthreads(); });
}

// Prefill / mixed steps: rotate k, then scatter k and v of every token into the pool.
template <int D>
__global__ void __launch_bounds__(128) rope_append_kernel(Params p) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int G = p.G;
  const bool rope = p.cos != nullptr;
  const int64_t pk = rope ? p.pos_k[t] : 0;
  const int64_t slot_tok = p.chunk_idx[t] * p.chunk + p.local_pos[t];
  for (int i = threadIdx.x; i < p.nkv * (D / 2); i += blockDim.x) {
    const int h = i / (D / 2);
    const int j = i - h * (D / 2);
    const __nv_bfloat16* kn = p.qkv + (static_cast<int64_t>(t) * p.nkv + h) * (G + 2) * D + G * D;
    const __nv_bfloat16* vn = kn + D;
    float x1 = __bfloat162float(kn[j]);
    float x2 = __bfloat162float(kn[j + D / 2]);
    if (rope)
      rope_pair(x1, x2, __bfloat162float(p.cos[pk * (D / 2) + j]), __bfloat162float(p.sin[pk * (D / 2) + j]), x1, x2);
    const int64_t base = (slot_tok * p.nkv + h) * D;
    p.k_cache[base + j] = __float2bfloat16_rn(x1);
    p.k_cache[base + j + D / 2] = __float2bfloat16_rn(x2);
    p.v_cache[base + j] = vn[j];
    p.v_cache[base + j + D / 2] = vn[j + D / 2];
  }
}

static int fill_params(const b200_attention_args* a, Params& p) {
  if (!a || (!a->qkv && !a->qkv_partials) || !a->k_cache || !a->v_cache || !a->kv_seq_lengths || !a->block_table)
    return B200_ERR_INVALID_ARGUMENT;
  if (a->qkv_partials && (a->qkv_num_splits < 1 || !aligned16(a->qkv_partials))) return B200_ERR_INVALID_ARGUMENT;
  if (a->head_dim != 64 && a->head_dim != 128) return B200_ERR_INVALID_ARGUMENT;
  if (a->num_tokens <= 0 || a->num_kv_heads <= 0 || a->num_q_heads % a->num_kv_heads != 0)
    return B200_ERR_INVALID_ARGUMENT;
  const int G = a->num_q_heads / a->num_kv_heads;
  if (G < 1 || G > 16) return B200_ERR_INVALID_ARGUMENT;
  if (a->chunk_size <= 0 || a->chunk_size % kTile != 0 || a->num_chunks <= 0) return B200_ERR_INVALID_ARGUMENT;
  if (a->num_splits < 1 || a->num_splits > kMaxSplits) return B200_ERR_INVALID_ARGUMENT;
  if ((a->rope_cos == nullptr) != (a->rope_sin == nullptr)) return B200_ERR_INVALID_ARGUMENT;
  if (a->rope_cos && (!a->token_to_pos_ids || !a->token_to_pos_in_request)) return B200_ERR_INVALID_ARGUMENT;
  if (!aligned16(a->k_cache) || !aligned16(a->v_cache) || (a->qkv && !aligned16(a->qkv))) return B200_ERR_ALIGNMENT;
  p.qkv = static_cast<const __nv_bfloat16*>(a->qkv);
  p.qkv_partials = a->qkv_partials;
  p.qkv_splits = a->qkv_num_splits;
  p.k_cache = static_cast<__nv_bfloat16*>(a->k_cache);
  p.v_cache = static_cast<__nv_bfloat16*>(a->v_cache);
  p.block_table = a->block_table;
  p.kv_len = a->kv_seq_lengths;
  p.row_of_token = a->row_of_token;
  p.row_order = a->row_order;
  p.pos_q = a->token_to_pos_ids;
  p.pos_k = a->token_to_pos_in_request;
  p.chunk_idx = a->token_to_chunk_idx;
  p.local_pos = a->token_to_local_pos;
  p.cos = static_cast<const __nv_bfloat16*>(a->rope_cos);
  p.sin = static_cast<const __nv_bfloat16*>(a->rope_sin);
  p.out = static_cast<__nv_bfloat16*>(a->out);
  p.out_q = static_cast<uint8_t*>(a->out_q);
  p.out_sf = a->out_scales;
  p.out_q_mode = a->out_q_mode;
  p.out_m_pad = a->out_m_pad;
  if (a->out_q != nullptr) {
    const int64_t width = static_cast<int64_t>(a->num_q_heads) * a->head_dim;
    if (!a->out_scales || !aligned16(a->out_q) || !aligned16(a->out_scales) || width % 128 != 0)
      return B200_ERR_INVALID_ARGUMENT;
    if (a->out_q_mode == mx::kQuantBlock128) {
      if (a->head_dim != 128 || a->out_m_pad < a->num_tokens || a->out_m_pad % 4 != 0) return B200_ERR_INVALID_ARGUMENT;
    } else if (a->out_q_mode != mx::kQuantMx) {
      return B200_ERR_INVALID_ARGUMENT;
    }
  }
  p.T = a->num_tokens;
  p.nq = a->num_q_heads;
  p.nkv = a->num_kv_heads;
  p.G = G;
  p.chunk = a->chunk_size;
  p.num_chunks = a->num_chunks;
  p.max_chunks = a->max_chunks_per_row;
  p.num_splits = a->num_splits;
  p.fused = a->fuse_rope_append;
  p.min_split = a->chunk_size < 256 ? a->chunk_size : 256;
  const float scale = a->softmax_scale > 0.f ? a->softmax_scale : 1.0f / sqrtf(static_cast<float>(a->head_dim));
  p.scale_log2 = scale * 1.4426950408889634f;
  p.ws_o = nullptr;
  p.ws_lse = nullptr;
  p.k_scale = a->k_scale;
  p.v_scale = a->v_scale;
  if (a->kv_cache_fp8) {
    if (a->head_dim != 128 || !a->k_scale || !a->v_scale || !a->qkv || a->chunk_size % 128 != 0) return B200_ERR_INVALID_ARGUMENT;
  }
  return B200_OK;
}

template <int D>
static int launch_attention(const b200_attention_args* a, Params& p, cudaStream_t stream) {
  using C = Cfg<D>;
  constexpr int kElem = 2;
  const uint64_t dims[3] = {static_cast<uint64_t>(D), static_cast<uint64_t>(p.nkv),
                            static_cast<uint64_t>(p.num_chunks) * p.chunk};
  const uint64_t strides[2] = {static_cast<uint64_t>(D) * kElem, static_cast<uint64_t>(p.nkv) * D * kElem};
  const uint32_t box[3] = {64u, 1, kTile};
  const CUtensorMapDataType dt = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  const CUtensorMap* mk = get_tensor_map(p.k_cache, 3, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B,
                                         CU_TENSOR_MAP_L2_PROMOTION_L2_256B, dt);
  const CUtensorMap* mv = get_tensor_map(p.v_cache, 3, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B,
                                         CU_TENSOR_MAP_L2_PROMOTION_L2_256B, dt);
  if (!mk || !mv) return B200_ERR_DRIVER;
  static std::atomic<uint64_t> smem_attr_done{0};
  if (ensure_dynamic_smem(paged_attention_kernel<D>, C::kSmemBytes, smem_attr_done) != B200_OK) return B200_ERR_LAUNCH;
  const int64_t units = static_cast<int64_t>(p.T) * p.nkv * p.num_splits;
  if (units > 0x7fffffff) return B200_ERR_INVALID_ARGUMENT;
  int rc = launch_pdl(paged_attention_kernel<D>, dim3(static_cast<unsigned>(units)), dim3(kThreads), C::kSmemBytes,
                      stream, *mk, *mv, p);
  if (rc != B200_OK) return rc;
  if (p.num_splits > 1) rc = launch_pdl(combine_kernel<D>, dim3(p.T * p.nq), dim3(D), 0, stream, p);
  return rc;
}

template <int D>
static int launch_prefill(Params& p, const int32_t* units, int num_units, cudaStream_t stream) {
  using C = Cfg<D>;
  const uint64_t dims[3] = {static_cast<uint64_t>(D), static_cast<uint64_t>(p.nkv),
                            static_cast<uint64_t>(p.num_chunks) * p.chunk};
  const uint64_t strides[2] = {static_cast<uint64_t>(D) * 2, static_cast<uint64_t>(p.nkv) * D * 2};
  const uint32_t box[3] = {64u, 1, kTile};
  const CUtensorMap* mk = get_tensor_map(p.k_cache, 3, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B,
                                         CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16);
  const CUtensorMap* mv = get_tensor_map(p.v_cache, 3, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B,
                                         CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16);
  if (!mk || !mv) return B200_ERR_DRIVER;
  static std::atomic<uint64_t> smem_attr_done{0};
  if (ensure_dynamic_smem(paged_prefill_kernel<D>, C::kSmemBytes, smem_attr_done) != B200_OK) return B200_ERR_LAUNCH;
  const int64_t ctas = static_cast<int64_t>(num_units) * p.nkv;
  if (ctas > 0x7fffffff) return B200_ERR_INVALID_ARGUMENT;
  return launch_pdl(paged_prefill_kernel<D>, dim3(static_cast<unsigned>(ctas)), dim3(kThreads), C::kSmemBytes, stream, *mk,
                    *mv, p, units);
}

}  // namespace attn

// E4M3 pool: kernels of attention_fp8.cu (same translation unit, compiled after this file)
namespace attn8 {
static int launch_attention_fp8(attn::Params& p, bool two_terms, cudaStream_t stream);
__global__ void rope_append_fp8_kernel(attn::Params p);
}  // namespace attn8
}  // namespace b200

extern "C" {

int b200_paged_prefill_attention(const b200_attention_args* a, const int32_t* units, int num_units,
                                 b200_stream_t stream) {
  using namespace b200;
  attn::Params p;
  int rc = attn::fill_params(a, p);
  if (rc != B200_OK) return rc;
  if (!a->out || a->out_q || !a->qkv || !units || num_units <= 0 || a->kv_cache_fp8) return B200_ERR_INVALID_ARGUMENT;
  if (64 % p.G != 0) return B200_ERR_INVALID_ARGUMENT;  // group sizes 1, 2, 4, 8, 16
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  return a->head_dim == 128 ? attn::launch_prefill<128>(p, units, num_units, s)
                            : attn::launch_prefill<64>(p, units, num_units, s);
}

size_t b200_paged_attention_workspace_bytes(int num_tokens, int num_q_heads, int head_dim, int num_splits) {
  if (num_splits <= 1 || num_tokens <= 0 || num_q_heads <= 0 || head_dim <= 0) return 0;
  const size_t rows = static_cast<size_t>(num_tokens) * num_q_heads * num_splits;
  return rows * head_dim * sizeof(float) + rows * sizeof(float);
}

int b200_rope_append(const b200_attention_args* a, b200_stream_t stream) {
  using namespace b200;
  attn::Params p;
  int rc = attn::fill_params(a, p);
  if (rc != B200_OK) return rc;
  if (!a->token_to_chunk_idx || !a->token_to_local_pos || !a->qkv) return B200_ERR_INVALID_ARGUMENT;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (a->kv_cache_fp8) return launch_pdl(attn8::rope_append_fp8_kernel, dim3(p.T), dim3(128), 0, s, p);
  if (a->head_dim == 128) return launch_pdl(attn::rope_append_kernel<128>, dim3(p.T), dim3(128), 0, s, p);
  return launch_pdl(attn::rope_append_kernel<64>, dim3(p.T), dim3(128), 0, s, p);
}

int b200_paged_attention(const b200_attention_args* a, b200_stream_t stream) {
  using namespace b200;
  attn::Params p;
  int rc = attn::fill_params(a, p);
  if (rc != B200_OK) return rc;
  if (!a->out && !a->out_q) return B200_ERR_INVALID_ARGUMENT;
  if (a->fuse_rope_append && (!a->token_to_chunk_idx || !a->token_to_local_pos)) return B200_ERR_INVALID_ARGUMENT;
  if (a->qkv_partials && (a->num_q_heads / a->num_kv_heads + 2) * a->head_dim % 4 != 0) return B200_ERR_ALIGNMENT;
  if (a->num_splits > 1) {
    const size_t need =
        b200_paged_attention_workspace_bytes(a->num_tokens, a->num_q_heads, a->head_dim, a->num_splits);
    if (!a->workspace || a->workspace_bytes < need) return B200_ERR_WORKSPACE;
    p.ws_o = static_cast<float*>(a->workspace);
    p.ws_lse = p.ws_o + static_cast<size_t>(a->num_tokens) * a->num_q_heads * a->num_splits * a->head_dim;
  }
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (a->kv_cache_fp8) return attn8::launch_attention_fp8(p, a->kv_cache_fp8 != 2, s);
  return a->head_dim == 128 ? attn::launch_attention<128>(a, p, s) : attn::launch_attention<64>(a, p, s);
}

}  // extern "C"
