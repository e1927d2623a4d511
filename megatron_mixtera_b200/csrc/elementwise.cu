// Memory-bound row kernels of the decode step: embedding / row gather, fused residual-add +
// RMSNorm / LayerNorm, SwiGLU / GELU.  All use 16-byte vector accesses; one CTA per token row.
#include "common.cuh"
#include "quant.cuh"

namespace b200 {
namespace ew {

struct alignas(16) Vec8 {
  uint32_t w[4];  // 8 bf16
};

__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nw = (blockDim.x + 31) >> 5;
  __syncthreads();  // protect `red` against the previous use
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = lane < nw ? red[lane] : 0.f;
  return warp_sum(t);
}

// out[i] = table[ids[i] - lo] (zero outside [lo, hi)) (+ add_table[add_ids[i]], bf16 add)
__global__ void gather_rows_kernel(const __nv_bfloat16* __restrict__ table, const int64_t* __restrict__ ids,
                                   __nv_bfloat16* __restrict__ out, int row_elems, int64_t lo, int64_t hi,
                                   const __nv_bfloat16* __restrict__ add_table, const int64_t* __restrict__ add_ids) {
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x;
  const int64_t id = ids[r];
  const bool in_range = id >= lo && id < hi;
  const Vec8* src = reinterpret_cast<const Vec8*>(table + (in_range ? (id - lo) : 0) * row_elems);
  const Vec8* add = add_table ? reinterpret_cast<const Vec8*>(add_table + add_ids[r] * row_elems) : nullptr;
  Vec8* dst = reinterpret_cast<Vec8*>(out + static_cast<int64_t>(r) * row_elems);
  for (int i = threadIdx.x; i < row_elems / 8; i += blockDim.x) {
    Vec8 v;
    if (in_range) {
      v = src[i];
    } else {
      v.w[0] = v.w[1] = v.w[2] = v.w[3] = 0u;
    }
    if (add) {
      const Vec8 a = add[i];
#pragma unroll
      for (int k = 0; k < 4; ++k)
        v.w[k] = pack_bf16x2(bf16_lo(v.w[k]) + bf16_lo(a.w[k]), bf16_hi(v.w[k]) + bf16_hi(a.w[k]));
    }
    dst[i] = v;
  }
}

// Source "peers": x is the sum over the tensor-parallel ranks of each rank's bf16 partial output row (the
// all-reduce of RowParallelLinear), read straight from the peers' memory.
struct PeerSrc {
  const __nv_bfloat16* data[8];  // slot base of every rank's partial output [max_rows][hidden]; data[rank] is local
  int32_t* flags[8];             // every rank's flag array [world][max_rows]; flags[rank] is local
  int32_t* counters;             // local: [0] = calls completed, [1] = CTAs that finished the running call
  int world, rank, max_rows;
};

__device__ __forceinline__ void st_release_sys(int32_t* p, int32_t v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int32_t ld_acquire_sys(const int32_t* p) {
  int32_t v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Row handshake of one all-reduce call: tell every peer that this rank's row is complete, then wait (bounded)
// until every peer has said the same.  Flags carry the call number (monotonic), so nothing is ever reset; a
// peer can be at most one call ahead, which only makes its flag larger.
// The flag accesses are relaxed (system scope), without fences: the row a flag announces was written by an EARLIER
// kernel of this stream, whose completion - memory included - griddepcontrol.wait has awaited before this code runs;
// it sits in this GPU's L2, which is where a peer's load over NVLink is served.  A release store here would add a
// system-scope fence per flag: measured 16.1 us per call against 8.2 us (2 ranks, 128 x 4096).  In the other
// direction a peer announces call c + 1 only from the kernel after the one whose loads of call c's slot have returned,
// which is all the slot alternation needs.
__device__ __forceinline__ void st_relaxed_sys(int32_t* p, int32_t v) {
  asm volatile("st.relaxed.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int32_t ld_relaxed_sys(const int32_t* p) {
  int32_t v;
  asm volatile("ld.relaxed.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// Called by every thread of the CTA; thread q < world talks to rank q (its flag store and its polls are then one
// NVLink / L2 round trip in parallel with the other peers', not `world - 1` of them in a row), the caller's CTA barrier
// ends the handshake.
__device__ __forceinline__ void peer_row_handshake(const PeerSrc& ps, int row) {
  const int q = threadIdx.x;
  if (q >= ps.world || q == ps.rank) return;
  const int32_t call = ld_relaxed_sys(ps.counters) + 1;  // every CTA reads the same value: it moves when all are done
  st_relaxed_sys(ps.flags[q] + ps.rank * ps.max_rows + row, call);
  const int32_t* mine = ps.flags[ps.rank] + q * ps.max_rows + row;
  const uint64_t t0 = global_timer_ns();
  while (ld_relaxed_sys(mine) < call) {
    if (global_timer_ns() - t0 > g_wait_limit_ns) {  // give up, flag it, carry on with what is there
      atomicOr(&g_device_status, kStatusPeerTimeout);
      return;
    }
    __nanosleep(32);
  }
}

// h = x (+bias) (+residual) with a bf16 rounding after each add; normed = norm(h) * gamma (+beta).
// kMaxVec: vectors of 8 elements cached per thread so that the row is read once.
// kPartials: x is not read; it is bf16(sum over the `splits` fp32 partial products of a split-K GEMM, in split
// order) - the reduction the GEMM's own second kernel would have done, so that kernel is not launched.  One
// vector per thread and up to 1024 threads, so that all partial loads of a row are in flight at once.
// kSrc 2 ("peers"): x = bf16(sum over the tensor-parallel ranks, in rank order, of their bf16 rows), after the
// row handshake above; every rank computes the same bits.
template <int kMaxVec, int kSrc>
__global__ void __launch_bounds__(kSrc != 0 ? 1024 : 256)
add_norm_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ bias,
                const __nv_bfloat16* __restrict__ residual, const __nv_bfloat16* __restrict__ gamma,
                const __nv_bfloat16* __restrict__ beta, __nv_bfloat16* __restrict__ hidden_out,
                __nv_bfloat16* __restrict__ normed_out, int hidden, float eps, uint8_t* __restrict__ q_out,
                void* __restrict__ sf_out, int q_mode, int m_pad, const float* __restrict__ partials, int splits,
                int64_t split_stride, PeerSrc ps) {
  __shared__ float red[32];
  pdl_launch_dependents();
  pdl_wait();
  if constexpr (kSrc == 2) {
    peer_row_handshake(ps, blockIdx.x);
    __syncthreads();
  }
  // peers: the call counter moves on when the last CTA of this launch is done with the peers' rows
  auto finish = [&]() {
    if constexpr (kSrc == 2) {
      __syncthreads();
      if (threadIdx.x == 0) {
        if (atomicAdd(&ps.counters[1], 1) == static_cast<int>(gridDim.x) - 1) {
          ps.counters[1] = 0;
          __threadfence();
          atomicAdd(&ps.counters[0], 1);
        }
      }
    }
  };
  const int64_t off = static_cast<int64_t>(blockIdx.x) * hidden;
  const Vec8* xv = reinterpret_cast<const Vec8*>(x + off);
  const Vec8* rv = residual ? reinterpret_cast<const Vec8*>(residual + off) : nullptr;
  const Vec8* bv = bias ? reinterpret_cast<const Vec8*>(bias) : nullptr;
  const int nvec = hidden / 8;
  float vals[kMaxVec][8];
  float sum = 0.f, sumsq = 0.f;
#pragma unroll
  for (int it = 0; it < kMaxVec; ++it) {
    const int i = threadIdx.x + it * blockDim.x;
    if (i < nvec) {
      float f[8];
      if constexpr (kSrc == 2) {
        // all peers' vectors are requested before any is used: one NVLink round trip, not `world` of them
        uint4 u[8];
#pragma unroll
        for (int q = 0; q < 8; ++q)
          if (q < ps.world) u[q] = __ldcg(reinterpret_cast<const uint4*>(ps.data[q] + off) + i);
#pragma unroll
        for (int k = 0; k < 8; ++k) f[k] = 0.f;
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          if (q < ps.world) {  // rank order: every rank adds in the same order
            const uint32_t w4[4] = {u[q].x, u[q].y, u[q].z, u[q].w};
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              f[2 * k] += bf16_lo(w4[k]);
              f[2 * k + 1] += bf16_hi(w4[k]);
            }
          }
        }
#pragma unroll
        for (int k = 0; k < 8; ++k) f[k] = bf16_round(f[k]);
      } else if constexpr (kSrc == 1) {
        const float4* src = reinterpret_cast<const float4*>(partials + off) + 2 * i;
        const int64_t stride4 = split_stride / 4;
        float4 a = make_float4(0.f, 0.f, 0.f, 0.f), b = a;
#pragma unroll 8
        for (int sp = 0; sp < splits; ++sp) {
          const float4 u = __ldcg(src + sp * stride4);
          const float4 w = __ldcg(src + sp * stride4 + 1);
          a.x += u.x; a.y += u.y; a.z += u.z; a.w += u.w;
          b.x += w.x; b.y += w.y; b.z += w.z; b.w += w.w;
        }
        f[0] = bf16_round(a.x); f[1] = bf16_round(a.y); f[2] = bf16_round(a.z); f[3] = bf16_round(a.w);
        f[4] = bf16_round(b.x); f[5] = bf16_round(b.y); f[6] = bf16_round(b.z); f[7] = bf16_round(b.w);
      } else {
        const Vec8 v = xv[i];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          f[2 * k] = bf16_lo(v.w[k]);
          f[2 * k + 1] = bf16_hi(v.w[k]);
        }
      }
      if (bv) {
        const Vec8 b = bv[i];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          f[2 * k] = bf16_round(f[2 * k] + bf16_lo(b.w[k]));
          f[2 * k + 1] = bf16_round(f[2 * k + 1] + bf16_hi(b.w[k]));
        }
      }
      if (rv) {
        const Vec8 r = rv[i];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          f[2 * k] = bf16_round(f[2 * k] + bf16_lo(r.w[k]));
          f[2 * k + 1] = bf16_round(f[2 * k + 1] + bf16_hi(r.w[k]));
        }
      }
      if (hidden_out) {
        Vec8 o;
#pragma unroll
        for (int k = 0; k < 4; ++k) o.w[k] = pack_bf16x2(f[2 * k], f[2 * k + 1]);
        reinterpret_cast<Vec8*>(hidden_out + off)[i] = o;
      }
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        vals[it][k] = f[k];
        sum += f[k];
        sumsq += f[k] * f[k];
      }
    }
  }
  if (normed_out == nullptr && q_out == nullptr) {
    finish();
    return;
  }
  float mean = 0.f, rstd;
  if (beta != nullptr) {  // LayerNorm: two-pass variance on the cached values
    mean = block_sum(sum, red) / hidden;
    float var = 0.f;
#pragma unroll
    for (int it = 0; it < kMaxVec; ++it) {
      const int i = threadIdx.x + it * blockDim.x;
      if (i < nvec) {
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const float d = vals[it][k] - mean;
          var += d * d;
        }
      }
    }
    rstd = rsqrtf(block_sum(var, red) / hidden + eps);
  } else {
    rstd = rsqrtf(block_sum(sumsq, red) / hidden + eps);
  }
  const Vec8* gv = reinterpret_cast<const Vec8*>(gamma);
  const Vec8* betav = beta ? reinterpret_cast<const Vec8*>(beta) : nullptr;
#pragma unroll
  for (int it = 0; it < kMaxVec; ++it) {
    const int i = threadIdx.x + it * blockDim.x;
    const bool valid = i < nvec;
    float y[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    if (valid) {
      const Vec8 g = gv[i];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        y[2 * k] = (vals[it][2 * k] - mean) * rstd * bf16_lo(g.w[k]);
        y[2 * k + 1] = (vals[it][2 * k + 1] - mean) * rstd * bf16_hi(g.w[k]);
      }
      if (betav) {
        const Vec8 b = betav[i];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          y[2 * k] += bf16_lo(b.w[k]);
          y[2 * k + 1] += bf16_hi(b.w[k]);
        }
      }
      if (normed_out) {
        Vec8 o;
#pragma unroll
        for (int k = 0; k < 4; ++k) o.w[k] = pack_bf16x2(y[2 * k], y[2 * k + 1]);
        reinterpret_cast<Vec8*>(normed_out + off)[i] = o;
      }
    }
    if (q_out) {  // quantise the bf16-rounded normalised row (what an unfused quantiser would read)
#pragma unroll
      for (int k = 0; k < 8; ++k) y[k] = bf16_round(y[k]);
      mx::quantize8_any(q_mode, y, valid, blockIdx.x, i * 8, q_out, hidden, sf_out, hidden / 128, m_pad);
    }
  }
  finish();
}

__device__ __forceinline__ float silu_f(float x) { return x / (1.f + expf(-x)); }
__device__ __forceinline__ float gelu_erf_f(float x) { return 0.5f * x * (1.f + erff(x * 0.70710678118654752f)); }

// kind 0: out = bf16(bf16(silu(gate)) * up); kind 1: out = bf16(gelu(bf16(in + bias)))
// kind 2: SwiGLU on the layout of the fused-epilogue weights: of every 128 input columns the first 64 are gate
// features, the last 64 the matching up features.
// x = bf16(sum over the splits, in split order, of 8 consecutive fp32 partial sums): what the GEMM's own reduction
// kernel would have written.
__device__ __forceinline__ Vec8 sum_partials8(const float* __restrict__ src, int splits, int64_t split_stride) {
  float4 a = make_float4(0.f, 0.f, 0.f, 0.f), b = a;
#pragma unroll 4
  for (int sp = 0; sp < splits; ++sp) {
    const float4 u = __ldcg(reinterpret_cast<const float4*>(src + sp * split_stride));
    const float4 w = __ldcg(reinterpret_cast<const float4*>(src + sp * split_stride) + 1);
    a.x += u.x; a.y += u.y; a.z += u.z; a.w += u.w;
    b.x += w.x; b.y += w.y; b.z += w.z; b.w += w.w;
  }
  Vec8 o;
  o.w[0] = pack_bf16x2(a.x, a.y);
  o.w[1] = pack_bf16x2(a.z, a.w);
  o.w[2] = pack_bf16x2(b.x, b.y);
  o.w[3] = pack_bf16x2(b.z, b.w);
  return o;
}

__global__ void activation_kernel(const __nv_bfloat16* __restrict__ in, const __nv_bfloat16* __restrict__ bias,
                                  __nv_bfloat16* __restrict__ out, int F, int kind, uint8_t* __restrict__ q_out,
                                  void* __restrict__ sf_out, int q_mode, int m_pad, const float* __restrict__ partials,
                                  int splits, int64_t split_stride) {
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x;
  const int nvec = F / 8;
  const int i = blockIdx.y * blockDim.x + threadIdx.x;
  const bool valid = i < nvec;
  Vec8 o;
  o.w[0] = o.w[1] = o.w[2] = o.w[3] = 0u;
  if (!valid) {
  } else if (kind == 0 || kind == 2) {
    const int gi = kind == 0 ? i : ((i >> 3) << 4) + (i & 7);  // 8 vectors = 64 features per half tile
    const int ui = kind == 0 ? nvec + i : gi + 8;
    Vec8 g, u;
    if (partials != nullptr) {  // the fc1 GEMM left its split-K partial sums: reduce them here
      const float* row = partials + static_cast<int64_t>(r) * 2 * F;
      g = sum_partials8(row + gi * 8, splits, split_stride);
      u = sum_partials8(row + ui * 8, splits, split_stride);
    } else {
      const Vec8* row = reinterpret_cast<const Vec8*>(in + static_cast<int64_t>(r) * 2 * F);
      g = row[gi];
      u = row[ui];
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float a = bf16_round(silu_f(bf16_lo(g.w[k]))) * bf16_lo(u.w[k]);
      const float b = bf16_round(silu_f(bf16_hi(g.w[k]))) * bf16_hi(u.w[k]);
      o.w[k] = pack_bf16x2(a, b);
    }
  } else {
    const Vec8 v = partials != nullptr ? sum_partials8(partials + static_cast<int64_t>(r) * F + i * 8, splits, split_stride)
                                       : reinterpret_cast<const Vec8*>(in + static_cast<int64_t>(r) * F)[i];
    Vec8 b;
    b.w[0] = b.w[1] = b.w[2] = b.w[3] = 0u;
    if (bias) b = reinterpret_cast<const Vec8*>(bias)[i];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      float lo = bf16_lo(v.w[k]), hi = bf16_hi(v.w[k]);
      if (bias) {
        lo = bf16_round(lo + bf16_lo(b.w[k]));
        hi = bf16_round(hi + bf16_hi(b.w[k]));
      }
      o.w[k] = pack_bf16x2(gelu_erf_f(lo), gelu_erf_f(hi));
    }
  }
  if (valid && out) reinterpret_cast<Vec8*>(out + static_cast<int64_t>(r) * F)[i] = o;
  if (q_out) {
    float y[8];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      y[2 * k] = bf16_lo(o.w[k]);
      y[2 * k + 1] = bf16_hi(o.w[k]);
    }
    mx::quantize8_any(q_mode, y, valid, r, i * 8, q_out, F, sf_out, F / 128, m_pad);
  }
}

}  // namespace ew
}  // namespace b200

extern "C" {

int b200_gather_rows_bf16(const void* table, const int64_t* ids, void* out, int n_rows, int row_elems,
                          int64_t vocab_start, int64_t vocab_end, const void* add_table, const int64_t* add_ids,
                          b200_stream_t stream) {
  using namespace b200;
  if (!table || !ids || !out || n_rows <= 0 || row_elems <= 0) return B200_ERR_INVALID_ARGUMENT;
  if ((add_table == nullptr) != (add_ids == nullptr)) return B200_ERR_INVALID_ARGUMENT;
  if (row_elems % 8 != 0 || !aligned16(table) || !aligned16(out) || (add_table && !aligned16(add_table)))
    return B200_ERR_ALIGNMENT;
  int threads = row_elems / 8;
  threads = threads > 256 ? 256 : ((threads + 31) / 32) * 32;
  return launch_pdl(ew::gather_rows_kernel, dim3(n_rows), dim3(threads), 0, reinterpret_cast<cudaStream_t>(stream),
                    static_cast<const __nv_bfloat16*>(table), ids, static_cast<__nv_bfloat16*>(out), row_elems,
                    vocab_start, vocab_end, static_cast<const __nv_bfloat16*>(add_table), add_ids);
}

static int add_norm_impl(const void* x, const void* bias, const void* residual, const void* gamma, const void* beta,
                         void* hidden_out, void* normed_out, void* q_out, void* sf_out, int q_mode, int m_pad, int rows,
                         int hidden, float eps, b200_stream_t stream, const float* partials = nullptr, int splits = 0,
                         const b200::ew::PeerSrc* peers = nullptr) {
  using namespace b200;
  if ((!x && !partials && !peers) || rows <= 0 || hidden <= 0) return B200_ERR_INVALID_ARGUMENT;
  if (partials && (splits < 1 || hidden > 8192)) return B200_ERR_INVALID_ARGUMENT;
  if (peers && (hidden > 8192 || rows > peers->max_rows)) return B200_ERR_INVALID_ARGUMENT;
  if ((normed_out || q_out) && !gamma) return B200_ERR_INVALID_ARGUMENT;
  if (!normed_out && !hidden_out && !q_out) return B200_ERR_INVALID_ARGUMENT;
  if ((q_out == nullptr) != (sf_out == nullptr)) return B200_ERR_INVALID_ARGUMENT;
  if (hidden % 8 != 0 || (q_out && hidden % 128 != 0)) return B200_ERR_ALIGNMENT;
  const void* ptrs[] = {x, bias, residual, gamma, beta, hidden_out, normed_out, q_out, sf_out, partials};
  for (const void* q : ptrs)
    if (q && !aligned16(q)) return B200_ERR_ALIGNMENT;
  const int nvec = hidden / 8;
  int threads = nvec >= 256 ? 256 : ((nvec + 31) / 32) * 32;
  const int per_thread = (nvec + threads - 1) / threads;
  auto s = reinterpret_cast<cudaStream_t>(stream);
  auto X = static_cast<const __nv_bfloat16*>(x);
  auto B = static_cast<const __nv_bfloat16*>(bias);
  auto R = static_cast<const __nv_bfloat16*>(residual);
  auto Gm = static_cast<const __nv_bfloat16*>(gamma);
  auto Bt = static_cast<const __nv_bfloat16*>(beta);
  auto H = static_cast<__nv_bfloat16*>(hidden_out);
  auto Nn = static_cast<__nv_bfloat16*>(normed_out);
  auto Q = static_cast<uint8_t*>(q_out);
  const float* P = nullptr;
  const int64_t zero = 0;
  ew::PeerSrc none = {};
  const int wide = ((nvec + 31) / 32) * 32;  // <= 1024 for hidden <= 8192: one vector per thread
  if (peers)  // the tensor-parallel ranks' partial outputs instead of x
    return launch_pdl(ew::add_norm_kernel<1, 2>, dim3(rows), dim3(wide), 0, s, X, B, R, Gm, Bt, H, Nn, hidden, eps, Q, sf_out,
                      q_mode, m_pad, P, 0, zero, *peers);
  if (partials)  // split-K partial sums [splits][rows][hidden] instead of x
    return launch_pdl(ew::add_norm_kernel<1, 1>, dim3(rows), dim3(wide), 0, s, X, B, R, Gm, Bt, H, Nn, hidden, eps, Q, sf_out,
                      q_mode, m_pad, partials, splits, static_cast<int64_t>(rows) * hidden, none);
  if (per_thread <= 1)
    return launch_pdl(ew::add_norm_kernel<1, 0>, dim3(rows), dim3(threads), 0, s, X, B, R, Gm, Bt, H, Nn, hidden, eps, Q, sf_out, q_mode, m_pad, P, 0, zero, none);
  else if (per_thread <= 2)
    return launch_pdl(ew::add_norm_kernel<2, 0>, dim3(rows), dim3(threads), 0, s, X, B, R, Gm, Bt, H, Nn, hidden, eps, Q, sf_out, q_mode, m_pad, P, 0, zero, none);
  else if (per_thread <= 4)
    return launch_pdl(ew::add_norm_kernel<4, 0>, dim3(rows), dim3(threads), 0, s, X, B, R, Gm, Bt, H, Nn, hidden, eps, Q, sf_out, q_mode, m_pad, P, 0, zero, none);
  else if (per_thread <= 8)
    return launch_pdl(ew::add_norm_kernel<8, 0>, dim3(rows), dim3(threads), 0, s, X, B, R, Gm, Bt, H, Nn, hidden, eps, Q, sf_out, q_mode, m_pad, P, 0, zero, none);
  return B200_ERR_INVALID_ARGUMENT;  // hidden > 16384
}

int b200_add_norm_bf16(const void* x, const void* bias, const void* residual, const void* gamma, const void* beta,
                       void* hidden_out, void* normed_out, int rows, int hidden, float eps, b200_stream_t stream) {
  return add_norm_impl(x, bias, residual, gamma, beta, hidden_out, normed_out, nullptr, nullptr, 0, 0, rows, hidden, eps, stream);
}

int b200_add_norm_mxfp8(const void* x, const void* bias, const void* residual, const void* gamma, const void* beta,
                        void* hidden_out, void* q_out, void* sf_out, int rows, int hidden, float eps,
                        b200_stream_t stream) {
  if (!q_out || !sf_out) return B200_ERR_INVALID_ARGUMENT;
  return add_norm_impl(x, bias, residual, gamma, beta, hidden_out, nullptr, q_out, sf_out, b200::mx::kQuantMx, 0, rows, hidden,
                       eps, stream);
}

int b200_add_norm_fp8_rowblock(const void* x, const void* bias, const void* residual, const void* gamma, const void* beta,
                               void* hidden_out, void* q_out, float* scale_out, int m_pad, int rows, int hidden, float eps,
                               b200_stream_t stream) {
  if (!q_out || !scale_out || m_pad < rows || m_pad % 4 != 0) return B200_ERR_INVALID_ARGUMENT;
  return add_norm_impl(x, bias, residual, gamma, beta, hidden_out, nullptr, q_out, scale_out, b200::mx::kQuantBlock128, m_pad,
                       rows, hidden, eps, stream);
}

int b200_add_norm_splitk_bf16(const float* partials, int num_splits, const void* bias, const void* residual,
                              const void* gamma, const void* beta, void* hidden_out, void* normed_out, int rows, int hidden,
                              float eps, b200_stream_t stream) {
  if (!partials) return B200_ERR_INVALID_ARGUMENT;
  return add_norm_impl(nullptr, bias, residual, gamma, beta, hidden_out, normed_out, nullptr, nullptr, 0, 0, rows, hidden, eps,
                       stream, partials, num_splits);
}

int b200_add_norm_splitk_mxfp8(const float* partials, int num_splits, const void* bias, const void* residual,
                               const void* gamma, const void* beta, void* hidden_out, void* q_out, void* sf_out, int rows,
                               int hidden, float eps, b200_stream_t stream) {
  if (!partials || !q_out || !sf_out) return B200_ERR_INVALID_ARGUMENT;
  return add_norm_impl(nullptr, bias, residual, gamma, beta, hidden_out, nullptr, q_out, sf_out, b200::mx::kQuantMx, 0, rows,
                       hidden, eps, stream, partials, num_splits);
}

int b200_add_norm_splitk_fp8_rowblock(const float* partials, int num_splits, const void* bias, const void* residual,
                                      const void* gamma, const void* beta, void* hidden_out, void* q_out, float* scale_out,
                                      int m_pad, int rows, int hidden, float eps, b200_stream_t stream) {
  if (!partials || !q_out || !scale_out || m_pad < rows || m_pad % 4 != 0) return B200_ERR_INVALID_ARGUMENT;
  return add_norm_impl(nullptr, bias, residual, gamma, beta, hidden_out, nullptr, q_out, scale_out, b200::mx::kQuantBlock128,
                       m_pad, rows, hidden, eps, stream, partials, num_splits);
}

// ---------------------------------------------------------------------------------------------
// Tensor-parallel all-reduce fused into the residual-add + norm kernel (peer loads over NVLink)
// ---------------------------------------------------------------------------------------------
static int peer_src(const b200_tp_comm* c, int slot, b200::ew::PeerSrc& ps) {
  if (!c || c->world_size < 2 || c->world_size > 8 || c->rank < 0 || c->rank >= c->world_size) return B200_ERR_INVALID_ARGUMENT;
  if (slot < 0 || slot > 1 || c->max_rows <= 0 || c->hidden <= 0 || !c->counters) return B200_ERR_INVALID_ARGUMENT;
  const size_t slot_elems = static_cast<size_t>(c->max_rows) * c->hidden;
  for (int q = 0; q < c->world_size; ++q) {
    if (!c->data[q] || !c->flags[q]) return B200_ERR_INVALID_ARGUMENT;
    ps.data[q] = static_cast<const __nv_bfloat16*>(c->data[q]) + slot * slot_elems;
    ps.flags[q] = c->flags[q];
  }
  ps.counters = c->counters;
  ps.world = c->world_size;
  ps.rank = c->rank;
  ps.max_rows = c->max_rows;
  return B200_OK;
}

int b200_allreduce_add_norm_bf16(const b200_tp_comm* comm, int slot, const void* bias, const void* residual,
                                 const void* gamma, const void* beta, void* hidden_out, void* normed_out, int rows,
                                 int hidden, float eps, b200_stream_t stream) {
  b200::ew::PeerSrc ps = {};
  const int rc = peer_src(comm, slot, ps);
  if (rc != B200_OK) return rc;
  if (hidden != comm->hidden) return B200_ERR_INVALID_ARGUMENT;
  return add_norm_impl(nullptr, bias, residual, gamma, beta, hidden_out, normed_out, nullptr, nullptr, 0, 0, rows, hidden, eps,
                       stream, nullptr, 0, &ps);
}

int b200_allreduce_add_norm_mxfp8(const b200_tp_comm* comm, int slot, const void* bias, const void* residual,
                                  const void* gamma, const void* beta, void* hidden_out, void* q_out, void* sf_out, int rows,
                                  int hidden, float eps, b200_stream_t stream) {
  b200::ew::PeerSrc ps = {};
  const int rc = peer_src(comm, slot, ps);
  if (rc != B200_OK) return rc;
  if (hidden != comm->hidden || !q_out || !sf_out) return B200_ERR_INVALID_ARGUMENT;
  return add_norm_impl(nullptr, bias, residual, gamma, beta, hidden_out, nullptr, q_out, sf_out, b200::mx::kQuantMx, 0, rows,
                       hidden, eps, stream, nullptr, 0, &ps);
}

int b200_allreduce_add_norm_fp8_rowblock(const b200_tp_comm* comm, int slot, const void* bias, const void* residual,
                                         const void* gamma, const void* beta, void* hidden_out, void* q_out,
                                         float* scale_out, int m_pad, int rows, int hidden, float eps,
                                         b200_stream_t stream) {
  b200::ew::PeerSrc ps = {};
  const int rc = peer_src(comm, slot, ps);
  if (rc != B200_OK) return rc;
  if (hidden != comm->hidden || !q_out || !scale_out || m_pad < rows || m_pad % 4 != 0) return B200_ERR_INVALID_ARGUMENT;
  return add_norm_impl(nullptr, bias, residual, gamma, beta, hidden_out, nullptr, q_out, scale_out, b200::mx::kQuantBlock128,
                       m_pad, rows, hidden, eps, stream, nullptr, 0, &ps);
}

// Peer buffers: device memory that the other ranks of the node map through CUDA IPC handles.
int b200_peer_buffer_create(size_t bytes, void** ptr, unsigned char handle[64]) {
  if (!ptr || !handle || bytes == 0) return B200_ERR_INVALID_ARGUMENT;
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  void* p = nullptr;
  if (cudaMalloc(&p, bytes) != cudaSuccess || cudaMemset(p, 0, bytes) != cudaSuccess) {
    (void)cudaGetLastError();
    return B200_ERR_DRIVER;
  }
  cudaIpcMemHandle_t h;
  if (cudaIpcGetMemHandle(&h, p) != cudaSuccess) {
    (void)cudaGetLastError();
    cudaFree(p);
    return B200_ERR_DRIVER;
  }
  memcpy(handle, &h, 64);
  *ptr = p;
  return cudaDeviceSynchronize() == cudaSuccess ? B200_OK : B200_ERR_DRIVER;
}

int b200_peer_buffer_open(const unsigned char handle[64], void** ptr) {
  if (!ptr || !handle) return B200_ERR_INVALID_ARGUMENT;
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, 64);
  if (cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
    (void)cudaGetLastError();
    return B200_ERR_DRIVER;
  }
  return B200_OK;
}

int b200_peer_buffer_close(void* ptr) {
  if (!ptr) return B200_ERR_INVALID_ARGUMENT;
  if (cudaIpcCloseMemHandle(ptr) != cudaSuccess) {
    (void)cudaGetLastError();
    return B200_ERR_DRIVER;
  }
  return B200_OK;
}

int b200_peer_buffer_destroy(void* ptr) {
  if (!ptr) return B200_ERR_INVALID_ARGUMENT;
  if (cudaFree(ptr) != cudaSuccess) {
    (void)cudaGetLastError();
    return B200_ERR_DRIVER;
  }
  return B200_OK;
}

static int activation_impl(const void* in, const void* bias, void* out, void* q_out, void* sf_out, int q_mode, int m_pad,
                           int rows, int F, int kind, b200_stream_t stream, const float* partials = nullptr, int splits = 0) {
  using namespace b200;
  if ((!in && !partials) || (!out && !q_out) || rows <= 0 || F <= 0 || kind < 0 || kind > 2) return B200_ERR_INVALID_ARGUMENT;
  if (partials && splits < 1) return B200_ERR_INVALID_ARGUMENT;
  if (kind == 2 && F % 64 != 0) return B200_ERR_ALIGNMENT;
  if ((q_out == nullptr) != (sf_out == nullptr)) return B200_ERR_INVALID_ARGUMENT;
  if (F % 8 != 0 || (q_out && F % 128 != 0) || (in && !aligned16(in)) || (partials && !aligned16(partials)) ||
      (out && !aligned16(out)) || (bias && !aligned16(bias)) || (q_out && (!aligned16(q_out) || !aligned16(sf_out))))
    return B200_ERR_ALIGNMENT;
  const int nvec = F / 8;
  dim3 grid(rows, (nvec + 255) / 256);
  const int64_t split_stride = static_cast<int64_t>(rows) * (kind == 1 ? F : 2 * F);
  return launch_pdl(ew::activation_kernel, grid, dim3(256), 0, reinterpret_cast<cudaStream_t>(stream),
                    static_cast<const __nv_bfloat16*>(in), static_cast<const __nv_bfloat16*>(bias),
                    static_cast<__nv_bfloat16*>(out), F, kind, static_cast<uint8_t*>(q_out), sf_out, q_mode, m_pad, partials,
                    splits, split_stride);
}

int b200_activation_bf16(const void* in, const void* bias, void* out, int rows, int F, int kind, b200_stream_t stream) {
  return activation_impl(in, bias, out, nullptr, nullptr, 0, 0, rows, F, kind, stream);
}

int b200_activation_mxfp8(const void* in, const void* bias, void* q_out, void* sf_out, int rows, int F, int kind,
                          b200_stream_t stream) {
  if (!q_out || !sf_out) return B200_ERR_INVALID_ARGUMENT;
  return activation_impl(in, bias, nullptr, q_out, sf_out, b200::mx::kQuantMx, 0, rows, F, kind, stream);
}

int b200_activation_fp8_rowblock(const void* in, const void* bias, void* q_out, float* scale_out, int m_pad, int rows, int F,
                                 int kind, b200_stream_t stream) {
  if (!q_out || !scale_out || m_pad < rows || m_pad % 4 != 0) return B200_ERR_INVALID_ARGUMENT;
  return activation_impl(in, bias, nullptr, q_out, scale_out, b200::mx::kQuantBlock128, m_pad, rows, F, kind, stream);
}

int b200_activation_splitk_bf16(const float* partials, int num_splits, const void* bias, void* out, int rows, int F, int kind,
                                b200_stream_t stream) {
  if (!partials) return B200_ERR_INVALID_ARGUMENT;
  return activation_impl(nullptr, bias, out, nullptr, nullptr, 0, 0, rows, F, kind, stream, partials, num_splits);
}

int b200_activation_splitk_mxfp8(const float* partials, int num_splits, const void* bias, void* q_out, void* sf_out, int rows,
                                 int F, int kind, b200_stream_t stream) {
  if (!partials || !q_out || !sf_out) return B200_ERR_INVALID_ARGUMENT;
  return activation_impl(nullptr, bias, nullptr, q_out, sf_out, b200::mx::kQuantMx, 0, rows, F, kind, stream, partials,
                         num_splits);
}

int b200_activation_splitk_fp8_rowblock(const float* partials, int num_splits, const void* bias, void* q_out, float* scale_out,
                                        int m_pad, int rows, int F, int kind, b200_stream_t stream) {
  if (!partials || !q_out || !scale_out || m_pad < rows || m_pad % 4 != 0) return B200_ERR_INVALID_ARGUMENT;
  return activation_impl(nullptr, bias, nullptr, q_out, scale_out, b200::mx::kQuantBlock128, m_pad, rows, F, kind, stream,
                         partials, num_splits);
}

}  // extern "C"
