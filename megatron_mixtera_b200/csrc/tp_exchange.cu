// Two-shot tensor-parallel all-reduce fused with residual add + norm (+ FP8 quantisation), over peer memory.
//
// Every rank's row-parallel GEMM leaves its bf16 partial output [rows][hidden] in a buffer that the other ranks of
// the node map (CUDA IPC).  The token rows are divided among the ranks; rank r is the ONLY one that
//   1. sums the partial rows of its share from all ranks (plain peer loads over NVLink, rank order, fp32, one
//      bf16 rounding),
//   2. adds bias and residual, normalises, optionally quantises - the work of add_norm_kernel for those rows -
//   3. and stores the finished rows (hidden state, normalised / quantised row and its scales) into the output
//      buffers of EVERY rank (plain peer stores).
// Compared with the one-shot form (every rank pulls every peer's rows and normalises all of them), a rank moves
// 2 (w-1)/w of the data instead of (w-1) times the data over NVLink and does 1/w of the arithmetic; and because each
// row is computed exactly once, all ranks hold bit-identical results by construction.
//
// Synchronisation: two flag exchanges per call, both with bounded waits (g_wait_limit_ns; on expiry the status word
// gets kStatusPeerTimeout and the kernel carries on with what is there):
//   A  "my partial output of call c is complete"  - before anybody reads a peer's input buffer
//   B  "my share of the rows of call c is stored everywhere" - sent by the last CTA of a rank after a system-scope
//      fence; the same CTA waits for the peers' B flags before the kernel completes, so whatever follows on the
//      stream (the next GEMM reads the normalised rows, the next call reads the hidden state as its residual) sees
//      all rows.
// Flags carry the call number (monotonic, kept in device memory: CUDA-graph replays need no host involvement), so
// nothing is ever reset.  One buffer per kind suffices: a rank can only write a peer's input buffer for call c+1 after
// its own call c has completed, i.e. after every peer has passed exchange B of call c and is done reading call c's
// inputs; and output rows are written only after exchange A of the same call, when every rank has finished the
// kernels that read the previous call's outputs.  Rows of the hidden state are owned by one rank per call, which is
// why the residual may live in the very buffer the new hidden state is written to.
// Split-K inputs: when the row-parallel GEMM was split along K its fp32 partial sums [splits][rows][hidden] can be
// handed over as they are.  The kernel's CTAs then first sum them in split order (the arithmetic of the GEMM's own
// reduction kernel: fp32, one bf16 rounding) into this rank's input buffer - each CTA a strided share of ALL rows - and
// the CTA that finishes last sends exchange A.  One launch fewer per linear, same bits.
// No TMA, no multicast, no multimem: plain loads and stores.
#include "common.cuh"
#include "quant.cuh"

namespace b200 {
namespace tpx {

struct Exchange {
  const __nv_bfloat16* in[8];
  __nv_bfloat16* hidden_out[8];
  void* normed_out[8];
  void* scales_out[8];
  int32_t* flags[8];  // per rank: [2][8] int32 - [0][q]: exchange A from rank q, [1][q]: exchange B from rank q
  int32_t* counters;  // local: [0] calls completed, [1] CTAs of the running call that are done, [2] CTAs whose share of
                      // the split-K sums is written
  int world, rank, m_pad;
};

__device__ __forceinline__ void st_release_sys(int32_t* p, int32_t v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int32_t ld_acquire_sys(const int32_t* p) {
  int32_t v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Called by threads 0 .. world-1 of a CTA (thread q talks to rank q): announce `call` in slot `which` of every peer
// (if `announce`), then wait until every peer has announced it here.
// kRelaxed: relaxed system-scope flag accesses without fences.  Right for exchange A when the input was written by an
// earlier kernel of this stream: griddepcontrol.wait has awaited that kernel's completion, memory included, so the rows
// are in this GPU's L2 - where a peer's load is served - before the flag store is issued.  A release store would add a
// system-scope fence in front of the first NVLink hop of every call (measured 23.5 -> 17.7 us per call, 2 ranks,
// 128 x 4096).  Exchange B announces rows this kernel has just stored into the peers' memory and keeps release /
// acquire behind the CTAs' system-scope fences.
template <bool kRelaxed = false>
__device__ __forceinline__ void exchange(const Exchange& x, int which, int32_t call, bool announce) {
  const int q = threadIdx.x;
  if (q >= x.world || q == x.rank) return;
  if (announce) {
    if (kRelaxed) ew::st_relaxed_sys(x.flags[q] + which * 8 + x.rank, call);
    else st_release_sys(x.flags[q] + which * 8 + x.rank, call);
  }
  const int32_t* mine = x.flags[x.rank] + which * 8 + q;
  const uint64_t t0 = global_timer_ns();
  while ((kRelaxed ? ew::ld_relaxed_sys(mine) : ld_acquire_sys(mine)) < call) {
    if (global_timer_ns() - t0 > g_wait_limit_ns) {
      atomicOr(&g_device_status, kStatusPeerTimeout);
      return;
    }
    __nanosleep(20);
  }
}

__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nw = (blockDim.x + 31) >> 5;
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = lane < nw ? red[lane] : 0.f;
  return warp_sum(t);
}

// One CTA per owned token row, one 8-element vector per thread (hidden <= 8192).  q_mode 0: bf16 normalised rows;
// mx::kQuantMx / mx::kQuantBlock128: E4M3 rows + scales.
__global__ void __launch_bounds__(1024)
allreduce2_add_norm_kernel(Exchange x, const __nv_bfloat16* __restrict__ bias, const __nv_bfloat16* __restrict__ residual,
                           const __nv_bfloat16* __restrict__ gamma, const __nv_bfloat16* __restrict__ beta, int rows,
                           int hidden, float eps, int q_mode, const float* __restrict__ partials, int splits) {
  __shared__ float red[32];
  __shared__ int s_last;
  __shared__ int s_announce;
  pdl_launch_dependents();
  pdl_wait();
  // every CTA reads the same value: the counter moves only when the last CTA of this launch is done
  const int32_t call = ew::ld_relaxed_sys(x.counters) + 1;  // written by the previous call's kernel
  bool announce = blockIdx.x == 0;
  if (partials != nullptr) {
    // ---- split-K sums of this rank's GEMM into its input buffer: rows blockIdx.x, blockIdx.x + gridDim.x, ... ----
    __nv_bfloat16* mine = const_cast<__nv_bfloat16*>(x.in[x.rank]);
    const int64_t split_stride = static_cast<int64_t>(rows) * hidden;
    if (static_cast<int>(threadIdx.x) < hidden / 8) {
      for (int r = blockIdx.x; r < rows; r += gridDim.x) {
        const int64_t o = static_cast<int64_t>(r) * hidden + threadIdx.x * 8;
        const ew::Vec8 v = ew::sum_partials8(partials + o, splits, split_stride);
        *reinterpret_cast<uint4*>(mine + o) = make_uint4(v.w[0], v.w[1], v.w[2], v.w[3]);
      }
    }
    // the CTA barrier orders every thread's stores before thread 0's system-scope fence, and that fence before the
    // arrival count: the CTA that counts last (and then announces) sends the flag after all rows are visible
    __syncthreads();
    if (threadIdx.x == 0) {
      __threadfence_system();
      const bool last = atomicAdd(&x.counters[2], 1) == static_cast<int>(gridDim.x) - 1;
      if (last) x.counters[2] = 0;  // nobody touches it again before the next call (which starts after this kernel)
      __threadfence();
      s_announce = last;
    }
    __syncthreads();
    announce = s_announce != 0;
    // CTAs beyond this rank's share of the rows were launched for the sums only; the one that counted last still has
    // to deliver exchange A (it does not wait: nothing it does afterwards depends on the peers)
    if (static_cast<int>(blockIdx.x) >= (rows + x.world - 1) / x.world) {
      if (announce && threadIdx.x < 8 && static_cast<int>(threadIdx.x) < x.world && static_cast<int>(threadIdx.x) != x.rank) {
        __threadfence_system();
        st_release_sys(x.flags[threadIdx.x] + x.rank, call);
      }
      announce = false;
    }
  }
  // ---- exchange A: this rank's partial output (written by the kernel before this one, or just above) is complete ----
  const int per_rank = (rows + x.world - 1) / x.world;
  if (static_cast<int>(blockIdx.x) < per_rank) {
    if (threadIdx.x < 8) {
      if (partials != nullptr) {  // the input rows were written by this kernel's own CTAs: fence + release
        __threadfence_system();
        exchange(x, 0, call, announce);
      } else {
        exchange<true>(x, 0, call, announce);
      }
    }
    __syncthreads();
  }

  const int row = x.rank * per_rank + blockIdx.x;
  const int nvec = hidden / 8;
  const int i = threadIdx.x;
  if (blockIdx.x < per_rank && row < rows) {
    const bool valid = i < nvec;
    const int64_t off = static_cast<int64_t>(row) * hidden;
    float f[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    if (valid) {
      uint4 u[8];  // all peers' vectors are requested before any is used: one NVLink round trip
#pragma unroll
      for (int q = 0; q < 8; ++q)
        if (q < x.world) u[q] = __ldcg(reinterpret_cast<const uint4*>(x.in[q] + off) + i);
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        if (q < x.world) {  // rank order
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
      if (bias != nullptr) {
        const uint4 b = reinterpret_cast<const uint4*>(bias)[i];
        const uint32_t w4[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          f[2 * k] = bf16_round(f[2 * k] + bf16_lo(w4[k]));
          f[2 * k + 1] = bf16_round(f[2 * k + 1] + bf16_hi(w4[k]));
        }
      }
      if (residual != nullptr) {
        const uint4 r = reinterpret_cast<const uint4*>(residual + off)[i];
        const uint32_t w4[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          f[2 * k] = bf16_round(f[2 * k] + bf16_lo(w4[k]));
          f[2 * k + 1] = bf16_round(f[2 * k + 1] + bf16_hi(w4[k]));
        }
      }
      const uint4 h = make_uint4(pack_bf16x2(f[0], f[1]), pack_bf16x2(f[2], f[3]), pack_bf16x2(f[4], f[5]),
                                 pack_bf16x2(f[6], f[7]));
#pragma unroll
      for (int q = 0; q < 8; ++q)
        if (q < x.world) reinterpret_cast<uint4*>(x.hidden_out[q] + off)[i] = h;
    }
    float sum = 0.f, sumsq = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      sum += f[k];
      sumsq += f[k] * f[k];
    }
    float mean = 0.f, rstd;
    if (beta != nullptr) {  // LayerNorm: two-pass variance on the cached values
      mean = block_sum(sum, red) / hidden;
      float var = 0.f;
      if (valid) {
#pragma unroll
        for (int k = 0; k < 8; ++k) var += (f[k] - mean) * (f[k] - mean);
      }
      rstd = rsqrtf(block_sum(var, red) / hidden + eps);
    } else {
      rstd = rsqrtf(block_sum(sumsq, red) / hidden + eps);
    }
    float y[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    if (valid) {
      const uint4 g = reinterpret_cast<const uint4*>(gamma)[i];
      const uint32_t g4[4] = {g.x, g.y, g.z, g.w};
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        y[2 * k] = (f[2 * k] - mean) * rstd * bf16_lo(g4[k]);
        y[2 * k + 1] = (f[2 * k + 1] - mean) * rstd * bf16_hi(g4[k]);
      }
      if (beta != nullptr) {
        const uint4 b = reinterpret_cast<const uint4*>(beta)[i];
        const uint32_t b4[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          y[2 * k] += bf16_lo(b4[k]);
          y[2 * k + 1] += bf16_hi(b4[k]);
        }
      }
    }
    if (q_mode == 0) {
      if (valid) {
        const uint4 o = make_uint4(pack_bf16x2(y[0], y[1]), pack_bf16x2(y[2], y[3]), pack_bf16x2(y[4], y[5]),
                                   pack_bf16x2(y[6], y[7]));
#pragma unroll
        for (int q = 0; q < 8; ++q)
          if (q < x.world) reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(x.normed_out[q]) + off)[i] = o;
      }
    } else {
      // quantise the bf16-rounded normalised row (what an unfused quantiser would read); the scale block is 32
      // elements = 4 lanes (MXFP8) or 128 elements = 16 lanes (128-block recipe)
#pragma unroll
      for (int k = 0; k < 8; ++k) y[k] = bf16_round(y[k]);
      float amax = 0.f;
#pragma unroll
      for (int k = 0; k < 8; ++k) amax = fmaxf(amax, fabsf(y[k]));
      const int span = q_mode == mx::kQuantMx ? 4 : 16;
      for (int o = 1; o < span; o <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
      if (valid) {
        float inv, scale_f = 0.f;
        uint32_t e = 0;
        if (q_mode == mx::kQuantMx) {
          e = mx::e8m0_scale_byte(amax);
          inv = scalbnf(1.0f, 127 - static_cast<int>(e));
        } else {
          scale_f = fmaxf(amax / 448.0f, 1e-30f);
          inv = 0.f;
        }
        uint32_t w[2];
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
          float a0 = y[4 * hh], a1 = y[4 * hh + 1], a2 = y[4 * hh + 2], a3 = y[4 * hh + 3];
          if (q_mode == mx::kQuantMx) {
            a0 *= inv; a1 *= inv; a2 *= inv; a3 *= inv;
          } else {
            a0 /= scale_f; a1 /= scale_f; a2 /= scale_f; a3 /= scale_f;
          }
          const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a0, a1), __NV_SATFINITE, __NV_E4M3);
          const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(a2, a3), __NV_SATFINITE, __NV_E4M3);
          w[hh] = lo | (hi << 16);
        }
        const int col0 = i * 8;
        const uint2 packed = make_uint2(w[0], w[1]);
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          if (q < x.world) {
            *reinterpret_cast<uint2*>(static_cast<uint8_t*>(x.normed_out[q]) + off + col0) = packed;
            if (q_mode == mx::kQuantMx) {
              if ((col0 & 31) == 0)
                static_cast<uint8_t*>(x.scales_out[q])[mx::sf_offset(row, col0 >> 5, hidden / 128)] = static_cast<uint8_t>(e);
            } else if ((col0 & 127) == 0) {
              static_cast<float*>(x.scales_out[q])[static_cast<int64_t>(col0 >> 7) * x.m_pad + row] = scale_f;
            }
          }
        }
      }
    }
  }

  // ---- exchange B: this rank's rows are stored everywhere; wait for everybody else's ----
  // The CTA barrier orders every thread's peer stores before thread 0's system-scope fence (fences are cumulative), and
  // that fence before the counter update: whoever sees the counter (the last CTA, which then releases the B flags)
  // also sees the stores.  One fence per CTA instead of one per thread: a system-scope fence waits for the SM's
  // outstanding remote writes and costs microseconds.
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    s_last = atomicAdd(&x.counters[1], 1) == static_cast<int>(gridDim.x) - 1;
    __threadfence();
  }
  __syncthreads();
  if (s_last) {
    if (threadIdx.x < 8) exchange(x, 1, call, true);
    __syncthreads();
    if (threadIdx.x == 0) {
      x.counters[1] = 0;
      __threadfence();
      st_release_sys(x.counters, call);
    }
  }
}

}  // namespace tpx
}  // namespace b200

extern "C" {

static int allreduce2_impl(const b200_tp_exchange* c, const float* partials, int num_splits, const void* bias,
                           const void* residual, const void* gamma, const void* beta, int q_mode, int rows, int hidden,
                           float eps, b200_stream_t stream) {
  using namespace b200;
  if (partials != nullptr && (num_splits < 1 || num_splits > 32 || !aligned16(partials))) return B200_ERR_INVALID_ARGUMENT;
  // With split-K input the peers wait for ALL CTAs of this launch (the last one to finish its sums announces), so the
  // whole grid must be resident at once: one CTA per SM always is.
  if (partials != nullptr && c && (rows + c->world_size - 1) / c->world_size > 128) return B200_ERR_INVALID_ARGUMENT;
  if (!c || c->world_size < 2 || c->world_size > 8 || c->rank < 0 || c->rank >= c->world_size) return B200_ERR_INVALID_ARGUMENT;
  if (rows <= 0 || rows > c->max_rows || hidden != c->hidden || hidden <= 0 || hidden > 8192 || !gamma || !c->counters)
    return B200_ERR_INVALID_ARGUMENT;
  if (q_mode != 0 && q_mode != mx::kQuantMx && q_mode != mx::kQuantBlock128) return B200_ERR_INVALID_ARGUMENT;
  if (hidden % 8 != 0 || (q_mode != 0 && hidden % 128 != 0)) return B200_ERR_ALIGNMENT;
  if (q_mode == mx::kQuantBlock128 && (c->m_pad < c->max_rows || c->m_pad % 4 != 0)) return B200_ERR_INVALID_ARGUMENT;
  tpx::Exchange x = {};
  for (int q = 0; q < c->world_size; ++q) {
    if (!c->in[q] || !c->hidden_out[q] || !c->normed_out[q] || !c->flags[q] || (q_mode != 0 && !c->scales_out[q]))
      return B200_ERR_INVALID_ARGUMENT;
    if (!aligned16(c->in[q]) || !aligned16(c->hidden_out[q]) || !aligned16(c->normed_out[q])) return B200_ERR_ALIGNMENT;
    x.in[q] = static_cast<const __nv_bfloat16*>(c->in[q]);
    x.hidden_out[q] = static_cast<__nv_bfloat16*>(c->hidden_out[q]);
    x.normed_out[q] = c->normed_out[q];
    x.scales_out[q] = c->scales_out[q];
    x.flags[q] = c->flags[q];
  }
  const void* ptrs[] = {bias, residual, gamma, beta};
  for (const void* p : ptrs)
    if (p && !aligned16(p)) return B200_ERR_ALIGNMENT;
  x.counters = c->counters;
  x.world = c->world_size;
  x.rank = c->rank;
  x.m_pad = c->m_pad;
  const int nvec = hidden / 8;
  int threads = ((nvec + 31) / 32) * 32;
  if (threads < 32) threads = 32;
  const int per_rank = (rows + c->world_size - 1) / c->world_size;
  // split-K input: up to 128 CTAs share the sums (all rows); the first `per_rank` of them go on with the exchange
  const int grid = partials != nullptr ? (rows < 128 ? (rows > per_rank ? rows : per_rank) : 128) : per_rank;
  return launch_pdl(tpx::allreduce2_add_norm_kernel, dim3(grid), dim3(threads), 0, reinterpret_cast<cudaStream_t>(stream),
                    x, static_cast<const __nv_bfloat16*>(bias), static_cast<const __nv_bfloat16*>(residual),
                    static_cast<const __nv_bfloat16*>(gamma), static_cast<const __nv_bfloat16*>(beta), rows, hidden, eps, q_mode,
                    partials, num_splits);
}

int b200_allreduce2_add_norm(const b200_tp_exchange* c, const void* bias, const void* residual, const void* gamma,
                             const void* beta, int q_mode, int rows, int hidden, float eps, b200_stream_t stream) {
  return allreduce2_impl(c, nullptr, 0, bias, residual, gamma, beta, q_mode, rows, hidden, eps, stream);
}

int b200_allreduce2_add_norm_splitk(const b200_tp_exchange* c, const float* partials, int num_splits, const void* bias,
                                    const void* residual, const void* gamma, const void* beta, int q_mode, int rows,
                                    int hidden, float eps, b200_stream_t stream) {
  if (!partials) return B200_ERR_INVALID_ARGUMENT;
  return allreduce2_impl(c, partials, num_splits, bias, residual, gamma, beta, q_mode, rows, hidden, eps, stream);
}

}  // extern "C"
