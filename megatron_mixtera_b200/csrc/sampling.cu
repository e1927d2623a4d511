// Sampling over vocab-sized bf16 logit rows: greedy argmax, top-k and top-p filtered probabilities.
// One CTA per row; rows are read once with 16-byte loads where the row start allows it.
#include "common.cuh"

namespace b200 {
namespace sampling {

constexpr int kThreads = 1024;

// Order-preserving map of bf16 bits to unsigned: larger float <=> larger key.
__device__ __forceinline__ uint32_t bf16_key(uint16_t b) { return (b & 0x8000u) ? (~b & 0xffffu) : (b | 0x8000u); }
__device__ __forceinline__ float bf16_bits_to_float(uint16_t b) { return __uint_as_float(static_cast<uint32_t>(b) << 16); }

// Greedy: largest value, smallest index among equal values (NaN never wins).
__global__ void __launch_bounds__(kThreads)
argmax_kernel(const uint16_t* __restrict__ logits, int64_t ld, int64_t* __restrict__ out, int vocab,
              uint64_t* __restrict__ keys, int64_t index_offset) {
  pdl_launch_dependents();
  pdl_wait();
  const uint16_t* row = logits + static_cast<int64_t>(blockIdx.x) * ld;
  float best = -INFINITY;
  int best_i = 0x7fffffff;
  for (int i = threadIdx.x; i < vocab; i += kThreads) {
    const float v = bf16_bits_to_float(row[i]);
    if (v > best || (best_i == 0x7fffffff && v == best)) {  // strided scan visits indices in increasing order
      best = v;
      best_i = i;
    }
  }
  __shared__ float sv[32];
  __shared__ int si[32];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
    if (ov > best || (ov == best && oi < best_i)) {
      best = ov;
      best_i = oi;
    }
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) {
    sv[warp] = best;
    si[warp] = best_i;
  }
  __syncthreads();
  if (warp == 0) {
    best = sv[lane];
    best_i = si[lane];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
      if (ov > best || (ov == best && oi < best_i)) {
        best = ov;
        best_i = oi;
      }
    }
    if (lane == 0) {
      const int idx = best_i == 0x7fffffff ? 0 : best_i;
      if (keys == nullptr) {
        out[blockIdx.x] = idx;
      } else {
        // Vocabulary shard: a 64-bit key whose maximum over the shards is the global greedy choice - the value's
        // order-preserving 16-bit code (-0 counts as +0, as a float comparison does) above the complement of the global
        // index, so that among equal values the smallest index wins.
        uint16_t bits = best_i == 0x7fffffff ? 0xff80u : row[idx];  // a shard without a comparable value counts as -inf
        if (bits == 0x8000u) bits = 0;
        keys[blockIdx.x] = (static_cast<uint64_t>(bf16_key(bits)) << 32) |
                           (0xffffffffull - static_cast<uint64_t>(index_offset + idx));
      }
    }
  }
}

// Greedy token per row from the per-shard keys [shards][rows] written by argmax_kernel.
__global__ void argmax_merge_kernel(const uint64_t* __restrict__ keys, int shards, int rows, int64_t* __restrict__ out) {
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= rows) return;
  uint64_t best = 0;
  for (int s = 0; s < shards; ++s) {
    const uint64_t k = keys[static_cast<int64_t>(s) * rows + r];
    best = k > best ? k : best;
  }
  out[r] = static_cast<int64_t>(0xffffffffull - (best & 0xffffffffull));
}

// Top-k: the k-th largest value is found exactly by a two-pass radix select on the 16-bit keys
// (256-bin histograms in shared memory); logits below it become probability 0, the rest
// softmax((logit / temperature)) in fp32.  Division by the temperature is rounded to bf16 first,
// as the in-place `logits.div_(temperature)` on a bf16 tensor does.
__global__ void __launch_bounds__(kThreads)
topk_probs_kernel(const uint16_t* __restrict__ logits, int64_t ld, float* __restrict__ probs, int vocab, int top_k,
                  float temperature) {
  __shared__ int hist[256];
  __shared__ int sel_bin, sel_rank;
  __shared__ float red[32];
  pdl_launch_dependents();
  pdl_wait();
  const uint16_t* row = logits + static_cast<int64_t>(blockIdx.x) * ld;
  float* prow = probs + static_cast<int64_t>(blockIdx.x) * vocab;
  const bool scale = temperature != 1.0f;

  auto load_key = [&](int i) -> uint32_t {
    uint16_t b = row[i];
    if (scale) {
      __nv_bfloat16 q = __float2bfloat16_rn(bf16_bits_to_float(b) / temperature);
      b = *reinterpret_cast<uint16_t*>(&q);
    }
    return bf16_key(b);
  };
  auto key_to_float = [&](uint32_t key) -> float {
    const uint16_t b = (key & 0x8000u) ? static_cast<uint16_t>(key & 0x7fffu) : static_cast<uint16_t>(~key & 0xffffu);
    return bf16_bits_to_float(b);
  };

  // pass 1: high byte
  for (int i = threadIdx.x; i < 256; i += kThreads) hist[i] = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < vocab; i += kThreads) atomicAdd(&hist[load_key(i) >> 8], 1);
  __syncthreads();
  if (threadIdx.x == 0) {
    int need = top_k, b = 255;
    for (; b > 0; --b) {
      if (hist[b] >= need) break;
      need -= hist[b];
    }
    sel_bin = b;
    sel_rank = need;  // the threshold is the need-th largest key inside bin b
  }
  __syncthreads();
  const int hi_bin = sel_bin;
  const int need = sel_rank;
  __syncthreads();
  // pass 2: low byte inside the selected high bin
  for (int i = threadIdx.x; i < 256; i += kThreads) hist[i] = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < vocab; i += kThreads) {
    const uint32_t k = load_key(i);
    if (static_cast<int>(k >> 8) == hi_bin) atomicAdd(&hist[k & 0xff], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int n = need, b = 255;
    for (; b > 0; --b) {
      if (hist[b] >= n) break;
      n -= hist[b];
    }
    sel_bin = b;
  }
  __syncthreads();
  const uint32_t thr_key = (static_cast<uint32_t>(hi_bin) << 8) | static_cast<uint32_t>(sel_bin);

  // softmax over the kept entries: max is the largest key overall
  float mx = -INFINITY;
  for (int i = threadIdx.x; i < vocab; i += kThreads) {
    const uint32_t k = load_key(i);
    if (k >= thr_key) mx = fmaxf(mx, key_to_float(k));
  }
  mx = warp_max(mx);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) red[warp] = mx;
  __syncthreads();
  mx = warp_max(red[lane]);
  __syncthreads();
  float sum = 0.f;
  for (int i = threadIdx.x; i < vocab; i += kThreads) {
    const uint32_t k = load_key(i);
    if (k >= thr_key) sum += expf(key_to_float(k) - mx);
  }
  sum = warp_sum(sum);
  if (lane == 0) red[warp] = sum;
  __syncthreads();
  sum = warp_sum(red[lane]);
  const float inv = 1.f / sum;
  for (int i = threadIdx.x; i < vocab; i += kThreads) {
    const uint32_t k = load_key(i);
    prow[i] = k >= thr_key ? expf(key_to_float(k) - mx) * inv : 0.f;
  }
}


// Deterministic block reductions (fixed tree, independent of timing).
__device__ __forceinline__ float block_sum_1024(float v, float* red) {
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  return warp_sum(red[lane]);
}
__device__ __forceinline__ int block_sum_1024_int(int v, int* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  int t = red[lane];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
  return t;
}

// Top-p (nucleus): with the tokens in descending order of logit (equal logits: ascending index), a token is
// kept iff the probability mass strictly ahead of it is <= top_p (so the token that crosses top_p is kept and
// the first token always is) - the rule of `modify_logits_for_top_p_filtering`.  Kept tokens get
// softmax over the kept set, the rest 0.  All tokens with the same bf16 logit have the same probability, so
// the cut is found by a binary search over the 16-bit key space: A(k) = mass of the tokens with key > k is
// monotone in k, and the smallest key with A(k) <= top_p is the last (possibly partially) kept value; of its
// n tied tokens the first floor((top_p - A) / p) + 1 by index are kept.  Everything is computed in fp32 with
// fixed-order reductions.
__global__ void __launch_bounds__(kThreads)
topp_probs_kernel(const uint16_t* __restrict__ logits, int64_t ld, float* __restrict__ probs, int vocab, float top_p,
                  float temperature) {
  __shared__ float red[32];
  __shared__ int redi[32];
  __shared__ int warp_base[32];
  pdl_launch_dependents();
  pdl_wait();
  const uint16_t* row = logits + static_cast<int64_t>(blockIdx.x) * ld;
  float* prow = probs + static_cast<int64_t>(blockIdx.x) * vocab;
  const bool scale = temperature != 1.0f;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  auto load_key = [&](int i) -> uint32_t {
    uint16_t b = row[i];
    if (scale) {
      __nv_bfloat16 q = __float2bfloat16_rn(bf16_bits_to_float(b) / temperature);
      b = *reinterpret_cast<uint16_t*>(&q);
    }
    return bf16_key(b);
  };
  auto key_to_float = [&](uint32_t key) -> float {
    const uint16_t b = (key & 0x8000u) ? static_cast<uint16_t>(key & 0x7fffu) : static_cast<uint16_t>(~key & 0xffffu);
    return bf16_bits_to_float(b);
  };

  // row maximum (as a key) and the softmax denominator over the whole row
  uint32_t kmax = 0;
  for (int i = threadIdx.x; i < vocab; i += kThreads) kmax = max(kmax, load_key(i));
  kmax = static_cast<uint32_t>(warp_max(static_cast<float>(kmax)));  // keys < 2^16 are exact in fp32
  if (lane == 0) red[warp] = static_cast<float>(kmax);
  __syncthreads();
  kmax = static_cast<uint32_t>(warp_max(red[lane]));
  const float mx = key_to_float(kmax);
  float z = 0.f;
  for (int i = threadIdx.x; i < vocab; i += kThreads) z += expf(key_to_float(load_key(i)) - mx);
  z = block_sum_1024(z, red);
  const float budget = top_p * z;  // un-normalised mass allowed strictly ahead of a kept token

  // mass(k) = sum of exp over tokens with key > k
  auto mass_above = [&](uint32_t k) -> float {
    float a = 0.f;
    for (int i = threadIdx.x; i < vocab; i += kThreads) {
      const uint32_t ki = load_key(i);
      if (ki > k) a += expf(key_to_float(ki) - mx);
    }
    return block_sum_1024(a, red);
  };
  // smallest key in [0, kmax] with mass_above(key) <= budget (kmax always qualifies: mass 0)
  uint32_t lo = 0, hi = kmax;
  if (top_p >= 1.0f) hi = 0;  // everything is kept
  while (lo < hi) {
    const uint32_t mid = (lo + hi) >> 1;
    if (mass_above(mid) <= budget) {
      hi = mid;
    } else {
      lo = mid + 1;
    }
  }
  // `hi` may be a key no token has; move up to the smallest present key >= hi (same kept set)
  uint32_t kcut = 0xffffu;
  for (int i = threadIdx.x; i < vocab; i += kThreads) {
    const uint32_t ki = load_key(i);
    if (ki >= hi) kcut = min(kcut, ki);
  }
  kcut = 0xffffu - static_cast<uint32_t>(warp_max(static_cast<float>(0xffffu - kcut)));
  __syncthreads();
  if (lane == 0) red[warp] = static_cast<float>(0xffffu - kcut);
  __syncthreads();
  kcut = 0xffffu - static_cast<uint32_t>(warp_max(red[lane]));

  const float above = mass_above(kcut);
  const float e_cut = expf(key_to_float(kcut) - mx);
  int n_ties = 0;
  for (int i = threadIdx.x; i < vocab; i += kThreads) n_ties += load_key(i) == kcut ? 1 : 0;
  n_ties = block_sum_1024_int(n_ties, redi);
  int keep_ties = n_ties;
  if (top_p < 1.0f) {
    const float room = fmaxf(budget - above, 0.f);
    const float q = floorf(room / e_cut) + 1.f;
    if (q < static_cast<float>(n_ties)) keep_ties = static_cast<int>(q);
  }
  const float inv = 1.f / (above + static_cast<float>(keep_ties) * e_cut);

  // write: key > kcut kept; key == kcut kept for the first keep_ties tokens in index order
  int base = 0;  // ties seen in earlier chunks
  for (int c0 = 0; c0 < vocab; c0 += kThreads) {
    const int i = c0 + threadIdx.x;
    const uint32_t ki = i < vocab ? load_key(i) : 0u;
    const bool tie = i < vocab && ki == kcut;
    const uint32_t ballot = __ballot_sync(0xffffffffu, tie);
    if (keep_ties < n_ties) {  // uniform branch: rank the ties of this chunk by index
      __syncthreads();
      if (lane == 0) warp_base[warp] = __popc(ballot);
      __syncthreads();
      int before = 0, total = 0;
      for (int wI = 0; wI < 32; ++wI) {
        const int cnt = warp_base[wI];
        if (wI < warp) before += cnt;
        total += cnt;
      }
      const int rank = base + before + __popc(ballot & ((1u << lane) - 1u));
      base += total;
      if (i < vocab) {
        const bool keep = ki > kcut || (tie && rank < keep_ties);
        prow[i] = keep ? expf(key_to_float(ki) - mx) * inv : 0.f;
      }
    } else if (i < vocab) {
      prow[i] = ki >= kcut ? expf(key_to_float(ki) - mx) * inv : 0.f;
    }
  }
}

}  // namespace sampling
}  // namespace b200

extern "C" {

int b200_argmax_bf16(const void* logits, int64_t ld, int64_t* out, int rows, int vocab, b200_stream_t stream) {
  using namespace b200;
  if (!logits || !out || rows <= 0 || vocab <= 0 || ld < vocab) return B200_ERR_INVALID_ARGUMENT;
  return launch_pdl(sampling::argmax_kernel, dim3(rows), dim3(sampling::kThreads), 0,
                    reinterpret_cast<cudaStream_t>(stream), static_cast<const uint16_t*>(logits), ld, out, vocab,
                    static_cast<uint64_t*>(nullptr), static_cast<int64_t>(0));
}

int b200_argmax_shard_bf16(const void* logits, int64_t ld, uint64_t* keys, int rows, int vocab, int64_t index_offset,
                           b200_stream_t stream) {
  using namespace b200;
  if (!logits || !keys || rows <= 0 || vocab <= 0 || ld < vocab || index_offset < 0 || index_offset + vocab > 0xffffffffll)
    return B200_ERR_INVALID_ARGUMENT;
  return launch_pdl(sampling::argmax_kernel, dim3(rows), dim3(sampling::kThreads), 0,
                    reinterpret_cast<cudaStream_t>(stream), static_cast<const uint16_t*>(logits), ld,
                    static_cast<int64_t*>(nullptr), vocab, keys, index_offset);
}

int b200_argmax_merge(const uint64_t* keys, int shards, int rows, int64_t* out, b200_stream_t stream) {
  using namespace b200;
  if (!keys || !out || shards <= 0 || rows <= 0) return B200_ERR_INVALID_ARGUMENT;
  return launch_pdl(sampling::argmax_merge_kernel, dim3((rows + 127) / 128), dim3(128), 0,
                    reinterpret_cast<cudaStream_t>(stream), keys, shards, rows, out);
}

int b200_topk_probs_bf16(const void* logits, int64_t ld, float* probs, int rows, int vocab, int top_k,
                         float temperature, b200_stream_t stream) {
  using namespace b200;
  if (!logits || !probs || rows <= 0 || vocab <= 0 || ld < vocab) return B200_ERR_INVALID_ARGUMENT;
  if (top_k < 1 || top_k > vocab || !(temperature > 0.f)) return B200_ERR_INVALID_ARGUMENT;
  return launch_pdl(sampling::topk_probs_kernel, dim3(rows), dim3(sampling::kThreads), 0,
                    reinterpret_cast<cudaStream_t>(stream), static_cast<const uint16_t*>(logits), ld, probs, vocab,
                    top_k, temperature);
}

int b200_topp_probs_bf16(const void* logits, int64_t ld, float* probs, int rows, int vocab, float top_p,
                         float temperature, b200_stream_t stream) {
  using namespace b200;
  if (!logits || !probs || rows <= 0 || vocab <= 0 || ld < vocab) return B200_ERR_INVALID_ARGUMENT;
  if (!(top_p > 0.f) || top_p > 1.f || !(temperature > 0.f)) return B200_ERR_INVALID_ARGUMENT;
  return launch_pdl(sampling::topp_probs_kernel, dim3(rows), dim3(sampling::kThreads), 0,
                    reinterpret_cast<cudaStream_t>(stream), static_cast<const uint16_t*>(logits), ld, probs, vocab,
                    top_p, temperature);
}

}  // extern "C"
