// Stand-alone MXFP8 quantiser: bf16 [rows, K] -> E4M3 [rows, K] + E8M0 scales in the GEMM's tile layout.
// Used for weights (once, at load) and for activations whose producer is not fused with quantisation.
#include "quant.cuh"

namespace b200 {
namespace mx {

__global__ void __launch_bounds__(256)
quantize_kernel(const __nv_bfloat16* __restrict__ x, int64_t ldx, uint8_t* __restrict__ q, void* __restrict__ sf,
                int K, int k_tiles, int mode, int m_pad, int packed) {
  pdl_launch_dependents();
  pdl_wait();
  const int row = blockIdx.x;
  const int nvec = K / 8;
  const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<int64_t>(row) * ldx);
  for (int base = blockIdx.y * blockDim.x; base < nvec; base += gridDim.y * blockDim.x) {
    const int i = base + threadIdx.x;
    const bool valid = i < nvec;
    float v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    if (valid) {
      const uint4 u = src[i];
      const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        v[2 * k] = bf16_lo(w[k]);
        v[2 * k + 1] = bf16_hi(w[k]);
      }
    }
    quantize8_any(mode, v, valid, row, i * 8, q, K, sf, k_tiles, m_pad, packed != 0);
  }
}

// Weights of the 128-block recipe: one fp32 scale = amax / 448 per 128 x 128 block.  One CTA per block.
__global__ void __launch_bounds__(256)
quantize_weight_block128_kernel(const __nv_bfloat16* __restrict__ w, uint8_t* __restrict__ q, float* __restrict__ scale,
                                int N, int K) {
  __shared__ float red[8];
  __shared__ float s_scale;
  const int nb = blockIdx.x, kb = blockIdx.y;
  const int k_tiles = K / 128;
  // thread t handles row (t / 16) + 16 * i, columns (t % 16) * 8 .. +7
  const int c0 = kb * 128 + (threadIdx.x & 15) * 8;
  float v[8][8];
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int r = nb * 128 + (threadIdx.x >> 4) + 16 * i;
#pragma unroll
    for (int k = 0; k < 8; ++k) v[i][k] = 0.f;
    if (r < N) {
      const uint4 u = *reinterpret_cast<const uint4*>(w + static_cast<int64_t>(r) * K + c0);
      const uint32_t ww[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        v[i][2 * k] = bf16_lo(ww[k]);
        v[i][2 * k + 1] = bf16_hi(ww[k]);
      }
    }
#pragma unroll
    for (int k = 0; k < 8; ++k) amax = fmaxf(amax, fabsf(v[i][k]));
  }
  amax = warp_max(amax);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
  __syncthreads();
  if (threadIdx.x == 0) {
    float a = red[0];
    for (int i = 1; i < 8; ++i) a = fmaxf(a, red[i]);
    s_scale = fmaxf(a / 448.0f, 1e-30f);
    scale[static_cast<int64_t>(nb) * k_tiles + kb] = s_scale;
  }
  __syncthreads();
  const float sc = s_scale;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int r = nb * 128 + (threadIdx.x >> 4) + 16 * i;
    if (r < N) {
      uint32_t o[2];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(v[i][4 * h] / sc, v[i][4 * h + 1] / sc), __NV_SATFINITE, __NV_E4M3);
        const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(v[i][4 * h + 2] / sc, v[i][4 * h + 3] / sc), __NV_SATFINITE, __NV_E4M3);
        o[h] = lo | (hi << 16);
      }
      *reinterpret_cast<uint2*>(q + weight_tile_offset(r, c0, k_tiles)) = make_uint2(o[0], o[1]);  // tile-major
    }
  }
}

}  // namespace mx
}  // namespace b200

extern "C" {

int b200_quantize_mxfp8(const void* x, int64_t ldx, void* q, void* sf, int rows, int K, b200_stream_t stream) {
  using namespace b200;
  if (!x || !q || !sf || rows <= 0 || K <= 0) return B200_ERR_INVALID_ARGUMENT;
  if (K % 128 != 0 || ldx % 8 != 0 || ldx < K || !aligned16(x) || !aligned16(q) || !aligned16(sf)) return B200_ERR_ALIGNMENT;
  const int nvec = K / 8;
  int chunks = (nvec + 255) / 256;
  if (chunks > 8) chunks = 8;
  return launch_pdl(mx::quantize_kernel, dim3(rows, chunks), dim3(256), 0, reinterpret_cast<cudaStream_t>(stream),
                    static_cast<const __nv_bfloat16*>(x), ldx, static_cast<uint8_t*>(q), sf, K, K / 128,
                    static_cast<int>(mx::kQuantMx), 0, 0);
}

size_t b200_fp8_weight_bytes(int N, int K) {
  if (N <= 0 || K <= 0 || K % 128 != 0) return 0;
  return static_cast<size_t>((N + 127) / 128) * 128 * static_cast<size_t>(K);
}

int b200_quantize_mxfp8_weight(const void* w, void* q, void* sf, int N, int K, b200_stream_t stream) {
  using namespace b200;
  if (!w || !q || !sf || N <= 0 || K <= 0) return B200_ERR_INVALID_ARGUMENT;
  if (K % 128 != 0 || !aligned16(w) || !aligned16(q) || !aligned16(sf)) return B200_ERR_ALIGNMENT;
  const int nvec = K / 8;
  int chunks = (nvec + 255) / 256;
  if (chunks > 8) chunks = 8;
  return launch_pdl(mx::quantize_kernel, dim3(N, chunks), dim3(256), 0, reinterpret_cast<cudaStream_t>(stream),
                    static_cast<const __nv_bfloat16*>(w), static_cast<int64_t>(K), static_cast<uint8_t*>(q), sf, K, K / 128,
                    static_cast<int>(mx::kQuantMx), 0, 1);
}

int b200_quantize_fp8_rowblock(const void* x, int64_t ldx, void* q, float* scale, int rows, int K, int m_pad,
                               b200_stream_t stream) {
  using namespace b200;
  if (!x || !q || !scale || rows <= 0 || K <= 0) return B200_ERR_INVALID_ARGUMENT;
  if (K % 128 != 0 || ldx % 8 != 0 || ldx < K || m_pad < rows || m_pad % 4 != 0 || !aligned16(x) || !aligned16(q) ||
      !aligned16(scale))
    return B200_ERR_ALIGNMENT;
  const int nvec = K / 8;
  int chunks = (nvec + 255) / 256;
  if (chunks > 8) chunks = 8;
  return launch_pdl(mx::quantize_kernel, dim3(rows, chunks), dim3(256), 0, reinterpret_cast<cudaStream_t>(stream),
                    static_cast<const __nv_bfloat16*>(x), ldx, static_cast<uint8_t*>(q), static_cast<void*>(scale), K,
                    K / 128, static_cast<int>(mx::kQuantBlock128), m_pad, 0);
}

int b200_quantize_fp8_weight_block128(const void* w, void* q, float* scale, int N, int K, b200_stream_t stream) {
  using namespace b200;
  if (!w || !q || !scale || N <= 0 || K <= 0) return B200_ERR_INVALID_ARGUMENT;
  if (K % 128 != 0 || !aligned16(w) || !aligned16(q)) return B200_ERR_ALIGNMENT;
  return launch_pdl(mx::quantize_weight_block128_kernel, dim3((N + 127) / 128, K / 128), dim3(256), 0,
                    reinterpret_cast<cudaStream_t>(stream), static_cast<const __nv_bfloat16*>(w), static_cast<uint8_t*>(q),
                    scale, N, K);
}

}  // extern "C"
