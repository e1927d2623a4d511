// MXFP8 quantisation helpers shared by the stand-alone quantiser and the fused producers.
#pragma once

#include <cuda_fp8.h>

#include "common.cuh"

namespace b200 {
namespace mx {

// E8M0 scale byte for a 32-element block with absolute maximum `amax`: the smallest power of two
// 2^(byte-127) >= amax / 448, so that the scaled block never exceeds the E4M3 range (the rounding-up
// rule of Transformer Engine's MXFP8 recipe; the OCP text would round down and saturate).
__device__ __forceinline__ uint32_t e8m0_scale_byte(float amax) {
  const float v = amax / 448.0f;
  const uint32_t bits = __float_as_uint(v);
  uint32_t e = (bits >> 23) & 0xffu;
  if ((bits & 0x7fffffu) != 0u) e += 1u;
  return e > 254u ? 254u : e;
}

// Byte offset of the scale of (row, 32-block kb) in the tile layout [row tile][K/128][512].
__device__ __forceinline__ int64_t sf_offset(int row, int kb, int k_tiles) {
  const int tile = row >> 7;
  const int r = row & 127;
  return (static_cast<int64_t>(tile) * k_tiles + (kb >> 2)) * 512 + (r & 31) * 16 + (r >> 5) * 4 + (kb & 3);
}

// FP8 WEIGHTS are stored tile-major ("packed"): [ceil(N/128)][K/128] tiles of 128 rows x 128 bytes, each tile 16 KiB
// of consecutive memory, so that the GEMM's TMA box (128 rows x 128 bytes of K) is one contiguous DRAM read instead
// of 128 reads of 128 bytes that lie a whole weight row apart.  Offset of byte (row, col) of an [N, K] matrix:
__host__ __device__ __forceinline__ int64_t weight_tile_offset(int row, int col, int k_tiles) {
  return (static_cast<int64_t>(row >> 7) * k_tiles + (col >> 7)) * 16384 + (row & 127) * 128 + (col & 127);
}

// Quantise 8 consecutive values held by this lane; lanes 4j .. 4j+3 of the warp hold one 32-element block.
// Every lane of the warp must call this (inactive lanes pass valid = false and zeros).
__device__ __forceinline__ void quantize8(const float (&v)[8], bool valid, int row, int col0, uint8_t* q, int64_t ldq,
                                          uint8_t* sf, int k_tiles, bool packed = false) {
  float amax = 0.f;
#pragma unroll
  for (int k = 0; k < 8; ++k) amax = fmaxf(amax, fabsf(v[k]));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
  if (!valid) return;
  const uint32_t e = e8m0_scale_byte(amax);
  const float inv = scalbnf(1.0f, 127 - static_cast<int>(e));
  uint32_t w[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(v[4 * h] * inv, v[4 * h + 1] * inv), __NV_SATFINITE, __NV_E4M3);
    const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(v[4 * h + 2] * inv, v[4 * h + 3] * inv), __NV_SATFINITE, __NV_E4M3);
    w[h] = lo | (hi << 16);
  }
  uint8_t* dst = packed ? q + weight_tile_offset(row, col0, k_tiles) : q + static_cast<int64_t>(row) * ldq + col0;
  *reinterpret_cast<uint2*>(dst) = make_uint2(w[0], w[1]);
  if ((col0 & 31) == 0) sf[sf_offset(row, col0 >> 5, k_tiles)] = static_cast<uint8_t>(e);
}

// The 128-block recipe: one fp32 scale = amax / 448 per token per 128 elements of K, stored as
// scale[K/128][m_pad] (block-major, so that the GEMM fetches the scales of a token block with one copy).
// Lanes 16j .. 16j+15 of the warp hold one 128-element block, 8 consecutive values each.
__device__ __forceinline__ void quantize8_block128(const float (&v)[8], bool valid, int row, int col0, uint8_t* q,
                                                   int64_t ldq, float* scale, int m_pad) {
  float amax = 0.f;
#pragma unroll
  for (int k = 0; k < 8; ++k) amax = fmaxf(amax, fabsf(v[k]));
#pragma unroll
  for (int o = 1; o < 16; o <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  if (!valid) return;
  const float sc = fmaxf(amax / 448.0f, 1e-30f);
  uint32_t w[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(v[4 * h] / sc, v[4 * h + 1] / sc), __NV_SATFINITE, __NV_E4M3);
    const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(v[4 * h + 2] / sc, v[4 * h + 3] / sc), __NV_SATFINITE, __NV_E4M3);
    w[h] = lo | (hi << 16);
  }
  *reinterpret_cast<uint2*>(q + static_cast<int64_t>(row) * ldq + col0) = make_uint2(w[0], w[1]);
  if ((col0 & 127) == 0) scale[static_cast<int64_t>(col0 >> 7) * m_pad + row] = sc;
}

enum : int { kQuantMx = 1, kQuantBlock128 = 2 };

// Dispatch used by the fused producers: `sf` is the E8M0 tile buffer (mode 1) or the fp32 scale matrix (mode 2).
__device__ __forceinline__ void quantize8_any(int mode, const float (&v)[8], bool valid, int row, int col0, uint8_t* q,
                                              int64_t ldq, void* sf, int k_tiles, int m_pad, bool packed = false) {
  if (mode == kQuantMx)
    quantize8(v, valid, row, col0, q, ldq, static_cast<uint8_t*>(sf), k_tiles, packed);
  else
    quantize8_block128(v, valid, row, col0, q, ldq, static_cast<float*>(sf), m_pad);
}

}  // namespace mx
}  // namespace b200
