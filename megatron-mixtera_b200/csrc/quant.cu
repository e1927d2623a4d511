// Stand-alone MXFP8 quantiser: bf16 [rows, K] -> E4M3 [rows, K] + E8M0 scales in the GEMM's tile layout.
// Used for weights (once, at load) and for activations whose producer is not fused with quantisation.
#include "quant.cuh"

namespace b200 {
namespace mx {

__global__ void __launch_bounds__(256)
quantize_kernel(const __nv_bfloat16* __restrict__ x, int64_t ldx, uint8_t* __restrict__ q, uint8_t* __restrict__ sf,
                int K, int k_tiles) {
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
    quantize8(v, valid, row, i * 8, q, K, sf, k_tiles);
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
                    static_cast<const __nv_bfloat16*>(x), ldx, static_cast<uint8_t*>(q), static_cast<uint8_t*>(sf), K,
                    K / 128);
}

}  // extern "C"
