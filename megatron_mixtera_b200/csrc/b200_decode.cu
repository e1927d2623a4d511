// Single translation unit of libb200_decode.so: the kernels share one device status word and
// one tensor-map cache, so they are compiled together instead of being device-linked.
#include "common.cu"
#include "gemm_bf16.cu"
#include "gemm_mxfp8.cu"
#include "gemm_fp8_block.cu"
#include "quant.cu"
#include "attention.cu"
#include "attention_fp8.cu"
#include "elementwise.cu"
#include "tp_exchange.cu"
#include "sampling.cu"
