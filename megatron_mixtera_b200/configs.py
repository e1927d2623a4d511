"""Named model / workload shapes of the decode benchmark (synthetic weights, synthetic prompts)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Tuple


@dataclass(frozen=True)
class Workload:
    name: str
    num_layers: int
    hidden_size: int
    num_attention_heads: int
    num_query_groups: int
    kv_channels: int
    ffn_hidden_size: int
    vocab_size: int
    num_requests: int
    prompt_len_range: Tuple[int, int]
    num_tokens_to_generate: int
    chunk_size_tokens: int = 256
    rotary_base: float = 500000.0
    log_uniform_lengths: bool = False
    fp8: str = None  # None (bf16 linears), "mxfp8" (E8M0 scale per 32) or "blockwise" (fp32 scale per 128x128 / 1x128)
    kv_fp8: str = None  # None (bf16 KV pool), "two_term" or "one_term": E4M3 KV pool and the arithmetic of its kernel
    min_tp: int = 1  # smallest tensor-parallel size whose weights fit one GPU
    # Prompt tokens admitted per engine step while the cache is being filled (bounds the activation memory of a
    # prefill step; requests beyond it wait in the engine's queue and are admitted over the following steps).
    max_prefill_tokens: int = 0  # 0: all prompts may enter in one step
    # True: the requests' keys / values are written into the pool as seeded noise and only the bookkeeping of the
    # prefill runs (32k - 128k token prompts through a prefill kernel would dominate the run and is not the measured path).
    synthesize_kv: bool = False

    @property
    def max_sequence_length(self) -> int:
        return self.prompt_len_range[1] + self.num_tokens_to_generate


# Llama-3-8B-shaped bf16 decode, 64 concurrent requests, prompts uniform in [128, 2048], 256 output tokens.
LLAMA3_8B_BF16_64REQ = Workload(
    name="llama3-8b-shape bf16 decode, 64 requests, prompt U[128,2048], 256 greedy tokens, KV chunk 256",
    num_layers=32, hidden_size=4096, num_attention_heads=32, num_query_groups=8, kv_channels=128,
    ffn_hidden_size=14336, vocab_size=128256, num_requests=64, prompt_len_range=(128, 2048),
    num_tokens_to_generate=256)

# Two layers of the same shape and batch: small enough for profiler captures (a few GB on the device).
LLAMA3_8B_SHAPE_2LAYER = Workload(
    name="llama3-8b-shape cut to 2 layers, 64 requests, prompt U[128,2048]", num_layers=2, hidden_size=4096,
    num_attention_heads=32, num_query_groups=8, kv_channels=128, ffn_hidden_size=14336, vocab_size=128256,
    num_requests=64, prompt_len_range=(128, 2048), num_tokens_to_generate=24)

# The same shape with MXFP8 linears (E4M3 values, E8M0 scale per 32-element block), bf16 KV cache,
# 128 concurrent requests, prompts uniform in [256, 4096].
LLAMA3_8B_MXFP8_128REQ = Workload(
    name="llama3-8b-shape MXFP8 linears + bf16 KV decode, 128 requests, prompt U[256,4096], 256 greedy tokens, KV chunk 256",
    num_layers=32, hidden_size=4096, num_attention_heads=32, num_query_groups=8, kv_channels=128,
    ffn_hidden_size=14336, vocab_size=128256, num_requests=128, prompt_len_range=(256, 4096),
    num_tokens_to_generate=256, fp8="mxfp8")

# Two-layer cut of the MXFP8 workload (same layer shapes, 128 requests): small enough for a full ncu capture.
LLAMA3_8B_MXFP8_SHAPE_2LAYER = Workload(
    name="llama3-8b-shape MXFP8 cut to 2 layers, 128 requests, prompt U[256,4096]", num_layers=2, hidden_size=4096,
    num_attention_heads=32, num_query_groups=8, kv_channels=128, ffn_hidden_size=14336, vocab_size=128256,
    num_requests=128, prompt_len_range=(256, 4096), num_tokens_to_generate=24, fp8="mxfp8")

# MXFP8 linears and an E4M3 KV pool (per-head scales; two-term attention arithmetic, the one inside the FP8 logit
# tolerance), 128 requests: the short-context form of the "FP8 weights + FP8 KV" configuration.
LLAMA3_8B_MXFP8_FP8KV_128REQ = Workload(
    name="llama3-8b-shape MXFP8 linears + E4M3 KV (two-term attention) decode, 128 requests, prompt U[256,4096], 256 greedy tokens, KV chunk 256",
    num_layers=32, hidden_size=4096, num_attention_heads=32, num_query_groups=8, kv_channels=128,
    ffn_hidden_size=14336, vocab_size=128256, num_requests=128, prompt_len_range=(256, 4096),
    num_tokens_to_generate=256, fp8="mxfp8", kv_fp8="two_term")

# Two-layer cut of it for profiler captures.
LLAMA3_8B_MXFP8_FP8KV_SHAPE_2LAYER = Workload(
    name="llama3-8b-shape MXFP8 + E4M3 KV (two-term attention) cut to 2 layers, 128 requests, prompt U[256,4096]",
    num_layers=2, hidden_size=4096, num_attention_heads=32, num_query_groups=8, kv_channels=128, ffn_hidden_size=14336,
    vocab_size=128256, num_requests=128, prompt_len_range=(256, 4096), num_tokens_to_generate=24, fp8="mxfp8",
    kv_fp8="two_term")

# Llama-3-70B-shaped FP8 decode: E4M3 weights with 128 x 128 block scales, 1 x 128 per-token activation scales,
# bf16 KV cache, 256 concurrent requests, prompts uniform in [512, 8192], 512 output tokens; tensor parallel 2 / 4 / 8.
LLAMA3_70B_FP8BLOCK_256REQ = Workload(
    name="llama3-70b-shape FP8 (128x128 block / 1x128 token scales) linears + bf16 KV decode, 256 requests, prompt U[512,8192], 512 greedy tokens, KV chunk 256",
    num_layers=80, hidden_size=8192, num_attention_heads=64, num_query_groups=8, kv_channels=128,
    ffn_hidden_size=28672, vocab_size=128256, num_requests=256, prompt_len_range=(512, 8192),
    num_tokens_to_generate=512, fp8="blockwise", min_tp=2, max_prefill_tokens=32768)

# Two layers of it with 256 requests and short prompts: the layer shapes and the 256-token GEMMs of the 70B
# workload in a few GB, for profiler captures and single-GPU kernel timing.
LLAMA3_70B_FP8BLOCK_SHAPE_2LAYER = Workload(
    name="llama3-70b-shape FP8-blockwise cut to 2 layers, 256 requests, prompt U[128,1024]", num_layers=2,
    hidden_size=8192, num_attention_heads=64, num_query_groups=8, kv_channels=128, ffn_hidden_size=28672,
    vocab_size=128256, num_requests=256, prompt_len_range=(128, 1024), num_tokens_to_generate=24, fp8="blockwise",
    max_prefill_tokens=32768)

# Long-context paged decode stress: Llama-3-8B shape, MXFP8 linears, E4M3 KV pool with per-head scales (two-term
# attention arithmetic, the one inside the FP8 logit tolerance), 32 requests with contexts log-uniform in
# [32768, 131072], 64 output tokens; KV written as noise (see `synthesize_kv`).
LLAMA3_8B_LONGCTX_FP8KV_32REQ = Workload(
    name="llama3-8b-shape MXFP8 linears + E4M3 KV (two-term attention) long-context decode, 32 requests, context log-U[32768,131072], 64 greedy tokens, KV chunk 256",
    num_layers=32, hidden_size=4096, num_attention_heads=32, num_query_groups=8, kv_channels=128,
    ffn_hidden_size=14336, vocab_size=128256, num_requests=32, prompt_len_range=(32768, 131072),
    num_tokens_to_generate=64, log_uniform_lengths=True, fp8="mxfp8", kv_fp8="two_term", synthesize_kv=True)

# Two-layer cut of the long-context workload (same block tables: 513 columns, 16+ context splits) for tests and captures.
LLAMA3_8B_LONGCTX_FP8KV_SHAPE_2LAYER = Workload(
    name="llama3-8b-shape MXFP8 + E4M3 KV (two-term) long-context cut to 2 layers, 32 requests, context log-U[32768,131072]",
    num_layers=2, hidden_size=4096, num_attention_heads=32, num_query_groups=8, kv_channels=128,
    ffn_hidden_size=14336, vocab_size=128256, num_requests=32, prompt_len_range=(32768, 131072),
    num_tokens_to_generate=24, log_uniform_lengths=True, fp8="mxfp8", kv_fp8="two_term", synthesize_kv=True)

WORKLOADS = {
    "llama3_8b": LLAMA3_8B_BF16_64REQ,
    "llama3_8b_mxfp8": LLAMA3_8B_MXFP8_128REQ,
    "llama3_8b_mxfp8_fp8kv": LLAMA3_8B_MXFP8_FP8KV_128REQ,
    "llama3_70b_fp8block": LLAMA3_70B_FP8BLOCK_256REQ,
    "llama3_8b_longctx_fp8kv": LLAMA3_8B_LONGCTX_FP8KV_32REQ,
    "smoke": LLAMA3_8B_SHAPE_2LAYER,
    "smoke_mxfp8": LLAMA3_8B_MXFP8_SHAPE_2LAYER,
    "smoke_mxfp8_fp8kv": LLAMA3_8B_MXFP8_FP8KV_SHAPE_2LAYER,
    "smoke_70b_fp8block": LLAMA3_70B_FP8BLOCK_SHAPE_2LAYER,
    "smoke_longctx_fp8kv": LLAMA3_8B_LONGCTX_FP8KV_SHAPE_2LAYER,
}
# The configuration the headline metric (FP8 decode tokens/s at TP 1/2/4/8) is quoted on that fits one GPU.
DEFAULT_WORKLOAD = "llama3_8b_mxfp8"
