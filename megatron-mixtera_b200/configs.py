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
    fp8: str = None  # None (bf16 linears) or "mxfp8"
    kv_fp8: str = None  # None (bf16 KV pool), "two_term" or "one_term": E4M3 KV pool and the arithmetic of its kernel

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

# MXFP8 linears and an E4M3 KV pool (per-head scales; one-term attention arithmetic), 128 requests: the single-GPU form of
# the "FP8 weights + FP8 KV" configuration.
LLAMA3_8B_MXFP8_FP8KV_128REQ = Workload(
    name="llama3-8b-shape MXFP8 linears + E4M3 KV (one-term attention) decode, 128 requests, prompt U[256,4096], 256 greedy tokens, KV chunk 256",
    num_layers=32, hidden_size=4096, num_attention_heads=32, num_query_groups=8, kv_channels=128,
    ffn_hidden_size=14336, vocab_size=128256, num_requests=128, prompt_len_range=(256, 4096),
    num_tokens_to_generate=256, fp8="mxfp8", kv_fp8="one_term")

# Two-layer cut of it for profiler captures.
LLAMA3_8B_MXFP8_FP8KV_SHAPE_2LAYER = Workload(
    name="llama3-8b-shape MXFP8 + E4M3 KV (one-term attention) cut to 2 layers, 128 requests, prompt U[256,4096]",
    num_layers=2, hidden_size=4096, num_attention_heads=32, num_query_groups=8, kv_channels=128, ffn_hidden_size=14336,
    vocab_size=128256, num_requests=128, prompt_len_range=(256, 4096), num_tokens_to_generate=24, fp8="mxfp8",
    kv_fp8="one_term")
