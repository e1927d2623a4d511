"""CPU oracle for the dynamic-inference decode step.  TEST INFRASTRUCTURE ONLY.

This file restates, on the CPU, the algorithm of the reference's dynamic-inference decode
path (Megatron Core 0.15.0rc6).  It is the checker the parity tests, the smoke test and the
benchmark's CPU-baseline leg use; nothing in the shipped package imports it, and the
shipped package never falls back to it.

Parity pins: every function below is checked (tests/test_oracle_golden.py) against
fixtures under tests/golden/ that were produced by running the reference itself on CPU
(tests/golden/make_golden.py): integer bookkeeping bit-exactly, logits and greedy tokens of
the fp32 and bf16 model cases exactly.  Two third-party pieces have no CPU implementation
in the reference and are therefore *parity unpinned* at kernel level: the flash-attn paged
attention call (restated here from its documented contract) and Transformer Engine's FP8
quantisation (restated here from the OCP MX / E4M3 definitions).

Reference files followed (paths inside the reference project):
  megatron/core/inference/contexts/dynamic_chunk_allocator.py
  megatron/core/inference/contexts/dynamic_context.py
  megatron/core/inference/text_generation_controllers/text_generation_controller.py
  megatron/core/models/gpt/gpt_model.py, megatron/core/transformer/{attention,mlp,transformer_layer}.py
  megatron/core/models/common/embeddings/{rope_utils,rotary_pos_embedding}.py
  megatron/core/tensor_parallel/layers.py, megatron/core/fusions/{fused_bias_swiglu,fused_bias_dropout}.py
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

import numpy as np
import torch
import torch.nn.functional as F


# ======================================================================================
# 1. Integer bookkeeping (numpy)
# ======================================================================================
class OverflowOracle(Exception):
    """kind in {'token','request','chunk','max_seq'}; is_transient as dynamic_context.py:30-83."""

    def __init__(self, kind: str, is_transient: bool = True):
        super().__init__(kind)
        self.kind = kind
        self.is_transient = is_transient


class ChunkAllocatorOracle:
    """LIFO stack of chunk ids; the last id is the dummy chunk (dynamic_chunk_allocator.py:23-34)."""

    def __init__(self, chunk_count_total: int, gtd_chunk_count: int):
        self.chunk_count_total = chunk_count_total
        self.gtd_chunk_count = gtd_chunk_count
        self.chunk_count_avail = chunk_count_total - 1
        self.dummy_chunk_idx = chunk_count_total - 1
        self.chunk_bag = np.arange(chunk_count_total, dtype=np.int32)

    def is_memory_available(self, n: int, safe: bool = False) -> bool:
        # dynamic_chunk_allocator.py:36-54
        return self.chunk_count_avail >= n + (self.gtd_chunk_count if safe else 0)

    def allocate(self, n: int = 1, safe: bool = False) -> Optional[np.ndarray]:
        # dynamic_chunk_allocator.py:56-71 — pops the top n entries, returned bottom-to-top
        if not self.is_memory_available(n, safe):
            return None
        self.chunk_count_avail -= n
        return self.chunk_bag[self.chunk_count_avail : self.chunk_count_avail + n].copy()

    def release(self, chunks: np.ndarray) -> None:
        # dynamic_chunk_allocator.py:73-84
        n = len(chunks)
        self.chunk_bag[self.chunk_count_avail : self.chunk_count_avail + n] = chunks
        self.chunk_count_avail += n


def _round_up(value: int, rounder: int, tp: int) -> int:
    # dynamic_context.py:416-456
    r = math.ceil(rounder / tp) * tp
    return r * int(math.ceil(int(value) / r))


class ContextOracle:
    """numpy restatement of DynamicInferenceContext's bookkeeping (no KV data, no CUDA graphs)."""

    def __init__(
        self,
        *,
        dtype_bytes: int,
        num_layers: int,
        kv_channels: int,
        num_attention_heads: int,
        max_sequence_length: int,
        buffer_size_gb: float,
        buffer_guaranteed_fraction: float,
        chunk_size_tokens: int = 256,
        buffer_overflow_factor: Optional[float] = None,
        max_requests_override: Optional[int] = None,
        max_tokens_override: Optional[int] = None,
        tensor_model_parallel_size: int = 1,
        token_rounder: int = 64,
        request_rounder: int = 4,
    ):
        tp = tensor_model_parallel_size
        self.tp = tp
        self.token_rounder, self.request_rounder = token_rounder, request_rounder
        heads_pp = num_attention_heads // tp
        self.chunk_size_tokens = chunk_size_tokens
        # dynamic_context.py:205-212
        self.chunk_size_bytes = dtype_bytes * 2 * num_layers * chunk_size_tokens * heads_pp * kv_channels
        # :215-217
        buf = int(buffer_size_gb * 1024**3)
        buf -= buf % self.chunk_size_bytes
        # :220-242
        n_tokens = buf / self.chunk_size_bytes * chunk_size_tokens
        n_requests = n_tokens / max_sequence_length
        self.max_requests = _round_up(int(n_requests), request_rounder, tp)
        self.max_tokens = _round_up(int(n_tokens), token_rounder, tp)
        if buffer_overflow_factor is not None:
            self.max_requests = _round_up(int(self.max_requests * buffer_overflow_factor), request_rounder, tp)
            self.max_tokens = _round_up(int(self.max_tokens * buffer_overflow_factor / 50.0), token_rounder, tp)
        if max_requests_override is not None:
            self.max_requests = _round_up(max_requests_override, request_rounder, tp)
        if max_tokens_override is not None:
            self.max_tokens = _round_up(max_tokens_override, token_rounder, tp)
        self.max_requests = min(self.max_requests, self.max_tokens)
        self.max_sequence_length = max_sequence_length
        self.total_request_count = 0
        self.active_token_count = 0
        self.paused_request_count = 0
        self.padded_active_token_count = None
        self.padded_active_request_count = None
        self.paused_tokens = None
        R, Tm = self.max_requests, self.max_tokens
        self.request_ids = np.full(R, -1, np.int32)
        self.request_query_lengths = np.zeros(R, np.int32)
        self.request_output_lengths = np.zeros(R, np.int32)
        self.request_kv_length_offsets = np.zeros(R, np.int32)
        self.request_kv_chunk_counts = np.zeros(R, np.int32)
        self.request_last_kv_chunk_id = np.zeros(R, np.int32)
        self.request_last_kv_chunk_offset = np.zeros(R, np.int32)
        self.token_to_input_ids = np.zeros(Tm, np.int64)
        self.token_to_pos_ids = np.zeros(Tm, np.int64)
        self.token_to_request_idx = np.zeros(Tm, np.int64)
        self.token_to_chunk_idx = np.zeros(Tm, np.int64)
        self.token_to_position_in_request = np.zeros(Tm, np.int64)
        self.token_to_local_position_within_kv_chunk = np.zeros(Tm, np.int64)
        self.chunk_count_total = buf // self.chunk_size_bytes  # :285
        self.max_kv_chunk_count = math.ceil(max_sequence_length / chunk_size_tokens)  # :311
        self.request_to_kv_chunk_ids = np.full((R, self.max_kv_chunk_count), -1, np.int32)
        # :398-401
        gtd = min(int(buffer_guaranteed_fraction * self.chunk_count_total), self.chunk_count_total)
        self.gtd_request_count = max(1, gtd // self.max_kv_chunk_count)
        self.gtd_chunk_count = self.gtd_request_count * self.max_kv_chunk_count
        self.chunk_allocator = ChunkAllocatorOracle(self.chunk_count_total, self.gtd_chunk_count)
        self.dummy_chunk_idx = self.chunk_allocator.dummy_chunk_idx
        self.kv_seq_lengths = None
        self.block_table = None
        self.cu_query_seq_lengths = None
        self.cu_kv_seq_lengths = None
        self.max_seqlen_q = self.max_seqlen_k = None

    # dynamic_context.py:472-479
    def is_decode_only(self) -> bool:
        return (self.total_request_count - self.paused_request_count) == self.active_token_count

    def has_unfinished_requests(self) -> bool:
        return self.total_request_count > 0

    # dynamic_context.py:920-1015
    def add_request(self, request_id: int, tokens: np.ndarray, num_tokens_to_generate: Optional[int] = None):
        n = int(len(tokens))
        if n > self.max_tokens:
            raise OverflowOracle("token", True)
        if self.active_token_count + n > self.max_tokens:
            raise OverflowOracle("token", True)
        if self.total_request_count >= self.max_requests:
            raise OverflowOracle("request", True)
        need = math.ceil(n / self.chunk_size_tokens)
        ids = self.chunk_allocator.allocate(need, safe=True)
        if ids is None:
            raise OverflowOracle("chunk", True)
        if num_tokens_to_generate is None:
            num_tokens_to_generate = self.max_sequence_length - n
        elif n + num_tokens_to_generate > self.max_sequence_length:
            # The reference raises after the chunks were popped (:967-974); the pop is not undone.
            raise OverflowOracle("max_seq", False)
        r = self.total_request_count
        self.request_ids[r] = request_id
        self.request_query_lengths[r] = n
        self.request_output_lengths[r] = n + num_tokens_to_generate
        self.request_kv_length_offsets[r] = 0
        self.request_to_kv_chunk_ids[r, :need] = ids
        self.request_kv_chunk_counts[r] = need
        self.request_last_kv_chunk_id[r] = ids[-1]
        self.request_last_kv_chunk_offset[r] = (n - 1) % self.chunk_size_tokens
        a = self.active_token_count
        ar = np.arange(n)
        self.token_to_pos_ids[a : a + n] = ar
        self.token_to_input_ids[a : a + n] = tokens
        self.token_to_request_idx[a : a + n] = r
        self.token_to_position_in_request[a : a + n] = ar
        self.token_to_chunk_idx[a : a + n] = ids[ar // self.chunk_size_tokens]
        self.token_to_local_position_within_kv_chunk[a : a + n] = ar % self.chunk_size_tokens
        self.total_request_count += 1
        self.active_token_count += n

    # dynamic_context.py:656-825, branch without CUDA graphs
    def initialize_attention_state(self):
        self.padded_active_token_count = _round_up(self.active_token_count, self.token_rounder, self.tp)
        dec = self.is_decode_only()
        if dec:
            self.padded_active_token_count = min(self.padded_active_token_count, self.max_requests)
        p, t = self.paused_request_count, self.total_request_count
        self.padded_active_request_count = self.padded_active_token_count if dec else (t - p)
        a, pa = self.active_token_count, self.padded_active_token_count
        self.token_to_chunk_idx[a:pa] = self.dummy_chunk_idx
        self.token_to_local_position_within_kv_chunk[a:pa] = 0
        self.token_to_position_in_request[a:pa] = 0
        ql = self.request_query_lengths[p:t]
        kv = (self.request_kv_length_offsets + self.request_query_lengths)[p:t]
        if dec:
            self.cu_query_seq_lengths = None
            self.max_seqlen_q = 1
            full = np.zeros(self.padded_active_request_count, np.int32)
            full[: t - p] = kv
            self.kv_seq_lengths = full
            self.cu_kv_seq_lengths = None
            self.max_seqlen_k = self.max_sequence_length
            bt = np.zeros((self.padded_active_request_count, self.max_kv_chunk_count), np.int32)
            bt[: t - p] = self.request_to_kv_chunk_ids[p:t]
            self.block_table = bt
        else:
            self.cu_query_seq_lengths = np.concatenate([[0], np.cumsum(ql)]).astype(np.int32)
            self.max_seqlen_q = int(ql.max())
            self.kv_seq_lengths = kv.astype(np.int32)
            self.cu_kv_seq_lengths = np.concatenate([[0], np.cumsum(kv)]).astype(np.int32)
            self.max_seqlen_k = int(kv.max())
            self.block_table = self.request_to_kv_chunk_ids[p:t].copy()

    def get_active_sequence_lengths(self):
        p, t = self.paused_request_count, self.total_request_count
        return (self.request_kv_length_offsets + self.request_query_lengths)[p:t]

    def get_max_sequence_lengths(self):
        return self.request_output_lengths[self.paused_request_count : self.total_request_count]

    def _move(self, src, dst, next_tokens):
        # dynamic_context.py:1017-1030 (right-hand sides are gathered before assignment)
        for arr in (
            self.request_kv_length_offsets,
            self.request_query_lengths,
            self.request_output_lengths,
            self.request_ids,
            next_tokens,
            self.request_to_kv_chunk_ids,
            self.request_kv_chunk_counts,
            self.request_last_kv_chunk_id,
            self.request_last_kv_chunk_offset,
        ):
            arr[dst] = arr[src]

    # dynamic_context.py:1033-1298
    def update_requests(self, active_requests_mask: np.ndarray, new_tokens: np.ndarray):
        mask = np.asarray(active_requests_mask)
        active = int((mask == 1).sum())
        finished = int((mask == 0).sum())
        assert active + finished + self.paused_request_count == self.total_request_count
        self.kv_seq_lengths = self.block_table = None
        P = self.paused_request_count
        if active + P == 0:  # step 2
            if finished > 0:
                idx = np.nonzero(mask == 0)[0] + P
                rows = self.request_to_kv_chunk_ids[idx]
                self.chunk_allocator.release(rows[rows != -1])
            self.request_to_kv_chunk_ids.fill(-1)
            self.total_request_count = 0
            self.active_token_count = 0
            return None
        new_tokens = np.asarray(new_tokens).copy()
        next_tokens = np.concatenate([self.paused_tokens, new_tokens]) if P != 0 else new_tokens  # step 3
        if finished > 0:  # step 4
            idx = np.nonzero(mask == 0)[0] + P
            rows = self.request_to_kv_chunk_ids[idx]
            self.chunk_allocator.release(rows[rows != -1])
            self.request_to_kv_chunk_ids[idx] = -1
            if active > 0:
                fin_left = np.nonzero(mask[:active] == 0)[0] + P
                act_right = np.nonzero(mask[active:])[0] + active + P
                self._move(act_right, fin_left, next_tokens)
                self.request_to_kv_chunk_ids[act_right] = -1
        newly_paused = None
        if active > 0:  # step 5
            last = self.request_last_kv_chunk_offset[P : P + active]
            need = (last == self.chunk_size_tokens - 1).astype(np.uint8)
            n_need = int(need.sum())
            if 0 < n_need != active:
                act_left = np.nonzero(need[:n_need] == 0)[0] + P
                pau_right = np.nonzero(need[n_need:])[0] + n_need + P
                dst = np.concatenate([act_left, pau_right])
                src = np.concatenate([pau_right, act_left])
                self._move(src, dst, next_tokens)
                newly_paused = self.request_ids[dst].copy()
            self.paused_request_count += n_need
            active -= n_need
        # step 6
        non_gtd = max(0, self.chunk_allocator.chunk_count_avail - self.gtd_chunk_count)
        if non_gtd:
            resume = min(non_gtd, self.paused_request_count)
        else:
            resume = min(max(self.gtd_request_count - active, 0), self.paused_request_count)
        self.paused_request_count -= resume
        active += resume
        assert active > 0
        if newly_paused is not None and resume > 0:
            newly_paused = newly_paused[:-resume]
        # step 7
        self.total_request_count = active + self.paused_request_count
        self.active_token_count = active
        P, T = self.paused_request_count, self.total_request_count
        self.token_to_input_ids[:active] = next_tokens[P:T]
        if P > 0:
            self.paused_tokens = next_tokens[:P].copy()
        self.request_kv_length_offsets[P:T] += self.request_query_lengths[P:T]
        self.request_query_lengths[P:T] = 1
        self.token_to_pos_ids[:active] = self.request_kv_length_offsets[P:T]
        self.request_last_kv_chunk_offset[P:T] = (self.request_last_kv_chunk_offset[P:T] + 1) % self.chunk_size_tokens
        if resume > 0:  # step 8
            assert np.all(self.request_last_kv_chunk_offset[P : P + resume] == 0)
            ids = self.chunk_allocator.allocate(resume)
            rows = np.arange(P, P + resume)
            cols = self.request_kv_chunk_counts[P : P + resume]
            self.request_to_kv_chunk_ids[rows, cols] = ids
            self.request_kv_chunk_counts[P : P + resume] += 1
            self.request_last_kv_chunk_id[P : P + resume] = ids
        # step 9
        self.token_to_request_idx[:active] = np.arange(P, T)
        self.token_to_position_in_request[:active] = self.request_kv_length_offsets[P:T]
        self.token_to_chunk_idx[:active] = self.request_last_kv_chunk_id[P:T]
        self.token_to_local_position_within_kv_chunk[:active] = self.request_last_kv_chunk_offset[P:T]
        return newly_paused


# ======================================================================================
# 2. Model arithmetic (torch CPU, in the parameter dtype, same op order as the local spec)
# ======================================================================================
@dataclass
class ModelSpec:
    num_layers: int
    hidden_size: int
    num_attention_heads: int
    num_query_groups: int
    kv_channels: int
    ffn_hidden_size: int
    vocab_size: int
    max_sequence_length: int
    llama: bool = True  # RMSNorm + RoPE + SwiGLU + no bias; False: LayerNorm + learned pos + GELU + bias
    rotary_base: float = 500000.0
    eps: float = 1e-5


def rope_freqs(max_seq: int, dim: int, base: float) -> torch.Tensor:
    """fp32 angle table [max_seq, dim], halves duplicated (rotary_pos_embedding.py:79-81,150-181)."""
    inv_freq = 1.0 / (base ** (torch.arange(0, dim, 2, dtype=torch.float32) / dim))
    seq = torch.arange(max_seq, dtype=torch.float32)
    f = torch.outer(seq, inv_freq)
    return torch.cat((f, f), dim=-1)


def apply_rope(t: torch.Tensor, freqs: torch.Tensor) -> torch.Tensor:
    """t [T, heads, d], freqs [T, d] fp32: cos/sin cast to t.dtype before use (rope_utils.py:92-126)."""
    cos_ = torch.cos(freqs).to(t.dtype)[:, None, :]
    sin_ = torch.sin(freqs).to(t.dtype)[:, None, :]
    x1, x2 = torch.chunk(t, 2, dim=-1)
    rot = torch.cat((-x2, x1), dim=-1)
    return (t * cos_) + (rot * sin_)


def quantize_kv_fp8(x: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    """E4M3 KV-pool entry (extension, not in the reference): RNE-saturate(x / scale[head]); x [T, heads, d]."""
    return _to_e4m3(x.float() / scale[None, :, None])


def paged_attention(q, k_cache, v_cache, kv_lens, block_table, cu_q=None, k_scale=None, v_scale=None):
    """flash-attn paged contract (attention.py:470-601): q [T,nq,d]; caches [chunks,chunk,nkv,d].

    fp32 softmax, scale d^-1/2, head h reads KV head h // g, causal bottom-right aligned,
    rows with kv_len 0 give zeros; output cast to q.dtype.  With ``k_scale`` / ``v_scale`` (fp32 [heads]) the
    caches hold E4M3 values that are multiplied by their head's scale.
    """
    T, H, D = q.shape
    Hkv, cs = k_cache.shape[2], k_cache.shape[1]
    g = H // Hkv
    out = torch.zeros_like(q)
    qlens = [1] * block_table.shape[0] if cu_q is None else (cu_q[1:] - cu_q[:-1]).tolist()
    off = 0
    for r, ql in enumerate(qlens):
        kl = int(kv_lens[r])
        if kl == 0 or ql == 0:
            off += ql
            continue
        nb = math.ceil(kl / cs)
        ids = torch.as_tensor(block_table[r, :nb]).long()
        kk = k_cache[ids].reshape(-1, Hkv, D)[:kl].float()
        vv = v_cache[ids].reshape(-1, Hkv, D)[:kl].float()
        if k_scale is not None:
            kk, vv = kk * k_scale[None, :, None], vv * v_scale[None, :, None]
        kk, vv = kk.repeat_interleave(g, 1), vv.repeat_interleave(g, 1)
        qq = q[off : off + ql].float()
        s = torch.einsum("qhd,khd->hqk", qq, kk) * (D**-0.5)
        m = torch.ones(ql, kl, dtype=torch.bool).tril(kl - ql)
        s = s.masked_fill(~m, float("-inf"))
        out[off : off + ql] = torch.einsum("hqk,khd->qhd", s.softmax(-1), vv).to(q.dtype)
        off += ql
    return out


class GPTOracle:
    """Forward of the local-spec GPT over a ContextOracle (gpt_model.py:279-560, transformer_layer.py:433-660)."""

    def __init__(self, spec: ModelSpec, weights: Dict[str, torch.Tensor], ctx: ContextOracle, dtype: torch.dtype,
                 fp8: Optional[str] = None, kv_fp8_scale: Optional[float] = None, tp: int = 1, reverse_k: bool = False):
        """``fp8="mxfp8"`` / ``"blockwise"``: every decoder linear multiplies FP8-quantised inputs by FP8-quantised
        weights with fp32 accumulation (the TE recipes of those names under ``fp8_autocast``,
        transformer_block.py:629-643; E8M0 scale per 32 elements, resp. fp32 scale per 128 x 128 / 1 x 128 block);
        embedding, norms, attention and the output layer stay in ``dtype``."""
        self.s, self.w, self.ctx, self.dtype = spec, weights, ctx, dtype
        self.fp8 = fp8
        # reverse_k: every linear accumulates its K dimension in the opposite order.  Same arithmetic, same rounding
        # points, another (equally valid) summation order: the distance between a run with and a run without it is
        # the noise floor that separates ANY two correct implementations of this model in this dtype.
        self.reverse_k = reverse_k
        # split_k = n > 1: every linear adds up n partial products over consecutive K ranges (fp32), the way a split-K
        # GEMM does.  Another equally valid summation order; combined with reverse_k it gives further "twins".
        self.split_k = 1
        # tp > 1 restates the arithmetic of the reference's tensor-parallel run: a row-parallel linear (out-proj,
        # fc2; layers.py:1225-1281) multiplies its K shard on every rank, each partial product is rounded to the
        # parameter dtype, and the all-reduce adds the rounded partials (mappings.py:22-33).  Column-parallel
        # linears and attention heads are exact under sharding, so nothing else changes.
        self.tp = tp
        self._wdq: Dict[str, torch.Tensor] = {}
        # E4M3 KV pool (extension): every head uses the same scale here; values are kept dequantised in the
        # caches (byte * scale is exact in fp32), so the attention restatement itself is unchanged
        self.kv_fp8_scale = kv_fp8_scale
        nkv = spec.num_query_groups
        self.k_cache = torch.full(
            (spec.num_layers, ctx.chunk_count_total, ctx.chunk_size_tokens, nkv, spec.kv_channels), -1.0,
            dtype=torch.float32 if kv_fp8_scale is not None else dtype
        )
        self.v_cache = self.k_cache.clone()
        self.freqs = rope_freqs(spec.max_sequence_length, spec.kv_channels, spec.rotary_base) if spec.llama else None

    def _norm(self, x, prefix):
        s = self.s
        if s.llama:
            return F.rms_norm(x, (s.hidden_size,), self.w[prefix + ".weight"], s.eps)
        return F.layer_norm(x, (s.hidden_size,), self.w[prefix + ".weight"], self.w[prefix + ".bias"], s.eps)

    def _mm(self, x, w):
        """x @ w.T (layers.py:333), optionally with the K dimension accumulated in another order."""
        if self.split_k > 1 and x.shape[-1] % self.split_k == 0:
            ks = x.shape[-1] // self.split_k
            parts = [torch.matmul(x[..., i * ks:(i + 1) * ks].float(), w[:, i * ks:(i + 1) * ks].float().t())
                     for i in (range(self.split_k - 1, -1, -1) if self.reverse_k else range(self.split_k))]
            acc = parts[0]
            for p in parts[1:]:
                acc = acc + p
            return acc.to(x.dtype)
        if self.reverse_k:
            key = ("flip", w.data_ptr(), tuple(w.shape))
            if key not in self._wdq:
                self._wdq[key] = w.flip(-1).contiguous()
            return torch.matmul(x.flip(-1).contiguous(), self._wdq[key].t())
        return torch.matmul(x, w.t())

    def _linear(self, x, prefix, add_bias=True):
        if self.tp > 1 and prefix.endswith(("linear_proj", "linear_fc2")):
            K = x.shape[-1]
            assert K % self.tp == 0
            ks = K // self.tp
            w_full = self.w[prefix + ".weight"]
            y = None
            for r in range(self.tp):
                part = self._matmul_shard(x[..., r * ks : (r + 1) * ks], w_full[:, r * ks : (r + 1) * ks], f"{prefix}@{r}")
                y = part.float() if y is None else y + part.float()
            y = y.to(x.dtype)
            b = self.w.get(prefix + ".bias")
            return y + b if (add_bias and b is not None) else y
        if self.fp8 == "mxfp8":
            if prefix not in self._wdq:
                self._wdq[prefix] = dequantize_mxfp8(*quantize_mxfp8(self.w[prefix + ".weight"]))
            y = self._mm(dequantize_mxfp8(*quantize_mxfp8(x)), self._wdq[prefix]).to(x.dtype)
        elif self.fp8 == "blockwise":
            if prefix not in self._wdq:
                self._wdq[prefix] = dequantize_fp8_block_weight(*quantize_fp8_block_weight(self.w[prefix + ".weight"]))
            y = self._mm(dequantize_fp8_rowblock(*quantize_fp8_rowblock(x)), self._wdq[prefix]).to(x.dtype)
        else:
            y = self._mm(x, self.w[prefix + ".weight"])  # layers.py:333
        b = self.w.get(prefix + ".bias")
        if add_bias and b is not None:
            y = y + b
        return y

    def _matmul_shard(self, x, w, key):
        """x @ w.T for one K shard, rounded to x.dtype (FP8 recipes quantise the shard like a whole operand)."""
        if self.fp8 == "mxfp8":
            if key not in self._wdq:
                self._wdq[key] = dequantize_mxfp8(*quantize_mxfp8(w.contiguous()))
            return self._mm(dequantize_mxfp8(*quantize_mxfp8(x.contiguous())), self._wdq[key]).to(x.dtype)
        if self.fp8 == "blockwise":
            if key not in self._wdq:
                self._wdq[key] = dequantize_fp8_block_weight(*quantize_fp8_block_weight(w.contiguous()))
            return self._mm(dequantize_fp8_rowblock(*quantize_fp8_rowblock(x.contiguous())), self._wdq[key]).to(x.dtype)
        return self._mm(x, w)

    def forward(self) -> torch.Tensor:
        """Returns last-token logits [active requests, vocab] in the parameter dtype."""
        s, c, w = self.s, self.ctx, self.w
        T = c.padded_active_token_count
        ids = torch.from_numpy(c.token_to_input_ids[:T])
        pos = torch.from_numpy(c.token_to_pos_ids[:T])
        x = w["embedding.word_embeddings.weight"][ids]
        if not s.llama:
            x = x + w["embedding.position_embeddings.weight"][pos]  # language_model_embedding.py:99-149
        nq, nkv, d = s.num_attention_heads, s.num_query_groups, s.kv_channels
        g = nq // nkv
        chunk_idx = torch.from_numpy(c.token_to_chunk_idx[:T])
        local = torch.from_numpy(c.token_to_local_position_within_kv_chunk[:T])
        pos_in_req = torch.from_numpy(c.token_to_position_in_request[:T])
        cu_q = None if c.cu_query_seq_lengths is None else torch.from_numpy(c.cu_query_seq_lengths)
        for l in range(s.num_layers):
            p = f"decoder.layers.{l}."
            h = self._norm(x, p + "input_layernorm")
            qkv = self._linear(h, p + "self_attention.linear_qkv").view(T, nkv, (g + 2) * d)  # attention.py:985-1021
            q = qkv[..., : g * d].reshape(T, nq, d)
            k = qkv[..., g * d : (g + 1) * d]
            v = qkv[..., (g + 1) * d :]
            if s.llama:
                k = apply_rope(k, self.freqs[pos_in_req])  # dynamic_context.py:600-631
            if self.kv_fp8_scale is not None:
                sc = torch.full((nkv,), self.kv_fp8_scale)
                k = (quantize_kv_fp8(k, sc).float() * self.kv_fp8_scale).to(torch.float32)
                v = (quantize_kv_fp8(v, sc).float() * self.kv_fp8_scale).to(torch.float32)
            self.k_cache[l][chunk_idx, local] = k.to(self.k_cache.dtype)  # dynamic_context.py:511-545
            self.v_cache[l][chunk_idx, local] = v.to(self.v_cache.dtype)
            if s.llama:
                q = apply_rope(q, self.freqs[pos])  # dynamic_context.py:566-598
            o = paged_attention(q, self.k_cache[l], self.v_cache[l], c.kv_seq_lengths, c.block_table, cu_q)
            a = self._linear(o.reshape(T, nq * d), p + "self_attention.linear_proj", add_bias=False)
            b = w.get(p + "self_attention.linear_proj.bias")
            if b is not None:
                a = a + b  # fused_bias_dropout.py:39-57
            x = a + x
            h = self._norm(x, p + "pre_mlp_layernorm")
            f1 = self._linear(h, p + "mlp.linear_fc1")  # mlp.py:140-213
            if s.llama:
                y1, y2 = torch.chunk(f1, 2, dim=-1)
                act = F.silu(y1) * y2  # fused_bias_swiglu.py:15-26
            else:
                act = F.gelu(f1)
            f2 = self._linear(act, p + "mlp.linear_fc2", add_bias=False)
            b = w.get(p + "mlp.linear_fc2.bias")
            if b is not None:
                f2 = f2 + b
            x = f2 + x
        x = self._norm(x, "decoder.final_layernorm")
        P, Tt = c.paused_request_count, c.total_request_count
        last = torch.from_numpy(np.cumsum(c.request_query_lengths[P:Tt]) - 1).long()  # dynamic_context.py:890-918
        return self._mm(x[last], w["output_layer.weight"])


# ======================================================================================
# 3. Sampling (text_generation_controller.py:172-315)
# ======================================================================================
def sample(logits: torch.Tensor, top_k: int = 1, top_p: float = 0.0, temperature: float = 1.0, generator=None):
    if top_k == 1:
        return torch.argmax(logits, dim=-1)
    probs = filtered_probabilities(logits, top_k, top_p, temperature)
    return torch.multinomial(probs, num_samples=1, generator=generator).view(-1)


def filtered_probabilities(logits, top_k: int, top_p: float, temperature: float, softmax_dtype=None) -> torch.Tensor:
    """The probability vector handed to multinomial (exact support; used for top-k/top-p parity).

    The reference takes the final softmax in the logits' dtype; ``softmax_dtype=torch.float32``
    gives the same distribution before that last rounding."""
    x = logits.clone()
    if temperature != 1.0:
        x.div_(temperature)
    if top_k > 1:
        kth = torch.topk(x, top_k)[0][..., -1, None]
        x.masked_fill_(x < kth, float("-inf"))
    elif top_p > 0.0:
        sl, si = torch.sort(x, descending=True, stable=True)  # equal logits keep index order
        cp = sl.softmax(dim=-1).cumsum(dim=-1)
        f = cp > top_p
        f[:, 1:] = f[:, :-1].clone()
        f[..., 0] = 0
        f = f.scatter(1, si, f)
        x.masked_fill_(f, float("-inf"))
    return (x if softmax_dtype is None else x.to(softmax_dtype)).softmax(dim=-1)


def decode_loop(model: GPTOracle, prompts, num_tokens_to_generate, arrival=None, termination_id=-1, on_step=None):
    """Drives add_request / forward / greedy sample / update_requests like
    text_generation_controller.py:410-555; returns {request id: generated tokens}."""
    c = model.ctx
    arrival = arrival or [0] * len(prompts)
    gen = {i: [] for i in range(len(prompts))}
    step, added = 0, 0
    while added < len(prompts) or c.has_unfinished_requests():
        for i, p in enumerate(prompts):
            if arrival[i] == step:
                c.add_request(i, np.asarray(p), num_tokens_to_generate)
                added += 1
        if c.active_token_count > 0:
            c.initialize_attention_state()
            logits = model.forward()
            new = sample(logits).numpy()
            P, T = c.paused_request_count, c.total_request_count
            ids = c.request_ids[P:T].copy()
            seq = c.get_active_sequence_lengths() + 1
            mask = ((new != termination_id) & (seq < c.get_max_sequence_lengths())).astype(np.uint8)
            if on_step is not None:
                on_step(step, c, logits, new, ids)
            for rid, tok in zip(ids.tolist(), new.tolist()):
                gen[rid].append(tok)
            c.update_requests(mask, new.copy())
        step += 1
    return gen


# ======================================================================================
# 4. FP8 quantisation restatements (parity unpinned: Transformer Engine is a third-party
#    dependency, version 2.7.0, absent from the reference checkout and from this image)
# ======================================================================================
E4M3_MAX = 448.0


def _to_e4m3(x: torch.Tensor) -> torch.Tensor:
    """Round-to-nearest-even, saturating cast to E4M3 (fn variant: no inf, max 448)."""
    return x.float().clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn)


def quantize_mxfp8(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """MX format: blocks of 32 along the last dim share a power-of-two scale 2^(e-127), stored E8M0.

    The scale is the smallest power of two >= amax / 448 (rounding the exponent UP, so nothing saturates):
    this is what Transformer Engine's MXFP8 recipe does; the OCP text rounds down and saturates.  The biased
    exponent is read off the fp32 bits of amax / 448, +1 if any mantissa bit is set, clamped to 254.
    elements = RNE-saturate(x / scale).  Returns (e4m3 values, uint8 biased exponents [..., K/32]).
    """
    shp = x.shape
    xb = x.float().reshape(*shp[:-1], shp[-1] // 32, 32)
    amax = xb.abs().amax(dim=-1)
    bits = (amax / 448.0).view(torch.int32)
    e = ((bits >> 23) & 0xFF) + ((bits & 0x7FFFFF) != 0).int()
    e = e.clamp(max=254)
    inv = torch.ldexp(torch.ones_like(amax), 127 - e)
    q = _to_e4m3(xb * inv[..., None]).reshape(shp)
    return q, e.to(torch.uint8)


def mxfp8_scales_to_tile_layout(e8m0: torch.Tensor) -> torch.Tensor:
    """[rows, K/32] scale bytes -> the GEMM's tile layout [ceil(rows/256)*2][K/128][512] (flattened)."""
    rows, kb = e8m0.shape
    tiles = -(-rows // 256) * 2
    out = torch.zeros(tiles, kb // 4, 512, dtype=torch.uint8)
    r = torch.arange(rows)
    b = torch.arange(kb)
    off = ((r % 32) * 16 + ((r % 128) // 32) * 4)[:, None] + (b % 4)[None, :]
    out[(r // 128)[:, None].expand(rows, kb), (b // 4)[None, :].expand(rows, kb), off] = e8m0
    return out.reshape(-1)


def dequantize_mxfp8(q: torch.Tensor, e8m0: torch.Tensor) -> torch.Tensor:
    shp = q.shape
    s = torch.ldexp(torch.ones(e8m0.shape), e8m0.int() - 127)
    return (q.float().reshape(*shp[:-1], shp[-1] // 32, 32) * s[..., None]).reshape(shp)


def quantize_fp8_block_weight(w: torch.Tensor, block: int = 128) -> Tuple[torch.Tensor, torch.Tensor]:
    """128x128-block fp32-scaled E4M3: scale = amax / 448 per block; q = RNE-saturate(w / scale)."""
    N, K = w.shape
    nb, kb = math.ceil(N / block), math.ceil(K / block)
    wp = torch.zeros(nb * block, kb * block)
    wp[:N, :K] = w.float()
    blocks = wp.reshape(nb, block, kb, block)
    amax = blocks.abs().amax(dim=(1, 3))
    scale = (amax / E4M3_MAX).clamp_min(1e-30)
    q = _to_e4m3(blocks / scale[:, None, :, None]).reshape(nb * block, kb * block)[:N, :K]
    return q.contiguous(), scale


def quantize_fp8_rowblock(a: torch.Tensor, block: int = 128) -> Tuple[torch.Tensor, torch.Tensor]:
    """1x128 per-token activation scales (fp32): scale = amax / 448 per row block."""
    M, K = a.shape
    ab = a.float().reshape(M, K // block, block)
    scale = (ab.abs().amax(dim=-1) / E4M3_MAX).clamp_min(1e-30)
    return _to_e4m3(ab / scale[..., None]).reshape(M, K), scale


def dequantize_fp8_block_weight(q, scale, block: int = 128):
    N, K = q.shape
    s = scale.repeat_interleave(block, 0)[:N].repeat_interleave(block, 1)[:, :K]
    return q.float() * s


def dequantize_fp8_rowblock(q, scale, block: int = 128):
    return q.float() * scale.repeat_interleave(block, 1)
