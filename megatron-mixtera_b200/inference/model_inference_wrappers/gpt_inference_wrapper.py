"""Forward-step wrapper of the dynamic path (reference
``megatron/core/inference/model_inference_wrappers/abstract_model_inference_wrapper.py:149-216, 352`` and
``inference_wrapper_config.py:9-45``).

Decode-only steps can be replayed from a CUDA graph of the WHOLE model forward, one graph per padded
token count, instead of the reference's one graph per layer: the kernels take all per-step state
through device arrays with fixed addresses, and grid sizes depend only on the padded token count.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional

import torch


@dataclass
class InferenceWrapperConfig:
    hidden_size: int
    params_dtype: torch.dtype
    inference_batch_times_seqlen_threshold: int = -1
    padded_vocab_size: Optional[int] = None
    inference_max_requests: int = 8
    inference_max_seq_length: int = 2560
    fp32_residual_connection: bool = False
    nccl_all_reduce_for_prefill: bool = False

    def add_attributes(self, attribute_value_pair: dict):
        for key, value in attribute_value_pair.items():
            setattr(self, key, value)


class GPTInferenceWrapper:
    def __init__(self, model, inference_wrapper_config: InferenceWrapperConfig, inference_context=None):
        self.model = model
        self.inference_wrapper_config = inference_wrapper_config
        self.inference_context = inference_context
        self.model_is_pipeline_parallel = False
        self._graphs: Dict[int, Any] = {}
        self.graph_replays = 0
        model.eval()
        cfg = getattr(model, "config", None)
        if inference_context is not None and cfg is not None and hasattr(inference_context, "set_prefill_q_block"):
            from ... import ops

            groups = cfg.num_query_groups or cfg.num_attention_heads
            fp8_pool = getattr(inference_context, "kv_cache_fp8", False)  # the prefill kernel reads a bf16 pool
            inference_context.set_prefill_q_block(0 if fp8_pool else ops.prefill_q_block(cfg.num_attention_heads, groups))

    def prep_model_for_inference(self, prompts_tokens=None):
        self.model.eval()

    def _gather_mode(self):
        """``True`` = all-gather the vocabulary-parallel logits inside the forward, as the reference does
        (``abstract_model_inference_wrapper.py:166``); ``"deferred"`` = hand the controller this rank's shard, which
        greedy sampling reduces with 8 bytes per row and rank instead (config ``defer_logits_gather``)."""
        return "deferred" if getattr(self.model.config, "defer_logits_gather", True) else True

    def _forward(self, inference_input):
        return self.model(inference_input["tokens"], inference_input["position_ids"], inference_input["attention_mask"],
                          inference_context=self.inference_context, runtime_gather_output=self._gather_mode())

    def _decode_rows(self, T: int):
        ctx = self.inference_context
        return self.model.forward_rows(ctx.token_to_input_ids[:T], ctx.token_to_pos_ids[:T], ctx, None, self._gather_mode())

    @torch.inference_mode()
    def run_one_forward_step(self, inference_input: Dict[str, Any]) -> torch.Tensor:
        """Logits ``[1, active requests, vocab]`` of the context's current step."""
        ctx = self.inference_context
        use_graph = (getattr(self.model.config, "enable_cuda_graph", False) and ctx.is_decode_only()
                     and ctx.materialize_only_last_token_logits and torch.cuda.is_available())
        if not use_graph:
            return self._forward(inference_input)
        T = ctx.padded_active_token_count
        n_req = ctx.total_request_count - ctx.paused_request_count
        entry = self._graphs.get(T)
        if entry is None:
            # One eager pass sizes every workspace; the decode step is idempotent (it rewrites the same
            # KV slots), so running it again under capture and replay changes nothing.
            self._decode_rows(T)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                out = self._decode_rows(T)
            entry = (graph, out)
            self._graphs[T] = entry
        graph, out = entry
        graph.replay()
        self.graph_replays += 1
        return out[:n_req].unsqueeze(0)
