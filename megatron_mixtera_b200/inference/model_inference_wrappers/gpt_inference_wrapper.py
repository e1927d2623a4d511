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
    # The reference wraps the forward in Transformer Engine's FP8 autocast when this is set.  Here the FP8 recipe belongs
    # to the model (`TransformerConfig.fp8`, weights quantised when they are loaded); a value here is only checked
    # against it.
    fp8: Optional[str] = None

    def add_attributes(self, attribute_value_pair: dict):
        for key, value in attribute_value_pair.items():
            setattr(self, key, value)


class GPTInferenceWrapper:
    def __init__(self, model, inference_wrapper_config: InferenceWrapperConfig, inference_context=None):
        self.model = model
        self.inference_wrapper_config = inference_wrapper_config
        self.inference_context = inference_context
        self.model_is_pipeline_parallel = False
        self._graphs: Dict[Any, Any] = {}
        self.graph_replays = 0
        self.non_decode_graph_replays = 0
        model.eval()
        cfg = getattr(model, "config", None)
        if getattr(inference_wrapper_config, "fp8", None) is not None and getattr(cfg, "fp8", None) is None:
            raise ValueError("InferenceWrapperConfig.fp8 is set but the model was built without an FP8 recipe "
                             "(TransformerConfig.fp8 = 'mxfp8' or 'blockwise')")
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

    def _mixed_rows(self, T: int, last_rows: torch.Tensor):
        ctx = self.inference_context
        return self.model.forward_rows(ctx.token_to_input_ids[:T], ctx.token_to_pos_ids[:T], ctx, last_rows, self._gather_mode())

    def _run_mixed_step_graph(self, T: int, n_req: int) -> torch.Tensor:
        """A prefill / mixed step whose token count the context padded to a CUDA-graph size (the reference's non-decode
        CUDA graphs, ``dynamic_context.py:354-356, 691-697``): every shape is then a function of ``T`` alone - the
        prefill work list has a fixed capacity with empty entries, padding tokens write to the dummy chunk - except
        which rows are the requests' last tokens.  Those indices live in a buffer of ``T`` entries at a fixed address
        that is refreshed before each replay (unused entries point at row 0; their logits are dropped)."""
        ctx = self.inference_context
        entry = self._graphs.get(("mixed", T))
        if entry is None:
            dev = ctx.token_to_input_ids.device
            last_rows = torch.zeros(T, dtype=torch.int64, device=dev)
            host_rows = torch.zeros(T, dtype=torch.int64, pin_memory=True)
            entry = [None, None, last_rows, host_rows]
        _, _, last_rows, host_rows = entry
        host_rows.zero_()
        host_rows[:n_req] = torch.from_numpy(ctx.last_token_indices()).clamp_(min=0)  # (a warm-up step has no tokens)
        last_rows.copy_(host_rows, non_blocking=True)
        if entry[0] is None:
            # One eager pass sizes every workspace; the step is idempotent (it rewrites the same KV slots and its
            # attention reads only what the step itself and earlier steps wrote), so running it again under capture
            # and replay changes nothing.
            self._mixed_rows(T, last_rows)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                out = self._mixed_rows(T, last_rows)
            entry[0], entry[1] = graph, out
            self._graphs[("mixed", T)] = entry
        entry[0].replay()
        self.graph_replays += 1
        self.non_decode_graph_replays += 1
        return entry[1][:n_req].unsqueeze(0)

    @torch.inference_mode()
    def run_one_forward_step(self, inference_input: Dict[str, Any], recv_buffer_seq_len: Optional[int] = None) -> torch.Tensor:
        """Logits ``[1, active requests, vocab]`` of the context's current step (``recv_buffer_seq_len`` is the reference's
        pipeline-parallel receive size: accepted, unused)."""
        ctx = self.inference_context
        graphs_on = (getattr(self.model.config, "enable_cuda_graph", False) and ctx.materialize_only_last_token_logits
                     and torch.cuda.is_available())
        n_req = ctx.total_request_count - ctx.paused_request_count
        if graphs_on and not ctx.is_decode_only() and ctx.using_cuda_graph_this_step() and n_req > 0:
            return self._run_mixed_step_graph(ctx.padded_active_token_count, n_req)
        use_graph = graphs_on and ctx.is_decode_only()
        if not use_graph:
            return self._forward(inference_input)
        T = ctx.padded_active_token_count
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
