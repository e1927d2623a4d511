"""Text generation controller of the dynamic path: forward -> last-token logits -> sample ->
finished mask -> context update (reference
``megatron/core/inference/text_generation_controllers/text_generation_controller.py:172-315, 410-565``).
"""
from __future__ import annotations

import asyncio
from typing import Dict, Optional

import numpy as np
import torch

from ... import ops
from ..sampling_params import SamplingParams


def get_asyncio_loop():
    try:
        return asyncio.get_running_loop()
    except RuntimeError:
        try:
            loop = asyncio.get_event_loop_policy().get_event_loop()
        except RuntimeError:
            loop = asyncio.new_event_loop()
            asyncio.set_event_loop(loop)
        return loop


class TextGenerationController:
    def __init__(self, inference_wrapped_model, tokenizer, pp_group=None):
        self.inference_wrapped_model = inference_wrapped_model
        self.tokenizer = tokenizer
        self.pp_group = pp_group
        self.model_is_pipeline_parallel = False
        cfg = inference_wrapped_model.model.config
        dev = "cuda" if torch.cuda.is_available() else "cpu"
        self.sampling_rng = torch.Generator(device=dev)
        self.sampling_rng.manual_seed(cfg.inference_sampling_seed)

    # Off by default (the reference's step is strictly forward -> sample -> update); the engine may switch it on.
    enqueue_next_forward_early = False
    _early_forward = None

    # --------------------------------------------------------------------------------------------
    def tokenize_prompt(self, prompt: str, add_BOS: bool = False):
        tokens = self.tokenizer.tokenize(prompt)
        return [self.tokenizer.bos] + tokens if add_BOS else tokens

    # --------------------------------------------------------------------------------------------
    def sample_from_logits(self, last_token_logits: torch.Tensor, sampling_params: Optional[SamplingParams] = None,
                           vocab_size: Optional[int] = None, generation_started: Optional[torch.Tensor] = None,
                           top_n_logprobs_dict=None, logits: Optional[torch.Tensor] = None, **kwargs) -> torch.Tensor:
        """Sample one token per row of ``last_token_logits [batch, vocab]`` (bf16, on the device).

        ``top_k == 1``: greedy, the argmax kernel (ties go to the smallest index).  ``top_k > 1``: the
        top-k kernel produces the filtered, temperature-scaled probabilities and ``torch.multinomial``
        draws from them with the controller's generator, as the reference does (:292-309).  ``top_k == 0``
        with ``top_p == 0`` keeps the whole vocabulary.  ``top_p > 0``: the nucleus kernel (the reference's
        sort + cumulative sum + shift-by-one rule, :221-240, evaluated in fp32 without a sort).
        ``generation_started``, ``top_n_logprobs_dict`` and ``logits`` serve the reference's top-n log-probabilities
        (static batching only); they are accepted for the signature and unused.
        """
        if kwargs.get("common_inference_params"):
            sampling_params = kwargs["common_inference_params"]
        top_p, top_k, temperature = sampling_params.top_p, sampling_params.top_k, sampling_params.temperature
        assert isinstance(top_p, float) and isinstance(top_k, int)
        assert not (top_k > 0 and top_p > 0.0), "Cannot have top-p and top-k both greater than zero"
        assert top_p <= 1.0, "top-p should be in (0,1]"
        if sampling_params.top_n_logprobs > 0:
            raise NotImplementedError("top-n log-probabilities are outside the decode path built here")
        if hasattr(last_token_logits, "greedy_tokens"):  # this rank's vocabulary shard (tensor parallel)
            if top_k == 1:
                return last_token_logits.greedy_tokens()
            last_token_logits = last_token_logits.gather()  # everything else samples from the full rows
        if top_k == 1:
            return ops.argmax(last_token_logits)
        if top_k > 1 or (top_k == 0 and top_p == 0.0):
            if top_k > 1:
                assert top_k <= last_token_logits.size(1), "top-k is larger than logit size."
                if vocab_size:
                    assert top_k < vocab_size, "top-k is larger than vocab size."
            keep = top_k if top_k > 1 else last_token_logits.size(1)
            probs = ops.topk_probs(last_token_logits, keep, temperature)
            sampled = torch.multinomial(probs, num_samples=1, generator=self.sampling_rng).view(-1)
            if vocab_size:
                sampled = torch.clamp(sampled, min=0, max=vocab_size - 1)
            return sampled
        probs = ops.topp_probs(last_token_logits, top_p, temperature)
        sampled = torch.multinomial(probs, num_samples=1, generator=self.sampling_rng).view(-1)
        if vocab_size:
            sampled = torch.clamp(sampled, min=0, max=vocab_size - 1)
        return sampled

    # --------------------------------------------------------------------------------------------
    @torch.inference_mode()
    async def async_generate_output_tokens_dynamic_batch(self, sampling_params: SamplingParams, termination_id: int) -> Optional[Dict]:
        """One engine step; returns the dict of the reference (:548-555) or None when idle.

        The sampled tokens are read back once (the only device->host transfer of the step); the finished
        mask and the context update then run on the host.  ``sample`` and the id tensors in the result
        are host tensors.
        """
        context = self.inference_wrapped_model.inference_context
        materialize_last = context.materialize_only_last_token_logits
        if sampling_params.return_log_probs:
            skip = getattr(sampling_params, "skip_prompt_log_probs_for_dynamic_inference", False)
            assert skip or materialize_last is False, "Materialize only last token logits must be false for returning log probs"
        early, self._early_forward = getattr(self, "_early_forward", None), None
        if context.active_token_count == 0:
            return None

        if early is not None and early[0] == context.state_version and context.is_decode_only():
            logits = early[1]  # this step's forward was enqueued at the end of the previous call (see below)
        else:
            context.initialize_attention_state()
            input_ids, position_ids = context.current_input_and_position_ids()
            logits = self.inference_wrapped_model.run_one_forward_step(
                {"tokens": input_ids, "position_ids": position_ids, "attention_mask": None})
        if hasattr(logits, "greedy_tokens") and (not materialize_last or sampling_params.return_log_probs):
            logits = logits.gather().unsqueeze(0)  # every token's logits / log-probs are wanted: the full rows
        cuda_graph_request_count = context.padded_active_request_count if context.is_decode_only() else None
        await asyncio.sleep(0)  # the forward is enqueued; let other coroutines run

        last_token_logits = logits.squeeze(0) if materialize_last else context.last_token_logits(logits)
        vocab_size = self.inference_wrapped_model.inference_wrapper_config.padded_vocab_size
        new_sample_dev = self.sample_from_logits(last_token_logits.contiguous(), sampling_params, vocab_size=vocab_size)
        new_sample = new_sample_dev.cpu()  # the step's one synchronising read

        # finished mask on the host (the request-level state lives there): numpy views, no tensor ops
        p, t = context.paused_request_count, context.total_request_count
        ids_np = context.request_ids.numpy()[p:t]
        seq_np = context.request_kv_length_offsets.numpy()[p:t] + context.request_query_lengths.numpy()[p:t] + 1
        mask_np = ((new_sample.numpy() != termination_id) & (seq_np < context.request_output_lengths.numpy()[p:t])).astype(np.uint8)
        active_request_ids = torch.from_numpy(ids_np.astype(np.int64))
        finished_request_ids = torch.from_numpy(ids_np[mask_np == 0].copy())

        log_probs = None
        if sampling_params.return_log_probs:
            log_probs = context.calculate_log_probs(logits, new_sample_dev, only_last_token_logits=materialize_last)

        newly_paused_request_ids = context.update_requests(mask_np, new_sample.numpy())
        if (self.enqueue_next_forward_early and not sampling_params.return_log_probs and materialize_last
                and context.active_token_count > 0 and context.is_decode_only()):
            # The next decode step depends on nothing the caller still has to do with this step's result (request
            # records, detokenisation, scheduling): enqueue its forward now, so that the GPU works while the host
            # does that.  If the set of requests changes before the next call (add_request / reset bump the
            # context's state version), the early forward is simply not used: it wrote the same keys / values the
            # repeated step writes again.
            context.initialize_attention_state()
            input_ids, position_ids = context.current_input_and_position_ids()
            self._early_forward = (context.state_version, self.inference_wrapped_model.run_one_forward_step(
                {"tokens": input_ids, "position_ids": position_ids, "attention_mask": None}))
        return {
            "active_request_ids": active_request_ids,
            "newly_paused_request_ids": newly_paused_request_ids,
            "finished_request_ids": finished_request_ids,
            "sample": new_sample,
            "log_probs": log_probs,
            "cuda_graph_request_count": cuda_graph_request_count,
        }

    @torch.inference_mode()
    def generate_output_tokens_dynamic_batch(self, sampling_params: SamplingParams, termination_id: int):
        """Synchronous wrapper of `async_generate_output_tokens_dynamic_batch`."""
        return get_asyncio_loop().run_until_complete(
            self.async_generate_output_tokens_dynamic_batch(sampling_params, termination_id))
