"""Dynamic inference engine: request admission, the step loop, per-request bookkeeping
(reference ``megatron/core/inference/engines/dynamic_engine.py:68-227, 363-706``).  The ZMQ data-parallel
coordinator of the reference is serving plumbing and is not part of this engine."""
from __future__ import annotations

import asyncio
import time
from collections import deque
from itertools import count, repeat
from typing import Dict, List, Optional, Union

import torch
from torch import Tensor

from ..contexts.dynamic_context import ContextOverflowError, DynamicInferenceContext, WarmupEngineMode
from ..inference_request import DynamicInferenceRequest, Status
from ..sampling_params import SamplingParams
from ..text_generation_controllers.text_generation_controller import TextGenerationController, get_asyncio_loop
from ...utils import nvtx_range_pop, nvtx_range_push


class DynamicInferenceEngine:
    def __init__(self, controller: TextGenerationController, context: DynamicInferenceContext, termination_id: int,
                 enable_cuda_graph: Optional[bool] = None, random_seed: Optional[int] = None, *,
                 track_paused_request_events: bool = False, overlap_host_and_device: bool = False):
        assert isinstance(controller, TextGenerationController)
        assert isinstance(context, DynamicInferenceContext)
        assert isinstance(termination_id, int)
        assert isinstance(random_seed, int)
        self.controller, self.context = controller, context
        self.termination_id, self.random_seed = termination_id, random_seed
        self.track_paused_request_events = track_paused_request_events
        # Not in the reference: in decode steps the controller enqueues the NEXT forward before it returns, so the
        # GPU runs while this engine post-processes the step (same tokens; see the controller).
        controller.enqueue_next_forward_early = bool(overlap_host_and_device)
        self.step_count = 0
        self.finished_request_count = 0
        self.waiting_request_ids = deque()
        self.failed_request_ids: List[int] = []
        self.request_counter = count()
        self.requests: Dict[int, DynamicInferenceRequest] = {}
        self.request_completion_futures: Dict[int, asyncio.Future] = {}
        self._cuda = torch.cuda.is_available()
        if self._cuda:
            self.step_start_event = torch.cuda.Event(enable_timing=True)
            self.step_end_event = torch.cuda.Event(enable_timing=True)
        self._loop = get_asyncio_loop()
        model = controller.inference_wrapped_model.model
        if enable_cuda_graph is not None:
            model.config.enable_cuda_graph = enable_cuda_graph
        self.enable_cuda_graph = model.config.enable_cuda_graph
        self.capture_stats = None
        if self.enable_cuda_graph and context.cuda_graph_token_counts is not None and self._cuda:
            # Warm up and capture one whole-model graph per token count, for decode steps and - when the context
            # pads short prefill / mixed steps to the same sizes - for those as well (reference :143-227 captures
            # per-layer graphs for the same sizes and modes; a mixed step needs at least two tokens).
            t0 = time.time()
            captured = 0
            for mode in (WarmupEngineMode.DECODE, WarmupEngineMode.NON_DECODE):
                if mode == WarmupEngineMode.NON_DECODE and not context.non_decode_cuda_graphs:
                    continue
                for n in context.cuda_graph_token_counts:
                    if n == 1 and mode == WarmupEngineMode.NON_DECODE:
                        continue
                    context.initialize_attention_state(num_warmup_tokens=n, warmup_engine_mode=mode)
                    assert n == context.padded_active_token_count
                    ids, pos = context.current_input_and_position_ids(num_warmup_tokens=n)
                    controller.inference_wrapped_model.run_one_forward_step(
                        {"tokens": ids, "position_ids": pos, "attention_mask": None})
                    context.reset()
                    captured += 1
            self.capture_stats = {"time": time.time() - t0, "graphs": captured}

    # ------------------------------------------------------------------------------------------
    def has_unfinished_requests(self) -> bool:
        return self.context.has_unfinished_requests() or len(self.waiting_request_ids) > 0

    def reset(self) -> None:
        self.context.reset()
        self.waiting_request_ids.clear()
        self.step_count = 0
        self.finished_request_count = 0

    def _add_request(self, request: DynamicInferenceRequest) -> asyncio.Future:
        request_id = request.request_id
        self.requests[request_id] = request
        if request.status is None:
            request.status = Status.ACTIVE_AND_GENERATING_TOKENS
        try:
            self.context.add_request(request_id, request.prompt_tokens, request.sampling_params.num_tokens_to_generate)
            request.add_event_add()
        except ContextOverflowError as e:
            if e.is_transient:
                request.status = Status.WAITING_IN_QUEUE
                self.waiting_request_ids.append(request_id)
                request.add_event_error_transient(e)
            else:
                request.status = Status.FAILED
                self.failed_request_ids.append(request_id)
                request.add_event_error_nontransient(e)
        self.request_completion_futures[request_id] = self._loop.create_future()
        return self.request_completion_futures[request_id]

    def add_request(self, request_id: int, prompt: Union[str, List[int], Tensor],
                    num_tokens_to_generate: Optional[int] = None) -> asyncio.Future:
        """Queue a request (text, token list, or int64 tensor on the host or the device)."""
        if isinstance(prompt, str):
            tokens = torch.tensor(self.controller.tokenize_prompt(prompt), dtype=torch.int64)
        elif isinstance(prompt, list):
            tokens = torch.tensor(prompt, dtype=torch.int64)
        elif isinstance(prompt, Tensor):
            assert prompt.dtype == torch.int64, prompt.dtype
            tokens = prompt
        else:
            raise Exception("specialize for <%s>." % type(prompt).__name__)
        request = DynamicInferenceRequest(
            request_id=request_id, prompt_tokens=tokens,
            sampling_params=SamplingParams(num_tokens_to_generate=num_tokens_to_generate))
        return self._add_request(request)

    def post_process_requests(self, request_ids, finished_request_ids, step_time, sample, log_probs):
        active_requests: List[DynamicInferenceRequest] = []
        finished_requests: List[DynamicInferenceRequest] = []
        finished = set(finished_request_ids.tolist())
        self.finished_request_count += len(finished)
        for request_id, token, lp in zip(request_ids.tolist(), sample.tolist(), log_probs if log_probs else repeat(None)):
            request = self.requests[request_id]
            request.generated_tokens.append(token)
            if request.tpot is None:
                request.tpot = []
            request.tpot.append(step_time)
            if lp is not None:
                if not request.prompt_log_probs:
                    request.prompt_log_probs = []
                if not request.generated_log_probs:
                    request.generated_log_probs = []
                (request.prompt_log_probs if len(lp) > 1 else request.generated_log_probs).extend(lp)
            if request_id in finished:
                request.generated_length = len(request.generated_tokens)
                request.status = Status.COMPLETED
                done = self.requests.pop(request_id)
                detok = getattr(self.controller.tokenizer, "detokenize", None)
                done.generated_text = detok(done.generated_tokens) if detok else None
                finished_requests.append(done)
                fut = self.request_completion_futures.get(request_id)
                if fut is not None and not fut.done():
                    fut.set_result(done)
            else:
                active_requests.append(request)
        return active_requests, finished_requests

    def schedule_waiting_requests(self) -> None:
        """Retry queued requests in arrival order; stop at the first that still does not fit."""
        for request_id in list(self.waiting_request_ids):
            request = self.requests[request_id]
            try:
                self.context.add_request(request_id, request.prompt_tokens, request.sampling_params.num_tokens_to_generate)
                request.add_event_add()
                request.status = Status.ACTIVE_AND_GENERATING_TOKENS
                self.waiting_request_ids.popleft()
            except Exception:
                break

    async def async_step(self, sampling_params: SamplingParams, *, verbose: Optional[bool] = False) -> Dict:
        prev_decode = self.context.is_decode_only()
        nvtx_range_push("Decode" if prev_decode else "Prefill")  # reference :562
        # The controller returns after reading the sampled tokens back, i.e. after the step's device work is done:
        # the host clock around the call measures the step (the reference brackets it with CUDA events and then
        # synchronises on the second one, dynamic_engine.py:560-575 - two more driver calls with the GPU idle).
        t0 = time.perf_counter()
        result = await self.controller.async_generate_output_tokens_dynamic_batch(sampling_params, self.termination_id)
        step_time = time.perf_counter() - t0
        cuda_graph_request_count = None
        active_requests: List[DynamicInferenceRequest] = []
        finished_requests: List[DynamicInferenceRequest] = []
        if result is not None:
            newly_paused = result["newly_paused_request_ids"]
            cuda_graph_request_count = result["cuda_graph_request_count"]
            if newly_paused is not None and self.track_paused_request_events:
                for i in newly_paused.tolist():
                    self.requests[i].add_event_pause()
            self.schedule_waiting_requests()
            for i in result["finished_request_ids"].tolist():
                self.requests[i].add_event_finish()
            active_requests, finished_requests = self.post_process_requests(
                result["active_request_ids"], result["finished_request_ids"], step_time, result["sample"], result["log_probs"])
        for failed_id in self.failed_request_ids:
            failed = self.requests.pop(failed_id)
            failed.status = Status.FAILED
            failed.add_event_fail()
            finished_requests.append(failed)
            fut = self.request_completion_futures.get(failed_id)
            if fut is not None and not fut.done():
                fut.set_result(failed)
        self.failed_request_ids.clear()
        if verbose:
            c = self.context
            print("* step %d | %s ... time: %.4f ... reqs: %d [ gtd %d, paused %d, finished %d ]" % (
                self.step_count, "decode" if prev_decode else "non-decode", step_time, c.total_request_count,
                c.gtd_request_count, c.paused_request_count, self.finished_request_count))
        self.step_count += 1
        nvtx_range_pop()  # reference :658
        return {"active_requests": active_requests, "finished_requests": finished_requests, "step_time": step_time,
                "cuda_graph_request_count": cuda_graph_request_count}

    def step_modern(self, sampling_params: SamplingParams, *, verbose: Optional[bool] = False) -> Dict:
        """Synchronous step.  The coroutine is driven to completion right here: its only suspension point is the
        `asyncio.sleep(0)` that lets other coroutines run while the forward is in flight, and the synchronous API
        has none, so the event loop's per-call overhead (tens of microseconds with the GPU idle) is not paid."""
        coro = self.async_step(sampling_params=sampling_params, verbose=verbose)
        try:
            while True:
                if coro.send(None) is not None:  # suspended on a real future: that needs the event loop
                    raise RuntimeError("async_step suspended on a future; use `await engine.async_step(...)`")
        except StopIteration as done:
            return done.value

    def step_legacy(self, sampling_params: SamplingParams, *, verbose: Optional[bool] = False):
        r = self.step_modern(sampling_params, verbose=verbose)
        return (r["active_requests"], r["finished_requests"], r["step_time"])

    step = step_legacy

    def generate(self, prompts: List, sampling_params: Optional[SamplingParams] = SamplingParams()) -> List[DynamicInferenceRequest]:
        """Completions for a static list of prompts (reference :692-706)."""
        for prompt in prompts:
            self.add_request(int(next(self.request_counter)), prompt, sampling_params.num_tokens_to_generate)
        finished: List[DynamicInferenceRequest] = []
        while self.has_unfinished_requests():
            finished.extend(self.step_modern(sampling_params)["finished_requests"])
        return finished
