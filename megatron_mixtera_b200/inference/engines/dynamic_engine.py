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

from ... import parallel_state
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
        self.paused = False   # set by PAUSE / UNPAUSE / STOP messages of the data-parallel coordinator
        self.stopped = False
        self._cond = asyncio.Condition()  # `run_engine` sleeps on it; `add_request` inside a running loop wakes it
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
        try:  # wake `run_engine` if it is waiting for work (reference :385-391); nothing to wake outside a running loop
            asyncio.get_running_loop().create_task(self._notify_cond_for_new_request())
        except RuntimeError:
            pass
        return self.request_completion_futures[request_id]

    async def _notify_cond_for_new_request(self):
        async with self._cond:
            self._cond.notify_all()

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
        """Retry queued requests in arrival order; stop at the first that still does not fit.

        A queued request that can never fit is failed instead of being retried for ever: one whose retry raises a
        non-transient overflow (it was queued because a transient limit was hit first), and one that does not fit a
        context that holds no other request.  The reference swallows both and leaves the request queued
        (``dynamic_engine.py:518-531``), so its `generate` never returns for such a prompt."""
        for request_id in list(self.waiting_request_ids):
            request = self.requests[request_id]
            try:
                self.context.add_request(request_id, request.prompt_tokens, request.sampling_params.num_tokens_to_generate)
                request.add_event_add()
                request.status = Status.ACTIVE_AND_GENERATING_TOKENS
                self.waiting_request_ids.popleft()
            except ContextOverflowError as e:
                if e.is_transient and self.context.total_request_count > 0:
                    break  # room will appear when running requests finish
                self.waiting_request_ids.popleft()
                request.status = Status.FAILED
                self.failed_request_ids.append(request_id)
                request.add_event_error_nontransient(e)
            except Exception:
                break

    async def async_step(self, sampling_params: SamplingParams, *, verbose: Optional[bool] = False,
                         post_process_requests_locally: bool = True):
        """One engine step.  With ``post_process_requests_locally=False`` (serving under the data-parallel coordinator,
        which keeps the request records) the step returns ``(request ids, finished ids, tokens, log probs)`` or None
        instead of request objects (reference ``dynamic_engine.py:596-605``)."""
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
            if not post_process_requests_locally:
                for i in result["finished_request_ids"].tolist():  # the coordinator owns the record; drop ours
                    self.requests.pop(i, None)
                    self.request_completion_futures.pop(i, None)
                self.finished_request_count += int(result["finished_request_ids"].numel())
                self.step_count += 1
                nvtx_range_pop()
                return result["active_request_ids"], result["finished_request_ids"], result["sample"], result["log_probs"]
            active_requests, finished_requests = self.post_process_requests(
                result["active_request_ids"], result["finished_request_ids"], step_time, result["sample"], result["log_probs"])
        else:
            if self.waiting_request_ids:
                self.schedule_waiting_requests()  # nothing ran: the queue's head gets the empty context (or fails)
            if not post_process_requests_locally:
                nvtx_range_pop()
                return None
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

    async def run_engine(self, sampling_params: SamplingParams, *, verbose: Optional[bool] = False):
        """Step for as long as the task lives: sleeps until a request is active, steps, repeats (reference :803-813).
        Requests still queued because the context is full count as work too: a step retries them."""
        try:
            while True:
                async with self._cond:
                    await self._cond.wait_for(
                        lambda: self.context.get_active_request_count() > 0 or len(self.waiting_request_ids) > 0)
                await self.async_step(sampling_params=sampling_params, verbose=verbose)
        except asyncio.CancelledError:
            pass

    # ------------------------------------------------------------------------------------------
    # Serving under the data-parallel coordinator (reference ``dynamic_engine.py:229-356, 708-872``)
    # ------------------------------------------------------------------------------------------
    async def start_listening_to_data_parallel_coordinator(self, sampling_params: SamplingParams,
                                                           inference_coordinator_port: int,
                                                           launch_inference_coordinator: bool = True):
        """Connect this replica to the coordinator and start the serving loop as a background task.

        The first rank of every tensor-parallel group talks to the coordinator (DEALER socket with the identity
        ``tp-coord-<data-parallel rank>``, registered with an empty frame) and republishes what it receives to the
        other ranks of its group over a PUB / SUB pair on an ``ipc`` endpoint (one node per tensor-parallel group, as
        in the reference), so that every rank adds the same requests before the same step.  With
        ``launch_inference_coordinator`` global rank 0 spawns the coordinator process first."""
        import multiprocessing
        import os
        import tempfile

        import zmq

        from ..data_parallel_inference_coordinator import DataParallelInferenceCoordinator

        dist_rank = torch.distributed.get_rank() if torch.distributed.is_initialized() else 0
        ready = None
        if launch_inference_coordinator and dist_rank == 0:
            spawn = multiprocessing.get_context("spawn")
            ready = spawn.Event()
            self.inference_coordinator_process = spawn.Process(
                target=DataParallelInferenceCoordinator.entrypoint,
                args=(ready, self.controller.tokenizer, inference_coordinator_port,
                      parallel_state.get_data_parallel_world_size()), daemon=True)
            self.inference_coordinator_process.start()
        self.zmq_context = zmq.Context()
        self.zmq_sockets = []
        address = os.getenv("MASTER_ADDR", "127.0.0.1")
        identity = f"tp-coord-{parallel_state.get_data_parallel_rank()}"
        base = os.path.join(tempfile.gettempdir(), f"b200-{inference_coordinator_port}-{identity}")
        self._is_tp_coordinator = parallel_state.get_tensor_model_parallel_rank() == 0
        self._tp_fanout = parallel_state.get_tensor_model_parallel_world_size() > 1
        if self._is_tp_coordinator:
            self.socket_for_receiving_requests = self.zmq_context.socket(zmq.DEALER)
            self.socket_for_receiving_requests.setsockopt(zmq.IDENTITY, identity.encode())
            self.socket_for_receiving_requests.connect(f"tcp://{address}:{inference_coordinator_port}")
            self.socket_for_receiving_requests.send(b"")  # registration
            self.zmq_sockets.append(self.socket_for_receiving_requests)
            if self._tp_fanout:
                self.tensor_parallel_publisher_socket = self.zmq_context.socket(zmq.PUB)
                self.tensor_parallel_publisher_socket.bind(f"ipc://{base}-req")
                self.tensor_parallel_num_msgs_publisher_socket = self.zmq_context.socket(zmq.PUB)
                self.tensor_parallel_num_msgs_publisher_socket.bind(f"ipc://{base}-len")
                self.zmq_sockets += [self.tensor_parallel_publisher_socket, self.tensor_parallel_num_msgs_publisher_socket]
        elif self._tp_fanout:
            self.tensor_parallel_subscriber_socket = self.zmq_context.socket(zmq.SUB)
            self.tensor_parallel_subscriber_socket.connect(f"ipc://{base}-req")
            self.tensor_parallel_subscriber_socket.setsockopt_string(zmq.SUBSCRIBE, "")
            self.tensor_parallel_num_msgs_subscriber_socket = self.zmq_context.socket(zmq.SUB)
            self.tensor_parallel_num_msgs_subscriber_socket.connect(f"ipc://{base}-len")
            self.tensor_parallel_num_msgs_subscriber_socket.setsockopt_string(zmq.SUBSCRIBE, "")
            self.zmq_sockets += [self.tensor_parallel_subscriber_socket, self.tensor_parallel_num_msgs_subscriber_socket]
        if self._tp_fanout:
            self._await_tensor_parallel_subscriptions()
        if ready is not None:
            ready.wait()
        self.engine_loop_task = asyncio.create_task(self.run_engine_with_coordinator(sampling_params))

    def _await_tensor_parallel_subscriptions(self, poll_ms: int = 100) -> None:
        """Collective over the tensor-parallel group: returns once every subscriber provably receives what the group's
        first rank publishes.  A SUB socket's subscription reaches the publisher some time after ``connect`` returns,
        and a PUB socket drops what it has nobody to send to; a barrier after ``connect`` therefore does not keep the
        first request batch from being lost on a rank, which would then step without it.  The publisher sends a probe
        on both sockets per round, the ranks agree (all-reduce, minimum) on whether everybody has seen one on both, and
        a closing marker lets the subscribers discard probes that arrived late."""
        group = parallel_state.get_tensor_model_parallel_group()
        device = "cuda" if torch.distributed.get_backend(group) == "nccl" else "cpu"
        probe, ready = b"\x00probe", b"\x00ready"
        if self._is_tp_coordinator:
            socks = (self.tensor_parallel_num_msgs_publisher_socket, self.tensor_parallel_publisher_socket)
        else:
            socks = (self.tensor_parallel_num_msgs_subscriber_socket, self.tensor_parallel_subscriber_socket)
        live = [False, False]
        while True:
            if self._is_tp_coordinator:
                for sock in socks:
                    sock.send(probe)
                live = [True, True]
            else:
                for i, sock in enumerate(socks):
                    if sock.poll(poll_ms):
                        sock.recv()
                        live[i] = True
            flag = torch.tensor([int(all(live))], dtype=torch.int32, device=device)
            torch.distributed.all_reduce(flag, op=torch.distributed.ReduceOp.MIN, group=group)
            if int(flag.item()) == 1:
                break
        for sock in socks:
            if self._is_tp_coordinator:
                sock.send(ready)
            else:
                while sock.recv() != ready:
                    pass

    def schedule_requests(self) -> int:
        """Drain the messages that have arrived from the coordinator and apply them: new requests are queued, PAUSE /
        UNPAUSE / STOP set the engine's flags.  Collective over the tensor-parallel group: its first rank drains its
        socket, publishes the count and then the messages; the others receive exactly that many, so that all ranks
        see the same batch before the same step (reference ``dynamic_engine.py:708-789``).  Returns the count."""
        import struct

        import msgpack
        import zmq

        from ..headers import Headers

        messages = []
        if self._is_tp_coordinator:
            while True:
                try:
                    messages.append(self.socket_for_receiving_requests.recv(flags=zmq.NOBLOCK))
                except zmq.Again:
                    break
            if self._tp_fanout:
                self.tensor_parallel_num_msgs_publisher_socket.send(struct.pack("!i", len(messages)))
                for m in messages:
                    self.tensor_parallel_publisher_socket.send(m)
        else:
            n = struct.unpack("!i", self.tensor_parallel_num_msgs_subscriber_socket.recv())[0]
            messages = [self.tensor_parallel_subscriber_socket.recv() for _ in range(n)]
        for m in messages:
            data = msgpack.unpackb(m, raw=False)
            header = Headers(data[0])
            if header == Headers.SUBMIT_REQUEST:
                request_id, prompt, params = data[1:]
                params = SamplingParams.deserialize(params)
                self.add_request(request_id, prompt, params.num_tokens_to_generate)
            elif header == Headers.PAUSE:
                self.paused = True
            elif header == Headers.UNPAUSE:
                self.paused = False
            elif header == Headers.STOP:
                self.stopped = True
        return len(messages)

    async def run_engine_with_coordinator(self, sampling_params: SamplingParams, *, verbose: Optional[bool] = False,
                                          idle_sleep_s: float = 0.02):
        """Serving loop of one replica: apply the coordinator's messages, step while there is work, and after every step
        send ``[ENGINE_REPLY, ids, finished ids, tokens, log probs]`` back (first tensor-parallel rank only)."""
        import msgpack

        from ..headers import Headers

        def report_failed_requests():
            # Requests this replica had to give up (they can never fit its context) are reported as finished without
            # tokens, so that the client's future resolves (with an empty completion) instead of waiting for ever; the
            # reference's loop never mentions them to the coordinator.
            if not self.failed_request_ids:
                return
            failed, self.failed_request_ids = list(self.failed_request_ids), []
            for i in failed:
                self.requests.pop(i, None)
                self.request_completion_futures.pop(i, None)
            if self._is_tp_coordinator:
                self.socket_for_receiving_requests.send(msgpack.packb(
                    [Headers.ENGINE_REPLY.value, [], failed, [], None], use_bin_type=True))

        try:
            while True:
                self.schedule_requests()
                report_failed_requests()
                if self.stopped:
                    if self._tp_fanout:
                        # every rank of the group has the STOP message (it arrived in the same batch on all of them)
                        # before the publisher's sockets close and drop what they have not delivered yet
                        torch.distributed.barrier(parallel_state.get_tensor_model_parallel_group())
                    self.stop()
                    return
                if self.paused or (self.context.get_active_request_count() == 0 and not self.waiting_request_ids):
                    await asyncio.sleep(idle_sleep_s)
                    continue
                if self.context.get_active_request_count() == 0:
                    self.schedule_waiting_requests()
                out = await self.async_step(sampling_params=sampling_params, verbose=verbose,
                                            post_process_requests_locally=False)
                if self._is_tp_coordinator and out is not None:
                    request_ids, finished_ids, sample, log_probs = out
                    self.socket_for_receiving_requests.send(msgpack.packb(
                        [Headers.ENGINE_REPLY.value, request_ids.tolist(), finished_ids.tolist(), sample.tolist(), log_probs],
                        use_bin_type=True))
                report_failed_requests()
                await asyncio.sleep(0)
        except asyncio.CancelledError:
            pass

    def stop(self) -> None:
        """Leave the serving set-up: end the coordinator process this engine spawned (if any) and close the sockets."""
        proc = getattr(self, "inference_coordinator_process", None)
        if proc is not None:
            proc.terminate()
        for sock in getattr(self, "zmq_sockets", []):
            sock.close(linger=0)
        self.zmq_sockets = []
        ctx = getattr(self, "zmq_context", None)
        if ctx is not None:
            ctx.term()
            self.zmq_context = None

