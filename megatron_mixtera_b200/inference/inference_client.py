"""Asynchronous client of the data-parallel coordinator (same protocol and public methods as the reference's
``InferenceClient``, ``megatron/core/inference/inference_client.py:30-190``): a ZMQ DEALER socket, one
`asyncio.Future` per submitted request, a background task that resolves them as the finished records arrive."""
from __future__ import annotations

import asyncio
import os
import time
from typing import Dict, List, Union

from .headers import Headers
from .inference_request import DynamicInferenceRequest
from .sampling_params import SamplingParams


class InferenceClient:
    def __init__(self, inference_coordinator_port: int):
        import msgpack
        import zmq

        self._zmq, self._msgpack = zmq, msgpack
        self.context = zmq.Context()
        self.socket = self.context.socket(zmq.DEALER)
        address = os.getenv("MASTER_ADDR", "127.0.0.1")
        self.socket.connect(f"tcp://{address}:{inference_coordinator_port}")
        self.completion_futures: Dict[int, asyncio.Future] = {}
        self.request_submission_times: Dict[int, float] = {}
        self.next_request_id = 0
        self.listener_task = None

    def _send(self, payload: list) -> None:
        self.socket.send(self._msgpack.packb(payload, use_bin_type=True))

    def add_request(self, prompt: Union[str, List[int]], sampling_params: SamplingParams) -> asyncio.Future:
        """Submit a prompt (text or token ids); the future resolves to the finished `DynamicInferenceRequest`."""
        request_id = self.next_request_id
        self.next_request_id += 1
        assert request_id not in self.completion_futures
        self.completion_futures[request_id] = asyncio.get_event_loop().create_future()
        self.request_submission_times[request_id] = time.perf_counter()
        self._send([Headers.SUBMIT_REQUEST.value, request_id, prompt, sampling_params.serializable()])
        return self.completion_futures[request_id]

    async def _listen_for_completed_requests(self, poll_s: float = 0.005):
        while True:
            try:
                request_id, reply = self._msgpack.unpackb(self.socket.recv(flags=self._zmq.NOBLOCK), raw=False)
            except self._zmq.Again:
                await asyncio.sleep(poll_s)
                continue
            latency = time.perf_counter() - self.request_submission_times.pop(request_id)
            record = DynamicInferenceRequest.deserialize(reply)
            record.latency = latency
            self.completion_futures.pop(request_id).set_result(record)

    def _connect_with_inference_coordinator(self, timeout_s: float = 30.0) -> None:
        self._send([Headers.CONNECT.value])
        if not self.socket.poll(int(timeout_s * 1000)):
            raise TimeoutError("the inference coordinator did not acknowledge the connection")
        reply = self._msgpack.unpackb(self.socket.recv(), raw=False)[0]
        assert Headers(reply) == Headers.ACK

    async def start(self):
        """Handshake with the coordinator, then start the listener; await this before submitting requests."""
        self._connect_with_inference_coordinator()
        self.listener_task = asyncio.create_task(self._listen_for_completed_requests())

    def _send_signal_to_engines(self, signal: Headers) -> None:
        self._send([signal.value])

    def pause_engines(self):
        self._send_signal_to_engines(Headers.PAUSE)

    def unpause_engines(self):
        self._send_signal_to_engines(Headers.UNPAUSE)

    def stop_engines(self):
        self._send_signal_to_engines(Headers.STOP)

    def stop(self):
        if self.listener_task is not None:
            self.listener_task.cancel()
        self.socket.close(linger=0)
        self.context.term()
