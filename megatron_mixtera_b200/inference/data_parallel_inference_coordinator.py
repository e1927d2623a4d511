"""Central router between serving clients and the data-parallel engine replicas.

Same role and wire protocol as the reference's ``DataParallelInferenceCoordinator``
(``megatron/core/inference/data_parallel_inference_coordinator.py:30-322``): one ZMQ ROUTER socket; every message is one
msgpack list whose first element is a `Headers` value.

  engine replica (DEALER, identity ``tp-coord-<dp rank>``)   registers with an empty frame
  client (DEALER)     CONNECT -> ACK;  SUBMIT_REQUEST [client id, prompt, sampling params] -> the coordinator numbers
                      the request, tokenises a text prompt and forwards [SUBMIT_REQUEST, id, tokens, sampling params]
                      to the next replica (round robin);  PAUSE / UNPAUSE / STOP are relayed to every replica
  engine replica      ENGINE_REPLY [ids, finished ids, tokens, log probs] after every step: tokens are appended to the
                      requests' records; a finished request is detokenised and sent to the client that owns it as
                      [client id, record]

Nothing here touches a GPU; the decode path does not depend on this module.  `stop()` from another thread ends the loop
(the reference's loop can only be interrupted from the keyboard)."""
from __future__ import annotations

from collections import deque
from itertools import cycle, repeat
from typing import Dict, List, Optional

import torch

from .headers import Headers
from .inference_request import DynamicInferenceRequest


def _zmq_and_msgpack():
    try:
        import msgpack
        import zmq
    except ImportError as e:  # pragma: no cover - both are present in the supported images
        raise ImportError("the data-parallel coordinator needs pyzmq and msgpack") from e
    return zmq, msgpack


class DataParallelInferenceCoordinator:
    def __init__(self, tokenizer, inference_coordinator_port: int, data_parallel_size: int, *,
                 registration_timeout_s: Optional[float] = None, bind_address: str = "0.0.0.0"):
        """Bind the router and wait until ``data_parallel_size`` engine replicas have registered (blocking, like the
        reference; ``registration_timeout_s`` turns an endless wait into a TimeoutError)."""
        zmq, msgpack = _zmq_and_msgpack()
        self._zmq, self._msgpack = zmq, msgpack
        self.tokenizer = tokenizer
        self.context = zmq.Context()
        self.router_socket = self.context.socket(zmq.ROUTER)
        self.router_socket.bind(f"tcp://{bind_address}:{inference_coordinator_port}")
        self.data_parallel_size = data_parallel_size
        self.identities_of_data_parallel_ranks = deque()
        self._early = []
        deadline_ms = None if registration_timeout_s is None else int(registration_timeout_s * 1000)
        while len(self.identities_of_data_parallel_ranks) < data_parallel_size:
            if deadline_ms is not None and not self.router_socket.poll(deadline_ms):
                raise TimeoutError(f"{len(self.identities_of_data_parallel_ranks)} of {data_parallel_size} engine replicas "
                                   "registered in time")
            identity, payload = self.router_socket.recv_multipart()
            if payload:  # a client was faster than the last replica: keep its message for the event loop
                self._early.append((identity, payload))
                continue
            assert identity not in self.identities_of_data_parallel_ranks, f"replica {identity!r} registered twice"
            self.identities_of_data_parallel_ranks.append(identity)
        self.data_parallel_rank_iterator = cycle(self.identities_of_data_parallel_ranks)
        self.request_id_to_client_id: Dict[int, bytes] = {}
        self.request_id_to_client_request_id: Dict[int, int] = {}
        self.next_request_id = 0
        self.requests: Dict[int, DynamicInferenceRequest] = {}
        self.known_clients = set()
        self._running = False
        self._handlers = {
            Headers.CONNECT: self._on_connect,
            Headers.SUBMIT_REQUEST: self._on_submit,
            Headers.ENGINE_REPLY: self._on_engine_reply,
            Headers.PAUSE: self._on_control,
            Headers.UNPAUSE: self._on_control,
            Headers.STOP: self._on_control,
        }

    # ------------------------------------------------------------------------------------------
    def get_next_data_parallel_rank(self) -> bytes:
        """Identity of the replica the next request goes to (round robin in registration order)."""
        return next(self.data_parallel_rank_iterator)

    def tokenize_prompt(self, prompt: str, add_BOS: bool = False) -> List[int]:
        tokens = self.tokenizer.tokenize(prompt)
        return [self.tokenizer.bos] + tokens if add_BOS else tokens

    def _send(self, identity: bytes, payload: list) -> None:
        self.router_socket.send_multipart([identity, self._msgpack.packb(payload, use_bin_type=True)])

    # ------------------------------------------------------------------------------------------ handlers
    def _on_connect(self, sender: bytes, header: Headers, body: list) -> None:
        if sender in self.known_clients:
            return  # a duplicate CONNECT is ignored
        self.known_clients.add(sender)
        self._send(sender, [Headers.ACK.value])

    def _on_submit(self, sender: bytes, header: Headers, body: list) -> None:
        if sender not in self.known_clients:
            return  # requests of clients that never connected are dropped
        client_request_id, prompt, sampling_params = body
        request_id = self.next_request_id
        self.next_request_id += 1
        self.request_id_to_client_id[request_id] = sender
        self.request_id_to_client_request_id[request_id] = client_request_id
        tokens = self.tokenize_prompt(prompt) if isinstance(prompt, str) else prompt  # (the engine validates token lists)
        self.requests[request_id] = DynamicInferenceRequest(
            request_id=request_id, prompt=prompt if isinstance(prompt, str) else None,
            prompt_tokens=torch.tensor(tokens, dtype=torch.int64))
        self._send(self.get_next_data_parallel_rank(), [Headers.SUBMIT_REQUEST.value, request_id, list(tokens), sampling_params])

    def _on_control(self, sender: bytes, header: Headers, body: list) -> None:
        if sender not in self.known_clients:
            return
        for replica in self.identities_of_data_parallel_ranks:
            self._send(replica, [header.value])

    def _on_engine_reply(self, sender: bytes, header: Headers, body: list) -> None:
        assert sender in self.identities_of_data_parallel_ranks, f"engine reply from unknown sender {sender!r}"
        request_ids, finished_request_ids, generated_tokens, log_probs = body
        self.postprocess(request_ids, finished_request_ids, generated_tokens, log_probs)

    def postprocess(self, request_ids: List[int], finished_request_ids: List[int], generated_tokens: List[int],
                    log_probs: Optional[list]) -> None:
        """Append the step's tokens (and log probs) to the records; send finished records to their clients."""
        for request_id, token, lp in zip(request_ids, generated_tokens, log_probs if log_probs else repeat(None)):
            request = self.requests[request_id]
            request.generated_tokens.append(token)
            if lp is not None:
                if request.prompt_log_probs is None:  # the first reply of a request carries the prompt's
                    request.prompt_log_probs = lp
                    request.generated_log_probs = []
                else:
                    request.generated_log_probs.extend(lp)
        for request_id in finished_request_ids or ():
            request = self.requests.pop(request_id)
            request.generated_length = len(request.generated_tokens)
            request.generated_text = self.tokenizer.detokenize(request.generated_tokens)
            client = self.request_id_to_client_id.pop(request_id)
            client_request_id = self.request_id_to_client_request_id.pop(request_id)
            self._send(client, [client_request_id, request.serializable()])

    # ------------------------------------------------------------------------------------------ loop
    def handle_one(self, timeout_ms: Optional[int] = None) -> bool:
        """Receive and dispatch one message; False if none arrived within ``timeout_ms``."""
        if timeout_ms is not None and not self.router_socket.poll(timeout_ms):
            return False
        sender, serialized = self.router_socket.recv_multipart()
        self._dispatch(sender, serialized)
        return True

    def _dispatch(self, sender: bytes, serialized: bytes) -> None:
        if not serialized:
            return  # a registration frame outside the registration phase carries nothing to do
        payload = self._msgpack.unpackb(serialized, raw=False)
        header = Headers(payload[0])
        self._handlers[header](sender, header, payload[1:])

    def start(self, poll_ms: int = 50) -> None:
        """The event loop: runs until `stop()` is called (from a handler, a signal or another thread)."""
        self._running = True
        early, self._early = self._early, []
        for sender, serialized in early:
            self._dispatch(sender, serialized)
        while self._running:
            self.handle_one(timeout_ms=poll_ms)
        self.router_socket.close(linger=0)
        self.context.term()

    def stop(self) -> None:
        """End the loop; when it is not running, release the socket right away."""
        if self._running:
            self._running = False
        else:
            self.router_socket.close(linger=0)
            self.context.term()

    @classmethod
    def entrypoint(cls, ready_event, tokenizer, inference_coordinator_port: int, data_parallel_size: int):
        """Body of the coordinator's process: construct (waits for the replicas), signal ``ready_event``, serve."""
        coordinator = cls(tokenizer, inference_coordinator_port, data_parallel_size)
        ready_event.set()
        try:
            coordinator.start()
        except KeyboardInterrupt:
            coordinator.stop()
