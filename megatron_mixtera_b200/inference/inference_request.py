"""Request records kept by the engine (fields follow the reference's
``megatron/core/inference/inference_request.py:15-193``)."""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from enum import Enum, auto
from typing import Any, List, Optional

import torch

from .sampling_params import SamplingParams


class Status(Enum):
    WAITING_IN_QUEUE = 1
    ACTIVE_AND_GENERATING_TOKENS = 2
    ACTIVE_BUT_NOT_GENERATING_TOKENS = 3
    COMPLETED = 4
    FAILED = 5


class DynamicInferenceEventType(Enum):
    ADD = auto()
    PAUSE = auto()
    FINISH = auto()
    FAIL = auto()
    ERROR_TRANSIENT = auto()
    ERROR_NONTRANSIENT = auto()


@dataclass(kw_only=True)
class DynamicInferenceEvent:
    """One lifecycle event; error events carry the exception as payload."""

    type: DynamicInferenceEventType
    payload: Optional[Any] = None
    timestamp: float = field(default_factory=time.time)

    def __post_init__(self):
        is_error = self.type in (DynamicInferenceEventType.ERROR_TRANSIENT, DynamicInferenceEventType.ERROR_NONTRANSIENT)
        assert (self.payload is not None) == is_error

    def __str__(self):
        payload = "" if self.payload is None else f", {type(self.payload).__name__}"
        return f"[{self.timestamp:.3f}] {self.type.name}{payload}"


@dataclass(kw_only=True)
class DynamicInferenceRequest:
    """A request of the dynamic engine: integer id, tokenised prompt, generated tokens, event log."""

    request_id: int
    prompt_tokens: torch.Tensor
    sampling_params: Optional[SamplingParams] = None
    prompt: Optional[str] = None
    status: Optional[Status] = None
    generated_text: Optional[str] = None
    generated_tokens: List[int] = field(default_factory=list)
    generated_length: Optional[int] = None
    prompt_log_probs: Optional[List[float]] = None
    generated_log_probs: Optional[List[float]] = None
    tpot: Optional[List[float]] = None
    events: List[DynamicInferenceEvent] = field(default_factory=list)
    latency: Optional[float] = None  # set by the client: submission to completion
    # Fields of the reference's record that only its static-batching engine fills (reference :33-51); they are kept so that
    # a serialised record has the reference's keys and either side's client can rebuild the other side's record.
    inference_parameters: Optional[SamplingParams] = None  # the reference's deprecated name of `sampling_params`
    arrival_time: Optional[float] = None
    encoder_prompt: Optional[str] = None
    segments: Optional[List[str]] = None
    generated_segments: Optional[List[str]] = None
    generated_sequence_lengths: Optional[List[int]] = None
    prompt_top_n_logprobs: Optional[list] = None
    generated_top_n_logprobs: Optional[list] = None

    def add_event(self, type: DynamicInferenceEventType, payload: Optional[Any] = None) -> None:
        self.events.append(DynamicInferenceEvent(type=type, payload=payload))

    def add_event_add(self):
        self.add_event(DynamicInferenceEventType.ADD)

    def add_event_pause(self):
        self.add_event(DynamicInferenceEventType.PAUSE)

    def add_event_finish(self):
        self.add_event(DynamicInferenceEventType.FINISH)

    def add_event_fail(self):
        self.add_event(DynamicInferenceEventType.FAIL)

    def add_event_error_transient(self, error: Exception):
        self.add_event(DynamicInferenceEventType.ERROR_TRANSIENT, error)

    def add_event_error_nontransient(self, error: Exception):
        self.add_event(DynamicInferenceEventType.ERROR_NONTRANSIENT, error)

    def failed(self) -> bool:
        return self.status == Status.FAILED

    def serializable(self) -> dict:
        """Plain-data form for the serving protocol (msgpack): tensors as lists, enums by name, events as strings
        (reference ``inference_request.py:58-77``)."""
        out = {}
        for key, value in self.__dict__.items():
            if isinstance(value, torch.Tensor):
                value = value.tolist()
            elif isinstance(value, Enum):
                value = value.name
            elif isinstance(value, SamplingParams):
                value = value.serializable()
            elif key == "events":
                value = [str(e) for e in value]
            out[key] = value
        return out

    @classmethod
    def deserialize(cls, data: dict) -> "DynamicInferenceRequest":
        """Inverse of `serializable` as far as a client needs it: events stay strings, extra keys become attributes."""
        data = dict(data)
        tokens = data.pop("prompt_tokens", None)
        status = data.pop("status", None)
        params = data.pop("sampling_params", None)
        events = data.pop("events", None) or []
        known = {k: data.pop(k) for k in list(data) if k in cls.__dataclass_fields__}
        obj = cls(prompt_tokens=torch.tensor(tokens if tokens is not None else [], dtype=torch.int64),
                  status=Status[status] if isinstance(status, str) else status,
                  sampling_params=SamplingParams.deserialize(params) if isinstance(params, dict) else params, **known)
        obj.events = events
        for key, value in data.items():
            setattr(obj, key, value)
        return obj
