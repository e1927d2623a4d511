"""Message headers of the data-parallel serving protocol (wire constants of the reference's
``megatron/core/inference/headers.py:6-17``: a client or engine of either implementation can talk to a coordinator
of the other)."""
from enum import Enum


class Headers(Enum):
    CONNECT = 0
    ACK = 1
    SUBMIT_REQUEST = 2
    ENGINE_REPLY = 3
    PAUSE = 4
    UNPAUSE = 5
    STOP = 6
