"""Message headers of the data-parallel serving protocol (wire constants of the reference's
``megatron/core/inference/headers.py:6-17``: a client or engine of either implementation can talk to a coordinator
of the other).  The first element of every msgpack list on the wire is one of these codes, numbered from 0 in this order."""
from enum import Enum

Headers = Enum(
    "Headers", ["CONNECT", "ACK", "SUBMIT_REQUEST", "ENGINE_REPLY", "PAUSE", "UNPAUSE", "STOP"], start=0, module=__name__)
