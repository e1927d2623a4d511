"""Serving plumbing on the CPU: the data-parallel coordinator, the client and the engine side of their protocol.

Reference: megatron/core/inference/data_parallel_inference_coordinator.py, inference_client.py, headers.py and the
coordinator-facing half of dynamic_engine.py (:229-356, 708-872).  The engine replicas here are stand-ins that speak the
engine's side of the protocol (register with an empty frame under the identity ``tp-coord-<i>``, take SUBMIT_REQUEST,
answer ENGINE_REPLY after every "step"); the GPU suite runs the real engine under the same coordinator."""
import asyncio
import socket
import threading
import time

import pytest

msgpack = pytest.importorskip("msgpack")
zmq = pytest.importorskip("zmq")

from megatron_mixtera_b200.inference.data_parallel_inference_coordinator import DataParallelInferenceCoordinator  # noqa: E402
from megatron_mixtera_b200.inference.headers import Headers  # noqa: E402
from megatron_mixtera_b200.inference.inference_client import InferenceClient  # noqa: E402
from megatron_mixtera_b200.inference.sampling_params import SamplingParams  # noqa: E402


class CharTokenizer:
    bos = 1

    def tokenize(self, text):
        return [ord(c) for c in text]

    def detokenize(self, tokens):
        return ",".join(str(t) for t in tokens)


def free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


class FakeReplica(threading.Thread):
    """Engine side of the protocol: every poll round is a "step" that emits one token per active request."""

    def __init__(self, port, index):
        super().__init__(daemon=True)
        self.port, self.index = port, index
        self.received, self.signals = [], []
        self.halt = threading.Event()

    def run(self):
        ctx = zmq.Context()
        sock = ctx.socket(zmq.DEALER)
        sock.setsockopt(zmq.IDENTITY, f"tp-coord-{self.index}".encode())
        sock.connect(f"tcp://127.0.0.1:{self.port}")
        sock.send(b"")
        active = {}  # request id -> [tokens still to emit, step]
        while not self.halt.is_set():
            while sock.poll(5):
                data = msgpack.unpackb(sock.recv(), raw=False)
                header = Headers(data[0])
                if header == Headers.SUBMIT_REQUEST:
                    rid, tokens, params = data[1:]
                    self.received.append((rid, tokens))
                    active[rid] = [SamplingParams.deserialize(params).num_tokens_to_generate, 0]
                else:
                    self.signals.append(header)
            if active and Headers.PAUSE not in self.signals[-1:]:
                ids = sorted(active)
                toks = [1000 * self.index + 100 * rid + active[rid][1] for rid in ids]
                for rid in ids:
                    active[rid][0] -= 1
                    active[rid][1] += 1
                done = [rid for rid in ids if active[rid][0] == 0]
                for rid in done:
                    del active[rid]
                sock.send(msgpack.packb([Headers.ENGINE_REPLY.value, ids, done, toks, None], use_bin_type=True))
        sock.close(linger=0)
        ctx.term()


def test_coordinator_routes_requests_round_robin_and_results_to_their_clients():
    port = free_port()
    replicas = [FakeReplica(port, i) for i in range(2)]
    box = {}

    def serve():
        box["c"] = DataParallelInferenceCoordinator(CharTokenizer(), port, 2, registration_timeout_s=20, bind_address="127.0.0.1")
        box["c"].start(poll_ms=10)

    server = threading.Thread(target=serve, daemon=True)
    server.start()
    for r in replicas:
        r.start()

    async def scenario():
        a, b = InferenceClient(port), InferenceClient(port)
        await a.start()
        await b.start()
        sp = SamplingParams(top_k=1, num_tokens_to_generate=3)
        futures = [a.add_request("hi", sp), b.add_request([7, 8, 9], sp), a.add_request("yo!", sp), b.add_request([5], sp)]
        done = await asyncio.wait_for(asyncio.gather(*futures), timeout=20)
        a.pause_engines()
        await asyncio.sleep(0.2)
        a.unpause_engines()
        await asyncio.sleep(0.2)
        b.stop_engines()
        await asyncio.sleep(0.2)
        a.stop()
        b.stop()
        await asyncio.sleep(0)  # lets the cancelled listener task finish before the loop goes away
        return done

    done = asyncio.new_event_loop().run_until_complete(scenario())
    coordinator = box["c"]
    # server-side ids follow arrival order at the router; replicas take them in turn (registration order)
    per_replica = {i: sorted(rid for rid, _ in r.received) for i, r in enumerate(replicas)}
    assert sorted(per_replica[0] + per_replica[1]) == [0, 1, 2, 3]
    assert all(abs(len(v) - 2) == 0 for v in per_replica.values())
    order = [rid for rid in range(4)]
    owner = {rid: next(i for i, v in per_replica.items() if rid in v) for rid in order}
    assert [owner[r] for r in order] in ([0, 1, 0, 1], [1, 0, 1, 0])
    # text prompts were tokenised by the coordinator, token lists were passed through
    all_received = dict(replicas[0].received + replicas[1].received)
    assert sorted(map(tuple, all_received.values())) == sorted([(104, 105), (7, 8, 9), (121, 111, 33), (5,)])
    # every client got its own requests back, complete and detokenised
    for record, prompt_len in zip(done, (2, 3, 3, 1)):
        assert record.generated_length == 3 and len(record.generated_tokens) == 3
        assert record.generated_text == ",".join(str(t) for t in record.generated_tokens)
        assert len(record.prompt_tokens) == prompt_len and record.latency > 0
        rid = record.request_id
        assert record.generated_tokens == [1000 * owner[rid] + 100 * rid + s for s in range(3)]
    assert done[0].prompt == "hi" and done[2].prompt == "yo!" and done[1].prompt is None
    # control signals reach every replica, in order
    for r in replicas:
        assert r.signals == [Headers.PAUSE, Headers.UNPAUSE, Headers.STOP]
    assert not coordinator.requests and not coordinator.request_id_to_client_id
    for r in replicas:
        r.halt.set()
    coordinator.stop()
    server.join(timeout=5)
    assert not server.is_alive()


def test_unknown_clients_and_duplicate_connects_are_ignored():
    port = free_port()
    replica = FakeReplica(port, 0)
    box = {}

    def serve():
        box["c"] = DataParallelInferenceCoordinator(CharTokenizer(), port, 1, registration_timeout_s=20, bind_address="127.0.0.1")
        box["c"].start(poll_ms=10)

    server = threading.Thread(target=serve, daemon=True)
    server.start()
    replica.start()
    ctx = zmq.Context()
    stranger = ctx.socket(zmq.DEALER)
    stranger.connect(f"tcp://127.0.0.1:{port}")
    sp = SamplingParams(num_tokens_to_generate=1).serializable()
    stranger.send(msgpack.packb([Headers.SUBMIT_REQUEST.value, 0, [1, 2], sp], use_bin_type=True))  # never connected
    stranger.send(msgpack.packb([Headers.STOP.value], use_bin_type=True))
    time.sleep(0.3)
    assert replica.received == [] and replica.signals == []
    stranger.send(msgpack.packb([Headers.CONNECT.value], use_bin_type=True))
    assert stranger.poll(5000) and Headers(msgpack.unpackb(stranger.recv(), raw=False)[0]) == Headers.ACK
    stranger.send(msgpack.packb([Headers.CONNECT.value], use_bin_type=True))  # duplicate: no second ACK
    assert not stranger.poll(300)
    stranger.send(msgpack.packb([Headers.SUBMIT_REQUEST.value, 42, [1, 2], sp], use_bin_type=True))
    assert stranger.poll(5000)
    client_request_id, record = msgpack.unpackb(stranger.recv(), raw=False)
    assert client_request_id == 42 and record["generated_length"] == 1 and record["prompt_tokens"] == [1, 2]
    stranger.close(linger=0)
    ctx.term()
    replica.halt.set()
    box["c"].stop()
    server.join(timeout=5)


def test_registration_times_out_instead_of_waiting_for_ever():
    with pytest.raises(TimeoutError):
        DataParallelInferenceCoordinator(CharTokenizer(), free_port(), 1, registration_timeout_s=0.2, bind_address="127.0.0.1")


def test_messages_fan_out_inside_a_tensor_parallel_group(tmp_path):
    """One replica of two tensor-parallel ranks (gloo processes running the engine's own serving loop over a stand-in
    model step): only the group's first rank talks to the coordinator; the other rank must see the same requests before
    the same steps, and STOP must reach both (reference dynamic_engine.py:708-789)."""
    import json
    import os
    import signal
    import subprocess
    import sys

    from conftest import ROOT

    port, out = free_port(), str(tmp_path / "ranks.json")
    box = {}

    def serve():
        box["c"] = DataParallelInferenceCoordinator(CharTokenizer(), port, 1, registration_timeout_s=180, bind_address="127.0.0.1")
        box["c"].start(poll_ms=10)

    threading.Thread(target=serve, daemon=True).start()
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", TORCHDYNAMO_DISABLE="1")
    ranks = subprocess.Popen(
        [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
         "--master-port", str(free_port()), os.path.join(ROOT, "tests", "serving_tp_worker.py"), str(port), out],
        env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, start_new_session=True)

    async def scenario():
        client = InferenceClient(port)
        await client.start()  # acknowledged once the replica has registered
        sp = SamplingParams(top_k=1, num_tokens_to_generate=3)
        first = await asyncio.wait_for(asyncio.gather(client.add_request("ab", sp), client.add_request([4, 5], sp)), timeout=120)
        client.pause_engines()
        client.unpause_engines()
        second = await asyncio.wait_for(client.add_request([9], sp), timeout=60)
        client.stop_engines()
        await asyncio.sleep(0.2)
        client.stop()
        await asyncio.sleep(0)  # lets the cancelled listener task finish before the loop goes away
        return first + [second]

    try:
        deadline = time.time() + 170  # the ranks import torch first; the coordinator exists once they have registered
        while "c" not in box and ranks.poll() is None and time.time() < deadline:
            time.sleep(0.1)
        assert "c" in box, "the replica did not register"
        done = asyncio.new_event_loop().run_until_complete(scenario())
        log, _ = ranks.communicate(timeout=90)
    finally:
        if ranks.poll() is None:
            os.killpg(ranks.pid, signal.SIGKILL)  # the launcher and its ranks: the process group this test started
        if "c" in box:
            box["c"].stop()
    assert ranks.returncode == 0, log[-3000:]
    assert [list(r.generated_tokens) for r in done] == [[0, 1, 2], [100, 101, 102], [200, 201, 202]]
    a, b = json.load(open(out))
    assert (a["rank"], b["rank"]) == (0, 1)
    assert [x[1:] for x in a["added"]] == [[0, [97, 98]], [1, [4, 5]], [2, [9]]]
    assert a["added"] == b["added"] and a["steps"] == b["steps"]  # same requests before the same steps on both ranks
