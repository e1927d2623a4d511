"""Wire compatibility of the serving plumbing with the reference's: this package's client against the REFERENCE's
coordinator, the reference's client against this package's coordinator (engine replicas are protocol stand-ins), and this
package's engine - its own serving loop around a stand-in model - as the replica of the reference's coordinator and client.
Runs in a child process that imports the reference checkout; skipped where it is absent (it cannot travel)."""
import os
import subprocess
import sys

import pytest

from conftest import ROOT

REFERENCE = os.environ.get("MEGATRON_REFERENCE", os.path.join(os.path.dirname(ROOT), "reference"))  # a sibling checkout

CHILD = r'''
import asyncio, json, os, sys, threading, time
ref, root = sys.argv[1], sys.argv[2]
sys.path.insert(0, ref); sys.path.insert(0, root); sys.path.insert(0, os.path.join(root, "tests"))
os.environ.setdefault("TORCHDYNAMO_DISABLE", "1")
import torch
torch.cuda.current_device = lambda: torch.device("cpu")
from megatron.core.inference.data_parallel_inference_coordinator import DataParallelInferenceCoordinator as RefCoordinator
from megatron.core.inference.inference_client import InferenceClient as RefClient
from megatron.core.inference.sampling_params import SamplingParams as RefSamplingParams
from megatron_mixtera_b200.inference.data_parallel_inference_coordinator import DataParallelInferenceCoordinator
from megatron_mixtera_b200.inference.inference_client import InferenceClient
from megatron_mixtera_b200.inference.sampling_params import SamplingParams
from megatron.core.inference.headers import Headers as RefHeaders
from megatron_mixtera_b200.inference.headers import Headers
from serving_helpers import CharTokenizer, free_port
from test_dp_coordinator import FakeReplica

assert {h.name: h.value for h in RefHeaders} == {h.name: h.value for h in Headers}

KEEP = []


def run(coordinator_cls, client_cls, params):
    port = free_port()
    replica = FakeReplica(port, 0)
    threading.Thread(target=lambda: coordinator_cls(CharTokenizer(), port, 1).start(), daemon=True).start()
    replica.start()
    time.sleep(1.5)  # (the reference's coordinator must have its replica before a client speaks)
    async def scenario():
        client = client_cls(port)
        KEEP.append(client)  # (a collected client would terminate its ZMQ context inside the loop and block on it)
        await client.start()
        futures = [client.add_request("ab", params), client.add_request([4, 5, 6], params)]
        records = await asyncio.wait_for(asyncio.gather(*futures), timeout=30)
        client.pause_engines()
        await asyncio.sleep(0.3)
        return [(r.request_id, list(r.generated_tokens), r.generated_text, r.generated_length) for r in records]
    out = asyncio.new_event_loop().run_until_complete(scenario())
    return {"records": out, "received": replica.received, "signals": [s.name for s in replica.signals]}

def run_engine(coordinator_cls, client_cls, params):
    """This package's ENGINE (its serving loop, context and controller step around the stand-in model of
    test_engine_host) as the replica of the given coordinator, driven by the given client."""
    import test_engine_host as H

    engine, ctx, model = H.make_engine(0.01)
    port = free_port()
    threading.Thread(target=lambda: coordinator_cls(CharTokenizer(H.VOCAB), port, 1).start(), daemon=True).start()
    prompts = H.prompts_of(4, 5)
    async def scenario():
        await engine.start_listening_to_data_parallel_coordinator(
            SamplingParams(top_k=1, num_tokens_to_generate=8), port, launch_inference_coordinator=False)
        await asyncio.sleep(1.5)  # (the reference's coordinator must have its replica before a client speaks)
        client = client_cls(port)
        KEEP.append(client)
        await client.start()
        records = await asyncio.wait_for(asyncio.gather(*[client.add_request(p, params) for p in prompts]), timeout=60)
        client.stop_engines()
        await asyncio.wait_for(engine.engine_loop_task, timeout=30)
        return [[int(t) for t in r.generated_tokens] for r in records]
    got = asyncio.new_event_loop().run_until_complete(scenario())
    return {"equal": got == [H.expected_completion(p, 8) for p in prompts], "n": len(got), "stopped": engine.stopped}


result = {
    "our_engine_ref_coordinator_ref_client": run_engine(RefCoordinator, RefClient, RefSamplingParams(top_k=1, num_tokens_to_generate=8)),
    "our_client_ref_coordinator": run(RefCoordinator, InferenceClient, SamplingParams(top_k=1, num_tokens_to_generate=2)),
    "ref_client_our_coordinator": run(DataParallelInferenceCoordinator, RefClient, RefSamplingParams(top_k=1, num_tokens_to_generate=2)),
}
print("RESULT " + json.dumps(result), flush=True)
os._exit(0)
'''


@pytest.mark.skipif(not os.path.isdir(os.path.join(REFERENCE, "megatron", "core")), reason="reference checkout absent")
def test_client_and_coordinator_interoperate_with_the_reference():
    import json

    proc = subprocess.run([sys.executable, "-c", CHILD, REFERENCE, ROOT], capture_output=True, text=True, timeout=240)
    lines = [l for l in proc.stdout.splitlines() if l.startswith("RESULT ")]
    assert lines, proc.stdout[-2000:] + proc.stderr[-3000:]
    out = json.loads(lines[-1][len("RESULT "):])
    assert out["our_engine_ref_coordinator_ref_client"] == {"equal": True, "n": 5, "stopped": True}, out
    for case in ("our_client_ref_coordinator", "ref_client_our_coordinator"):
        got = out[case]
        assert [r[0] for r in got["records"]] == [0, 1], (case, got)
        assert [r[1] for r in got["records"]] == [[0, 1], [100, 101]], (case, got)          # the stand-in's tokens
        assert [r[2] for r in got["records"]] == ["0,1", "100,101"] and [r[3] for r in got["records"]] == [2, 2]
        assert [tuple(t) for _, t in got["received"]] == [(97, 98), (4, 5, 6)], (case, got)  # text tokenised, ids passed
        assert got["signals"] == ["PAUSE"], (case, got)
