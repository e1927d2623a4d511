"""The real engine as a replica under the data-parallel coordinator (one GPU, one replica): requests submitted through
`InferenceClient` come back with the tokens the engine generates for the same prompts when driven directly."""
import asyncio
import json
import os

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
pytest.importorskip("zmq")
pytest.importorskip("msgpack")

from conftest import ROOT  # noqa: E402
from serving_helpers import CharTokenizer, free_port  # noqa: E402

GOLDEN = os.path.join(ROOT, "tests", "golden")


def _stack():
    from megatron_mixtera_b200.inference.engines.dynamic_engine import DynamicInferenceEngine
    from test_model_gpu import build_cuda_stack

    z = np.load(os.path.join(GOLDEN, "llama_tiny_bf16.npz"))
    meta = json.loads(str(z["meta"]))
    model, ctx, wrapper, Controller = build_cuda_stack(meta, enable_cuda_graph=True)
    ctl = Controller(wrapper, CharTokenizer(meta["vocab_size"]))
    return DynamicInferenceEngine(ctl, ctx, termination_id=-1, random_seed=0), meta


def test_engine_serves_requests_of_a_client_through_the_coordinator():
    from megatron_mixtera_b200 import ops
    from megatron_mixtera_b200.inference.inference_client import InferenceClient
    from megatron_mixtera_b200.inference.sampling_params import SamplingParams
    from megatron_mixtera_b200.inference.text_generation_controllers.text_generation_controller import get_asyncio_loop

    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(0, 1024, (n,), generator=g, dtype=torch.int64).tolist() for n in (40, 7, 19)] + ["hello there"]
    sp = SamplingParams(top_k=1, num_tokens_to_generate=6)

    engine, _ = _stack()
    direct = {i: r.generated_tokens for i, r in enumerate(sorted(engine.generate(prompts, sp), key=lambda r: r.request_id))}

    engine, _ = _stack()
    port = free_port()

    async def scenario():
        await engine.start_listening_to_data_parallel_coordinator(sp, port, launch_inference_coordinator=True)
        client = InferenceClient(port)
        await client.start()
        futures = [client.add_request(p, sp) for p in prompts]
        records = await asyncio.wait_for(asyncio.gather(*futures), timeout=120)
        client.pause_engines()
        await asyncio.sleep(0.2)
        assert engine.paused
        client.unpause_engines()
        await asyncio.sleep(0.2)
        assert not engine.paused
        client.stop_engines()
        await asyncio.wait_for(engine.engine_loop_task, timeout=30)
        client.stop()
        return records

    records = get_asyncio_loop().run_until_complete(scenario())
    assert engine.stopped
    for i, record in enumerate(records):
        assert record.generated_tokens == direct[i], (i, record.generated_tokens, direct[i])
        assert record.generated_length == 6
        assert record.generated_text == ",".join(str(t) for t in direct[i])
    assert records[3].prompt == "hello there" and records[0].prompt is None
    assert ops.device_status() == 0
