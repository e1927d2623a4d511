"""The engine, the controller's step and the context together on the CPU, with a stand-in for the model only.

The stand-in's logits make the next token a function of a request's own last token and position, so every request's
completion can be predicted independently of batching, queueing, pausing and row compaction - which is exactly what the
engine has to get right: requests that wait for room, requests paused when chunks run out, finished rows swapped out,
results delivered per request (reference dynamic_engine.py:363-706, text_generation_controller.py:410-555)."""
from types import SimpleNamespace

import numpy as np
import pytest
import torch

from megatron_mixtera_b200.inference.contexts.dynamic_context import DynamicInferenceContext
from megatron_mixtera_b200.inference.engines.dynamic_engine import DynamicInferenceEngine
from megatron_mixtera_b200.inference.inference_request import DynamicInferenceEventType, Status
from megatron_mixtera_b200.inference.sampling_params import SamplingParams
from megatron_mixtera_b200.inference.text_generation_controllers.text_generation_controller import TextGenerationController

VOCAB, EOD = 97, 5


def next_token(last_token: int, position: int) -> int:
    return (last_token * 7 + position + 3) % VOCAB


def expected_completion(prompt, limit):
    seq, out = list(prompt), []
    while len(out) < limit:
        out.append(next_token(seq[-1], len(seq) - 1))
        seq.append(out[-1])
        if out[-1] == EOD:
            break
    return out


class StandInModel:
    """What the engine and the controller touch of the wrapped model; the 'forward' reads the step the context published."""

    def __init__(self, context):
        self.inference_context = context
        self.model = SimpleNamespace(config=SimpleNamespace(enable_cuda_graph=False, inference_sampling_seed=0))
        self.inference_wrapper_config = SimpleNamespace(padded_vocab_size=VOCAB)
        self.steps = []

    def run_one_forward_step(self, inference_input, recv_buffer_seq_len=None):
        ctx = self.inference_context
        tokens, positions = inference_input["tokens"][0], inference_input["position_ids"][0]
        last = torch.from_numpy(ctx.last_token_indices())
        nxt = (tokens[last] * 7 + positions[last] + 3) % VOCAB
        self.steps.append((ctx.is_decode_only(), len(last), ctx.paused_request_count))
        logits = torch.zeros(1, len(last), VOCAB)
        logits[0, torch.arange(len(last)), nxt] = 1.0
        return logits


class HostController(TextGenerationController):
    def sample_from_logits(self, last_token_logits, sampling_params=None, vocab_size=None, **kwargs):
        return torch.argmax(last_token_logits, dim=-1)  # the CUDA sampling kernels are not what this test is about


def make_engine(buffer_size_gb, max_requests=8, **engine_kw):
    DynamicInferenceContext.TOKEN_ROUNDER, DynamicInferenceContext.REQUEST_ROUNDER = 4, 4
    ctx = DynamicInferenceContext(
        params_dtype=torch.float32, num_layers=2, kv_channels=8, num_attention_heads=2, max_sequence_length=96,
        buffer_size_gb=buffer_size_gb, buffer_guaranteed_fraction=0.1, chunk_size_tokens=16, tensor_model_parallel_size=1,
        max_requests_override=max_requests, max_tokens_override=128, device="cpu", allocate_memory_buffer=False)
    model = StandInModel(ctx)
    engine = DynamicInferenceEngine(HostController(model, tokenizer=None), ctx, termination_id=EOD, random_seed=0, **engine_kw)
    return engine, ctx, model


@pytest.fixture(autouse=True)
def _restore_rounders():
    yield
    DynamicInferenceContext.TOKEN_ROUNDER, DynamicInferenceContext.REQUEST_ROUNDER = 64, 4


def prompts_of(seed, count, lo=3, hi=40):
    rng = np.random.default_rng(seed)
    return [rng.integers(6, VOCAB, size=int(rng.integers(lo, hi))).tolist() for _ in range(count)]


@pytest.mark.parametrize("buffer_size_gb", [0.01, 0.0001])  # roomy; and so small that requests wait and get paused
def test_every_request_completes_with_its_own_tokens(buffer_size_gb):
    engine, ctx, model = make_engine(buffer_size_gb, track_paused_request_events=True)
    prompts = prompts_of(0, 14)
    finished = engine.generate(prompts, SamplingParams(top_k=1, num_tokens_to_generate=24))
    assert sorted(r.request_id for r in finished) == list(range(14)) and engine.finished_request_count == 14
    assert not engine.has_unfinished_requests() and ctx.total_request_count == 0
    assert ctx.chunk_allocator.chunk_count_avail == ctx.chunk_allocator.chunk_count_total - 1  # all chunks back (one is the dummy)
    for r in finished:
        want = expected_completion(prompts[r.request_id], 24)
        assert list(r.generated_tokens) == want, (r.request_id, r.generated_tokens, want)
        assert r.status == Status.COMPLETED and r.generated_length == len(want)
        kinds = [e.type for e in r.events]
        assert kinds[-1] == DynamicInferenceEventType.FINISH and DynamicInferenceEventType.ADD in kinds
        assert kinds.index(DynamicInferenceEventType.ADD) == max(i for i, k in enumerate(kinds) if k == DynamicInferenceEventType.ADD)
    waited = [r for r in finished if r.events[0].type == DynamicInferenceEventType.ERROR_TRANSIENT]
    paused = [r for r in finished if any(e.type == DynamicInferenceEventType.PAUSE for e in r.events)]
    if buffer_size_gb < 0.001:
        assert waited and any(p for _, _, p in model.steps), "the small pool should have made requests wait and pause"
        assert paused
    else:
        assert 14 - 8 <= len(waited) < 14  # the request limit (8 rows) or the token limit kept them out at first


def test_requests_arriving_between_steps_and_futures():
    engine, ctx, model = make_engine(0.01)
    prompts = prompts_of(1, 5)
    sp = SamplingParams(top_k=1, num_tokens_to_generate=10)
    futures = {i: engine.add_request(i, prompts[i], 10) for i in (0, 1)}
    done = {}
    for step in range(60):
        if step == 2:
            futures[2] = engine.add_request(2, torch.tensor(prompts[2]), 10)   # a tensor prompt, mid-flight
        if step == 4:
            futures[3] = engine.add_request(3, prompts[3], 10)
            futures[4] = engine.add_request(4, prompts[4], 10)
        result = engine.step_modern(sp)
        for r in result["finished_requests"]:
            done[r.request_id] = r
        if step >= 4 and not engine.has_unfinished_requests():
            break
    assert sorted(done) == [0, 1, 2, 3, 4]
    for i, r in done.items():
        assert list(r.generated_tokens) == expected_completion(prompts[i], 10)
        assert futures[i].done() and futures[i].result() is r
        assert len(r.tpot) == len(r.generated_tokens)
    assert any(not decode for decode, _, _ in model.steps[1:]), "a later arrival makes a mixed (non-decode) step"
    a, f, t = engine.step_legacy(sp) if engine.has_unfinished_requests() else ([], [], 0.0)
    assert (a, f) == ([], [])


def test_a_prompt_that_can_never_fit_fails_and_the_rest_carries_on():
    engine, ctx, model = make_engine(0.01)
    sp = SamplingParams(top_k=1, num_tokens_to_generate=8)
    engine.add_request(0, list(range(6, 30)), 8)
    engine.add_request(1, list(range(6, 96)) + list(range(6, 40)), 8)  # longer than max_sequence_length allows
    finished = []
    while engine.has_unfinished_requests():
        finished += engine.step_modern(sp)["finished_requests"]
    by_id = {r.request_id: r for r in finished}
    assert by_id[1].status == Status.FAILED and by_id[1].events[-1].type == DynamicInferenceEventType.FAIL
    assert by_id[0].status == Status.COMPLETED and list(by_id[0].generated_tokens) == expected_completion(list(range(6, 30)), 8)


def test_a_queued_prompt_that_does_not_fit_an_empty_context_fails_instead_of_waiting_for_ever():
    engine, ctx, model = make_engine(0.01)
    too_long = list(range(6, 96)) + list(range(6, 96))  # 180 tokens: more than the step's token limit (transient by class)
    finished = engine.generate([too_long], SamplingParams(top_k=1, num_tokens_to_generate=4))
    assert [r.status for r in finished] == [Status.FAILED] and model.steps == []
    assert [e.type for e in finished[0].events][-1] == DynamicInferenceEventType.FAIL
    assert not engine.has_unfinished_requests()


@pytest.mark.parametrize("buffer_size_gb", [0.01, 0.0001])
def test_enqueueing_the_next_forward_early_changes_no_token_and_repeats_few_forwards(buffer_size_gb):
    """`overlap_host_and_device`: the controller runs the next decode forward before the engine post-processes the step.
    The forward is repeated only when the set of requests changed in between (an arrival, an admission from the queue);
    a queue whose head still does not fit must not invalidate it."""
    prompts = prompts_of(2, 14)
    sp = SamplingParams(top_k=1, num_tokens_to_generate=24)
    plain, _, plain_model = make_engine(buffer_size_gb)
    want = {r.request_id: list(r.generated_tokens) for r in plain.generate(prompts, sp)}
    engine, ctx, model = make_engine(buffer_size_gb, overlap_host_and_device=True)
    for i, p in enumerate(prompts):
        engine.add_request(i, p, 24)
    got, steps, admissions = {}, 0, 0
    while engine.has_unfinished_requests():
        waiting_before = len(engine.waiting_request_ids)
        for r in engine.step_modern(sp)["finished_requests"]:
            got[r.request_id] = list(r.generated_tokens)
        admissions += int(len(engine.waiting_request_ids) < waiting_before)
        steps += 1
    assert got == want and want == {i: expected_completion(p, 24) for i, p in enumerate(prompts)}
    assert steps == len(plain_model.steps)
    repeated = len(model.steps) - steps
    assert 0 <= repeated <= admissions + 1, (repeated, admissions, steps)


def test_engine_serves_a_client_through_the_coordinator_on_the_cpu():
    """The engine's serving loop (registration, message intake, ENGINE_REPLY after every step, PAUSE / STOP) with the real
    context and controller step around the stand-in model; a prompt the replica can never hold comes back empty."""
    import asyncio
    import threading

    pytest.importorskip("zmq")
    pytest.importorskip("msgpack")
    from megatron_mixtera_b200.inference.data_parallel_inference_coordinator import DataParallelInferenceCoordinator
    from megatron_mixtera_b200.inference.inference_client import InferenceClient
    from serving_helpers import CharTokenizer, free_port

    engine, ctx, model = make_engine(0.01)
    port, box = free_port(), {}

    def serve():
        box["c"] = DataParallelInferenceCoordinator(CharTokenizer(VOCAB), port, 1, registration_timeout_s=60, bind_address="127.0.0.1")
        box["c"].start(poll_ms=10)

    threading.Thread(target=serve, daemon=True).start()
    prompts = prompts_of(3, 6) + ["hello"]
    sp = SamplingParams(top_k=1, num_tokens_to_generate=12)

    async def scenario():
        await engine.start_listening_to_data_parallel_coordinator(sp, port, launch_inference_coordinator=False)
        client = InferenceClient(port)
        await client.start()
        futures = [client.add_request(p, sp) for p in prompts]
        hopeless = client.add_request(list(range(6, 96)) + list(range(6, 96)), sp)
        records = await asyncio.wait_for(asyncio.gather(*futures), timeout=60)
        empty = await asyncio.wait_for(hopeless, timeout=60)
        client.pause_engines()
        await asyncio.sleep(0.2)
        assert engine.paused
        client.stop_engines()
        await asyncio.wait_for(engine.engine_loop_task, timeout=30)
        client.stop()
        await asyncio.sleep(0)  # lets the cancelled listener task finish before the loop goes away
        return records, empty

    try:
        records, empty = asyncio.new_event_loop().run_until_complete(scenario())
    finally:
        if "c" in box:
            box["c"].stop()
    assert engine.stopped and not engine.requests
    tokenised = prompts[:-1] + [CharTokenizer(VOCAB).tokenize("hello")]
    for prompt, record in zip(tokenised, records):
        assert list(record.generated_tokens) == expected_completion(prompt, 12)
    assert records[-1].prompt == "hello" and list(empty.generated_tokens) == [] and empty.generated_length == 0
