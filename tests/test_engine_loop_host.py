"""`DynamicInferenceEngine.run_engine` on the CPU: the loop sleeps while there is no work, `add_request` inside the running
loop wakes it, cancelling the task ends it (reference dynamic_engine.py:358-391, 803-813).  The context and the model step
are stand-ins; queueing, the wake-up and the loop are the engine's own code."""
import asyncio
from collections import deque

import torch

from megatron_mixtera_b200.inference.engines.dynamic_engine import DynamicInferenceEngine


class FakeContext:
    def __init__(self):
        self.remaining = {}

    def add_request(self, request_id, tokens, num_tokens_to_generate=None):
        self.remaining[request_id] = num_tokens_to_generate

    def get_active_request_count(self):
        return len(self.remaining)

    def has_unfinished_requests(self):
        return bool(self.remaining)


class LoopOnlyEngine(DynamicInferenceEngine):
    def __init__(self, loop):
        self.context = FakeContext()
        self.controller = None
        self.requests, self.request_completion_futures = {}, {}
        self.waiting_request_ids, self.failed_request_ids = deque(), []
        self.paused = self.stopped = False
        self._loop = loop
        self._cond = asyncio.Condition()
        self.steps = 0

    async def async_step(self, sampling_params, *, verbose=False, post_process_requests_locally=True):
        self.steps += 1
        for request_id in list(self.context.remaining):
            self.context.remaining[request_id] -= 1
            if self.context.remaining[request_id] == 0:
                del self.context.remaining[request_id]
                self.request_completion_futures.pop(request_id).set_result(self.requests.pop(request_id))
        await asyncio.sleep(0)


def test_run_engine_sleeps_until_a_request_arrives_and_ends_when_cancelled():
    loop = asyncio.new_event_loop()

    async def scenario():
        engine = LoopOnlyEngine(loop)
        task = asyncio.create_task(engine.run_engine(None))
        await asyncio.sleep(0.05)
        assert engine.steps == 0 and not task.done()           # nothing to do: no step, no spinning
        record = await asyncio.wait_for(engine.add_request(7, [1, 2, 3], 2), timeout=5)
        assert record.request_id == 7 and engine.steps == 2     # woken by the request, stepped until it was done
        await asyncio.sleep(0.05)
        assert engine.steps == 2 and not task.done()           # asleep again
        second = engine.add_request(8, torch.tensor([4, 5]), 1)
        await asyncio.wait_for(second, timeout=5)
        assert engine.steps == 3
        task.cancel()
        await asyncio.wait_for(task, timeout=5)                 # the loop swallows the cancellation and returns
        return True

    assert loop.run_until_complete(scenario())
    loop.close()
