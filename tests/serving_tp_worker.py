"""Child process of the serving fan-out test (launched by torchrun, gloo, CPU): the ranks form ONE tensor-parallel group,
i.e. one engine replica.  The serving loop, its sockets and the fan-out of the coordinator's messages inside the group are
the engine's own code; only the model step is a stand-in that emits ``100 * request id + position`` per active request.
Every rank records at which step it saw which request; rank 0 writes all ranks' records to the output file."""
import asyncio
import json
import os
import sys
from collections import deque

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main(port: int, out_path: str) -> None:
    from megatron_mixtera_b200 import parallel_state
    from megatron_mixtera_b200.inference.engines.dynamic_engine import DynamicInferenceEngine
    from megatron_mixtera_b200.inference.sampling_params import SamplingParams

    dist.init_process_group("gloo")
    world, rank = dist.get_world_size(), dist.get_rank()
    parallel_state.initialize_model_parallel(world)
    assert parallel_state.get_data_parallel_world_size() == 1 and parallel_state.get_data_parallel_rank() == 0

    class Context:
        def __init__(self, engine):
            self.engine = engine

        def get_active_request_count(self):
            return len(self.engine.active)

    class StubEngine(DynamicInferenceEngine):
        def __init__(self):
            self.paused = self.stopped = False
            self.waiting_request_ids, self.failed_request_ids = deque(), []
            self.requests, self.request_completion_futures = {}, {}
            self.context = Context(self)
            self.active = {}     # request id -> [tokens still to emit, position]
            self.steps = 0
            self.added = []      # [step count when the request arrived, request id, prompt tokens]
            self.pauses = 0

        def add_request(self, request_id, prompt, num_tokens_to_generate=None):
            self.active[request_id] = [num_tokens_to_generate, 0]
            self.added.append([self.steps, request_id, list(prompt)])

        def schedule_waiting_requests(self):
            pass

        async def async_step(self, sampling_params, *, verbose=False, post_process_requests_locally=True):
            assert not post_process_requests_locally  # the coordinator keeps the records
            ids = sorted(self.active)
            tokens = [100 * i + self.active[i][1] for i in ids]
            for i in ids:
                self.active[i][0] -= 1
                self.active[i][1] += 1
            done = [i for i in ids if self.active[i][0] == 0]
            for i in done:
                del self.active[i]
            self.steps += 1
            return torch.tensor(ids), torch.tensor(done, dtype=torch.int64), torch.tensor(tokens), None

    async def serve():
        engine = StubEngine()
        await engine.start_listening_to_data_parallel_coordinator(
            SamplingParams(top_k=1), port, launch_inference_coordinator=False)
        await engine.engine_loop_task  # ends with the STOP message
        return engine

    engine = asyncio.new_event_loop().run_until_complete(serve())
    assert engine.stopped and engine.zmq_sockets == []
    records = [None] * world
    dist.all_gather_object(records, {"rank": rank, "added": engine.added, "steps": engine.steps})
    if rank == 0:
        with open(out_path, "w") as f:
            json.dump(records, f)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main(int(sys.argv[1]), sys.argv[2])
