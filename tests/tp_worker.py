"""Child process of the tensor-parallel tests (launched by torchrun, one rank per process).

    mode "host" (gloo, CPU):  checks process-group plumbing, sharding rules and SPMD bookkeeping.
    mode "cuda" (nccl, GPUs): runs the tiny Llama through the whole CUDA stack tensor-parallel over the
                              world and writes rank 0's per-step logits/tokens to the output file.
"""
import json
import os
import sys
import types

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))


def host_mode(out_path):
    from megatron_mixtera_b200 import parallel_state
    from megatron_mixtera_b200.gpt.gpt_model import shard_for_rank
    from megatron_mixtera_b200.inference.contexts.dynamic_context import DynamicInferenceContext
    from megatron_mixtera_b200.tensor_parallel.mappings import (
        gather_from_tensor_model_parallel_region, reduce_from_tensor_model_parallel_region)

    dist.init_process_group("gloo")
    world, rank = dist.get_world_size(), dist.get_rank()
    parallel_state.initialize_model_parallel(world)
    assert parallel_state.get_tensor_model_parallel_world_size() == world
    assert parallel_state.get_tensor_model_parallel_rank() == rank
    # collectives (reference tests/unit_tests/tensor_parallel/test_mappings.py: exact equality)
    x = torch.full((3, 4), float(rank + 1))
    assert torch.equal(reduce_from_tensor_model_parallel_region(x.clone()), torch.full((3, 4), float(sum(range(1, world + 1)))))
    g = gather_from_tensor_model_parallel_region(torch.arange(6.0).view(3, 2) + 100 * rank)
    expect = torch.cat([torch.arange(6.0).view(3, 2) + 100 * r for r in range(world)], dim=-1)
    assert torch.equal(g, expect)
    # sharding rules: gathering every rank's shard reconstructs the full tensor
    gen = torch.Generator().manual_seed(0)
    full = {
        "decoder.layers.0.self_attention.linear_qkv.weight": torch.randn(8 * world * 6, 16, generator=gen),
        "decoder.layers.0.self_attention.linear_proj.weight": torch.randn(16, 8 * world, generator=gen),
        "decoder.layers.0.mlp.linear_fc1.weight": torch.randn(2 * 4 * world, 16, generator=gen),
        "decoder.layers.0.mlp.linear_fc2.weight": torch.randn(16, 4 * world, generator=gen),
        "decoder.layers.0.input_layernorm.weight": torch.randn(16, generator=gen),
        "output_layer.weight": torch.randn(10 * world, 16, generator=gen),
    }
    for k, t in full.items():
        shards = [shard_for_rank(k, t, r, world, gated=True) for r in range(world)]
        if k.endswith("layernorm.weight"):
            assert all(torch.equal(s, t) for s in shards)
        elif k.endswith("linear_fc1.weight"):
            gate = torch.cat([torch.chunk(s, 2, 0)[0] for s in shards], 0)
            up = torch.cat([torch.chunk(s, 2, 0)[1] for s in shards], 0)
            assert torch.equal(torch.cat([gate, up], 0), t)
        elif k.endswith(("linear_proj.weight", "linear_fc2.weight")):
            assert torch.equal(torch.cat(shards, 1), t)
        else:
            assert torch.equal(torch.cat(shards, 0), t)
    # SPMD bookkeeping: every rank computes identical state; KV pool holds nkv / tp heads
    DynamicInferenceContext.TOKEN_ROUNDER, DynamicInferenceContext.REQUEST_ROUNDER = 6, 3
    ctx = DynamicInferenceContext(params_dtype=torch.float32, num_layers=2, kv_channels=8, num_attention_heads=2 * world,
                                  max_sequence_length=128, buffer_size_gb=0.001, buffer_guaranteed_fraction=0.1,
                                  chunk_size_tokens=64, max_requests_override=5, device="cpu")
    assert ctx.memory_buffer.shape[4] == 2 and ctx.max_requests % world == 0 and ctx.max_tokens % world == 0
    rng = np.random.RandomState(3)
    for i in range(3):
        ctx.add_request(i, torch.from_numpy(rng.randint(0, 100, size=10 + 30 * i)), 20)
    for step in range(12):
        ctx.initialize_attention_state()
        assert ctx.padded_active_token_count % world == 0
        n = ctx.total_request_count - ctx.paused_request_count
        if n == 0:
            break
        seq = ctx.get_active_sequence_lengths() + 1
        ctx.update_requests(torch.less(seq, ctx.get_max_sequence_lengths()).byte(), torch.from_numpy(rng.randint(0, 100, size=n)))
    state = torch.cat([ctx.request_to_kv_chunk_ids.flatten().long(), ctx._h_tok.flatten()[:64], ctx.chunk_allocator.chunk_bag.long()])
    gathered = [torch.empty_like(state) for _ in range(world)]
    dist.all_gather(gathered, state)
    assert all(torch.equal(gathered[0], t) for t in gathered)
    if rank == 0:
        open(out_path, "w").write("ok")
    dist.barrier()
    dist.destroy_process_group()


def cuda_mode(out_path):
    from megatron_mixtera_b200 import ops, parallel_state
    from megatron_mixtera_b200.inference.sampling_params import SamplingParams
    from test_model_gpu import build_cuda_stack

    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    parallel_state.initialize_model_parallel(world)
    z = np.load(os.path.join(ROOT, "tests", "golden", "llama_tiny_bf16.npz"))
    meta = json.loads(str(z["meta"]))
    meta["tp"] = world
    meta["fuse_tp"] = os.environ.get("TP_WORKER_NCCL_ALLREDUCE") != "1"  # default: all-reduce inside the norm kernel
    if os.environ.get("TP_WORKER_TWO_SHOT") == "1":  # the two-shot exchange also for small groups
        from megatron_mixtera_b200.tensor_parallel import peer_allreduce

        peer_allreduce.ONE_SHOT_MAX_WORLD = 1
    if os.environ.get("TP_WORKER_SPLITK_EXCHANGE") == "1":  # split-K partial sums straight into the two-shot exchange
        from megatron_mixtera_b200.tensor_parallel import peer_allreduce

        peer_allreduce.SPLITK_INTO_EXCHANGE = True
    if os.environ.get("TP_WORKER_SPLIT_POLICY"):  # "ctas per SM,min K blocks per split,max splits": force split-K GEMMs
        from megatron_mixtera_b200 import _lib

        a, b, c = (int(v) for v in os.environ["TP_WORKER_SPLIT_POLICY"].split(","))
        assert _lib.load().b200_set_gemm_split_policy(a, b, c) == 0
    if os.environ.get("TP_WORKER_FP8"):
        meta["fp8"] = os.environ["TP_WORKER_FP8"]  # "mxfp8" | "blockwise": FP8 linears, sharded per rank
    model, ctx, wrapper, Controller = build_cuda_stack(meta, enable_cuda_graph=True)
    # tokens fed back every step: the reference's bf16 trace, or a trace made by the caller (e.g. the FP8 oracle's)
    forced = np.load(os.environ["TP_WORKER_TRACE"]) if os.environ.get("TP_WORKER_TRACE") else z
    out = {}
    state = {"step": 0}

    class Forced(Controller):
        def sample_from_logits(self, last_token_logits, sampling_params=None, vocab_size=None, **kw):
            own = super().sample_from_logits(last_token_logits, sampling_params, vocab_size, **kw)
            if hasattr(last_token_logits, "greedy_tokens"):  # vocabulary-parallel greedy sampling against the gathered rows
                full = last_token_logits.gather()
                assert torch.equal(own, ops.argmax(full.contiguous())), "shard-wise greedy sampling differs from argmax"
                state["vp_checked"] = state.get("vp_checked", 0) + 1
            out[f"s{state['step']}_logits"] = last_token_logits.float().cpu().numpy()
            out[f"s{state['step']}_own"] = own.cpu().numpy()
            return torch.from_numpy(forced[f"s{state['step']}_sample"]).to(last_token_logits.device)

    ctl = Forced(wrapper, types.SimpleNamespace(vocab_size=meta["vocab_size"]))
    sp = SamplingParams(top_k=1, num_tokens_to_generate=meta["num_tokens_to_generate"])
    n = len(meta["prompt_lengths"])
    arrival = meta["arrival_step"]
    step = added = 0
    while added < n or ctx.has_unfinished_requests():
        for i in range(n):
            if arrival[i] == step:
                ctx.add_request(i, torch.from_numpy(z[f"prompt_{i}"]), meta["num_tokens_to_generate"])
                added += 1
        if ctx.active_token_count > 0:
            state["step"] = step
            ctl.generate_output_tokens_dynamic_batch(sp, -1)
            if os.environ.get("TP_WORKER_VERBOSE"):
                print(f"[rank {os.environ.get('RANK', '0')}] step {step} done, decode_only={ctx.is_decode_only()}", file=sys.stderr, flush=True)
        step += 1
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    if world > 1:
        assert state.get("vp_checked", 0) > 5, "the vocabulary-parallel sampling path did not run"
        # every rank must have produced identical logits and tokens (SPMD sampling)
        for k in sorted(out):
            t = torch.from_numpy(out[k]).cuda().double()
            lo, hi = t.clone(), t.clone()
            dist.all_reduce(lo, op=dist.ReduceOp.MIN)
            dist.all_reduce(hi, op=dist.ReduceOp.MAX)
            assert torch.equal(lo, hi), k
    if int(os.environ.get("RANK", "0")) == 0:
        np.savez(out_path, replays=wrapper.graph_replays, tp_splitk_exchanges=ops.tp_splitk_exchanges, **out)
    if world > 1:
        dist.barrier()
        # Not destroy_process_group(): tearing the NCCL communicator down while captured CUDA graphs still
        # reference it blocks for ever (seen on torch 2.11 / NCCL 2.28); release the graphs and just exit.
        wrapper._graphs.clear()
        torch.cuda.synchronize()


if __name__ == "__main__":
    import faulthandler

    # a stuck rank prints where it is and exits instead of waiting for the launcher's timeout
    faulthandler.dump_traceback_later(int(os.environ.get("TP_WORKER_DEADLINE_S", "150")), exit=True)
    (host_mode if sys.argv[1] == "host" else cuda_mode)(sys.argv[2])
