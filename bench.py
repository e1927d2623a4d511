"""Decode benchmark: Llama-3-8B-shaped bf16 decode, 64 concurrent requests (synthetic weights and prompts).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

For N > 1 launch with torchrun (one rank per GPU); the model is tensor-parallel over the N GPUs.
Rank 0 prints ONE JSON line.  A "step" is one decode step of the whole batch: model forward,
greedy sampling and the context update.

  value      decode tokens/s with every input already on the device: the whole-model CUDA graph plus the
             sampling kernel replayed K times, timed with CUDA events.
  e2e        the same metric through the public API (DynamicInferenceEngine.step_modern): each step
             copies its inputs from pinned host memory, reads the sampled tokens back and updates the
             context on the host.
  roofline   the dominant kernel (the tcgen05 weight-streaming GEMM): algorithmic bytes / CUDA-event
             time of a sweep over the model's own layers, against the measured HBM copy bandwidth.
  cpu_baseline  the CPU oracle (a port of the reference's local-spec PyTorch decode) timed on the
             host cores on a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time
import types

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

METRIC = "decode_tokens_per_second"
UNIT = "tokens/s"


def measured_peak_hbm():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


# ---------------------------------------------------------------------------------------------
# clocks
# ---------------------------------------------------------------------------------------------
class ClockSampler:
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index: int):
        self.device_index = device_index
        self.proc = None
        self.path = None

    def __enter__(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.device_index)], stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None
        return self

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except Exception:
                self.proc.kill()

    def summary(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if not self.path or not os.path.exists(self.path):
            return out
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in open(self.path):
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                mx.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(names, parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        try:
            os.unlink(self.path)
        except OSError:
            pass
        if sm:
            out["sm_mhz"] = statistics.median(sm)
            out["sm_max_mhz"] = max(mx)
            out["samples"] = len(sm)
        out["reasons"] = sorted(reasons)
        return out


# ---------------------------------------------------------------------------------------------
# the CUDA stack
# ---------------------------------------------------------------------------------------------
def build_stack(w, tp: int, seed: int = 0, fuse_splitk: bool = True, fuse_tp: bool = True, fuse_swiglu: bool = True, fuse_qkv: bool = False, overlap: bool = True):
    from megatron_mixtera_b200 import build, parallel_state
    from megatron_mixtera_b200.gpt.gpt_model import GPTModel
    from megatron_mixtera_b200.inference.contexts.dynamic_context import DynamicInferenceContext
    from megatron_mixtera_b200.inference.engines.dynamic_engine import DynamicInferenceEngine
    from megatron_mixtera_b200.inference.model_inference_wrappers.gpt_inference_wrapper import (
        GPTInferenceWrapper, InferenceWrapperConfig)
    from megatron_mixtera_b200.inference.text_generation_controllers.text_generation_controller import (
        TextGenerationController)
    from megatron_mixtera_b200.transformer.transformer_config import TransformerConfig

    build.build()
    cfg = TransformerConfig(
        num_layers=w.num_layers, hidden_size=w.hidden_size, num_attention_heads=w.num_attention_heads,
        num_query_groups=w.num_query_groups, kv_channels=w.kv_channels, ffn_hidden_size=w.ffn_hidden_size,
        normalization="RMSNorm", gated_linear_unit=True, activation="silu", add_bias_linear=False,
        tensor_model_parallel_size=tp, enable_cuda_graph=True, inference_sampling_seed=seed, fp8=w.fp8,
        fuse_splitk_reduction_into_norm=fuse_splitk, fuse_tp_allreduce_into_norm=fuse_tp,
        fuse_swiglu_into_fc1=fuse_swiglu, fuse_qkv_reduction_into_attention=fuse_qkv)
    model = GPTModel(cfg, vocab_size=w.vocab_size, max_sequence_length=w.max_sequence_length,
                     position_embedding_type="rope", rotary_base=w.rotary_base)
    model.init_synthetic_weights(seed=seed)  # N(0, 0.02), generated on the device
    chunks_per_req = -(-w.max_sequence_length // w.chunk_size_tokens)
    kv_elem = 1 if w.kv_fp8 else 2
    chunk_bytes = 2 * kv_elem * w.num_layers * w.chunk_size_tokens * (w.num_query_groups // tp) * w.kv_channels
    n_chunks = int(w.num_requests * chunks_per_req * 1.15) + chunks_per_req + 2
    ctx = DynamicInferenceContext(
        params_dtype=torch.bfloat16, num_layers=w.num_layers, kv_channels=w.kv_channels,
        num_attention_heads=w.num_query_groups, max_sequence_length=w.max_sequence_length,
        buffer_size_gb=n_chunks * chunk_bytes / 1024**3, buffer_guaranteed_fraction=0.05,
        chunk_size_tokens=w.chunk_size_tokens, max_requests_override=w.num_requests,
        max_tokens_override=w.num_requests * w.prompt_len_range[1], tensor_model_parallel_size=tp,
        kv_cache_dtype=torch.float8_e4m3fn if w.kv_fp8 else None, kv_fp8_single_term=w.kv_fp8 == "one_term")
    if w.kv_fp8:
        ctx.kv_scales.fill_(2.0**-6)  # keys / values of the synthetic model stay below 448 * 2^-6 = 7
    wrapper = GPTInferenceWrapper(
        model, InferenceWrapperConfig(hidden_size=w.hidden_size, params_dtype=torch.bfloat16,
                                      padded_vocab_size=w.vocab_size), ctx)
    ctl = TextGenerationController(wrapper, types.SimpleNamespace(vocab_size=w.vocab_size, detokenize=lambda t: ""))
    engine = DynamicInferenceEngine(ctl, ctx, termination_id=-1, random_seed=seed, overlap_host_and_device=overlap)
    return model, ctx, wrapper, ctl, engine


def algorithmic_gemm_bytes(M, N, K, fp8=False):
    if fp8:  # E4M3 operands + one scale byte per 32 elements, bf16 output
        return (N * K + M * K) * (1.0 + 1.0 / 32.0) + 2.0 * M * N
    return 2.0 * (N * K + M * K + M * N)


def kernel_rooflines(model, ctx, T, peak_gbs):
    """Per-kernel algorithmic bytes and CUDA-event time: each kernel is run once per layer on that
    layer's own weights / KV pool (so nothing is served from L2) and the sweep is timed as a whole
    (as one CUDA-graph replay, the way the kernels run inside the decode step)."""
    from megatron_mixtera_b200 import ops

    layers = list(model.decoder.layers)
    H = model.config.hidden_size
    dev = layers[0].self_attention.linear_qkv.weight.device
    stream_events = lambda: (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))

    def sweep(fn, reps=3):
        # The sweep (one launch per layer) is captured into a CUDA graph and the replay is timed: issued one by
        # one from Python, launches shorter than ~15 us would measure the host's launch rate, not the kernel.
        fn()
        torch.cuda.synchronize()
        side = torch.cuda.Stream()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            with torch.cuda.graph(graph, stream=side):
                fn()
        graph.replay()
        torch.cuda.synchronize()
        best = None
        for _ in range(reps):
            e0, e1 = stream_events()
            e0.record()
            graph.replay()
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1)
            best = ms if best is None else min(best, ms)
        return best / 1e3 / len(layers)  # seconds per launch

    out = {}
    gemm_bytes = gemm_time = 0.0
    for name, get in (("linear_qkv", lambda l: l.self_attention.linear_qkv), ("linear_proj", lambda l: l.self_attention.linear_proj),
                      ("linear_fc1", lambda l: l.mlp.linear_fc1), ("linear_fc2", lambda l: l.mlp.linear_fc2)):
        mods = [get(l) for l in layers]
        N, K = mods[0].weight.shape
        fp8 = bool(mods[0].fp8)
        x = torch.randn(T, K, device=dev, dtype=torch.bfloat16)
        if fp8:
            x = ops.quantize_mxfp8(x)
        fused_act = name == "linear_fc1" and getattr(mods[0], "_layout_interleaved", False)
        if fused_act:  # fc1 + SwiGLU in one kernel: the output is [T, N/2]
            sec = sweep(lambda: [m.forward_swiglu(x) for m in mods])
            b = 2.0 * (N * K + T * K + T * N / 2)
        else:
            sec = sweep(lambda: [m._matmul(x, m.weight, None) for m in mods])
            b = algorithmic_gemm_bytes(T, N, K, fp8)
        out[name] = {"us": sec * 1e6, "GB/s": b / sec / 1e9, "frac": b / sec / 1e9 / peak_gbs, "shape": [T, N, K]}
        if fused_act:
            out[name]["fused"] = "swiglu"
        gemm_bytes += b
        gemm_time += sec
    # attention on the live context (decode state)
    attn = layers[0].self_attention.core_attention
    qkv = torch.randn(T, (attn.num_q_heads + 2 * attn.num_kv_heads) * attn.head_dim, device=dev, dtype=torch.bfloat16)
    kv_lens = ctx.kv_seq_lengths_cudagraph_only[:T].cpu()
    kv_elem = 1 if getattr(ctx, "kv_cache_fp8", False) else 2
    kv_bytes = float(kv_lens.sum()) * 2 * attn.num_kv_heads * attn.head_dim * kv_elem + 2.0 * T * qkv.shape[1] * 2
    sec = sweep(lambda: [l.self_attention.core_attention(qkv, ctx, model.rotary_pos_cos, model.rotary_pos_sin) for l in layers])
    out["paged_attention"] = {"us": sec * 1e6, "GB/s": kv_bytes / sec / 1e9, "frac": kv_bytes / sec / 1e9 / peak_gbs,
                              "kv_tokens": int(kv_lens.sum())}
    out["_gemm_total"] = {"bytes": gemm_bytes, "sec": gemm_time}
    return out


# ---------------------------------------------------------------------------------------------
# CPU baseline: the oracle port on the host cores, bounded sample of the same workload
# ---------------------------------------------------------------------------------------------
def cpu_oracle_sample(w, sample_layers: int = 2, reps: int = 2, seed: int = 0):
    """One decode step of the full batch (all requests at their real context lengths) through
    `sample_layers` of the model's layers in fp32 on the CPU, KV pool filled with noise; per-step time of
    the full depth is extrapolated linearly in the layer count (the LM head is timed once, unscaled)."""
    import numpy as np

    from megatron_mixtera_b200.synthetic import canonical_tensor, synthetic_prompts
    from oracle import decode_oracle as O

    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    spec = O.ModelSpec(num_layers=sample_layers, hidden_size=w.hidden_size, num_attention_heads=w.num_attention_heads,
                       num_query_groups=w.num_query_groups, kv_channels=w.kv_channels, ffn_hidden_size=w.ffn_hidden_size,
                       vocab_size=w.vocab_size, max_sequence_length=w.max_sequence_length, llama=True,
                       rotary_base=w.rotary_base)
    H, F, d = w.hidden_size, w.ffn_hidden_size, w.kv_channels
    qkv = (w.num_attention_heads + 2 * w.num_query_groups) * d
    shapes = {"embedding.word_embeddings.weight": (w.vocab_size, H), "decoder.final_layernorm.weight": (H,),
              "output_layer.weight": (w.vocab_size, H)}
    for l in range(sample_layers):
        p = f"decoder.layers.{l}."
        shapes.update({p + "input_layernorm.weight": (H,), p + "self_attention.linear_qkv.weight": (qkv, H),
                       p + "self_attention.linear_proj.weight": (H, w.num_attention_heads * d),
                       p + "pre_mlp_layernorm.weight": (H,), p + "mlp.linear_fc1.weight": (2 * F, H),
                       p + "mlp.linear_fc2.weight": (H, F)})
    weights = {k: canonical_tensor(k, s, seed=seed) for k, s in shapes.items()}
    chunks_per_req = -(-w.max_sequence_length // w.chunk_size_tokens)
    chunk_bytes = 4 * 2 * sample_layers * w.chunk_size_tokens * w.num_query_groups * d
    n_chunks = w.num_requests * chunks_per_req + chunks_per_req + 2
    ctx = O.ContextOracle(dtype_bytes=4, num_layers=sample_layers, kv_channels=d, num_attention_heads=w.num_query_groups,
                          max_sequence_length=w.max_sequence_length, buffer_size_gb=n_chunks * chunk_bytes / 1024**3,
                          buffer_guaranteed_fraction=0.05, chunk_size_tokens=w.chunk_size_tokens,
                          max_requests_override=w.num_requests, max_tokens_override=w.num_requests * w.prompt_len_range[1])
    model = O.GPTOracle(spec, weights, ctx, torch.float32)
    model.k_cache.normal_(0, 0.5)
    model.v_cache.normal_(0, 0.5)
    prompts = synthetic_prompts(w.num_requests, *w.prompt_len_range, w.vocab_size, seed=seed)
    for i, p in enumerate(prompts):
        ctx.add_request(i, p.numpy(), w.num_tokens_to_generate)
    # jump straight to the decode phase: bookkeeping only, the KV of the prompts is the noise above
    ctx.update_requests(np.ones(w.num_requests, dtype=np.uint8), np.zeros(w.num_requests, dtype=np.int64))
    times = []
    with torch.inference_mode():
        for _ in range(reps + 1):
            ctx.initialize_attention_state()
            t0 = time.perf_counter()
            logits = model.forward()
            O.sample(logits)
            times.append(time.perf_counter() - t0)
        # LM head alone, to keep it out of the per-layer extrapolation
        x = torch.randn(w.num_requests, H)
        t0 = time.perf_counter()
        torch.matmul(x, weights["output_layer.weight"].t())
        head = time.perf_counter() - t0
    step = min(times[1:])
    per_layer = max(step - head, 0.0) / sample_layers
    full_step = per_layer * w.num_layers + head
    return {"value": w.num_requests / full_step, "unit": UNIT, "cores": threads, "kind": "port",
            "sample": f"{sample_layers} of {w.num_layers} layers + LM head, fp32, full batch of {w.num_requests} requests at "
                      f"their real context lengths, {reps} decode steps (best), per-layer time scaled to full depth",
            "sample_step_s": step}


def run_reference(args, w):
    """`--impl reference`: the reference's CPU implementation of the path (the oracle port; the Python
    reference itself cannot be shipped to the benchmark machine), all host threads."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    results = [cpu_oracle_sample(w, sample_layers=2, reps=1, seed=i) for i in range(max(1, min(args.steps, 3)))]
    best = max(results, key=lambda r: r["value"])
    line = {"impl": "reference", "metric": METRIC, "value": best["value"], "unit": UNIT, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": w.num_requests / best["value"] * 1e3,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": w.name}, "cpu_baseline": best,
            "e2e": {"value": best["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    emit(line)


# ---------------------------------------------------------------------------------------------
# our arm
# ---------------------------------------------------------------------------------------------
def run_ours(args, w):
    import torch.distributed as dist

    from megatron_mixtera_b200 import ops, parallel_state
    from megatron_mixtera_b200.inference.sampling_params import SamplingParams
    from megatron_mixtera_b200.synthetic import synthetic_prompts

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the decode kernels have no CPU fallback")
    torch.cuda.set_device(local_rank)
    tp = world
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    parallel_state.initialize_model_parallel(tp)
    if args.gpus != world and rank == 0:
        print(f"# note: --gpus {args.gpus} but WORLD_SIZE={world}; running tensor-parallel over {world}", file=sys.stderr)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    model, ctx, wrapper, ctl, engine = build_stack(w, tp, fuse_splitk=not args.unfused_splitk, fuse_tp=not args.nccl_allreduce,
                                                     fuse_swiglu=not args.unfused_swiglu, fuse_qkv=args.fused_qkv, overlap=not args.no_overlap)
    prompts = synthetic_prompts(w.num_requests, *w.prompt_len_range, w.vocab_size, seed=0)
    for i, p in enumerate(prompts):
        engine.add_request(i, p, w.num_tokens_to_generate)
    sp = SamplingParams(top_k=1, num_tokens_to_generate=w.num_tokens_to_generate)
    t0 = time.perf_counter()
    while not ctx.is_decode_only() or ctx.total_request_count < w.num_requests:
        engine.step_modern(sp)  # prefill (excluded from the timed region)
    torch.cuda.synchronize()
    prefill_s = time.perf_counter() - t0
    assert ctx.total_request_count - ctx.paused_request_count == w.num_requests and not engine.waiting_request_ids
    B = w.num_requests
    T = ctx.round_up_tokens(B, tp_size=tp)
    steps, warmup = args.steps, max(args.warmup, 3)
    if warmup + 2 * steps + 2 > w.num_tokens_to_generate:
        raise SystemExit(f"--steps/--warmup too large for {w.num_tokens_to_generate} output tokens per request")

    # ---- e2e: the public API, host<->device copies inside the timed region ----
    for _ in range(warmup):
        engine.step_modern(sp)
    launches0, h2d0 = ops.launch_count, ctx.h2d_bytes
    step_ms = []
    barrier()
    with ClockSampler(local_rank) as clk_e2e:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            r = engine.step_modern(sp)
            step_ms.append(r["step_time"] * 1e3)
            assert len(r["active_requests"]) + len(r["finished_requests"]) == B
        e1.record()
        barrier()
    e2e_s = e0.elapsed_time(e1) / 1e3
    h2d_per_step = (ctx.h2d_bytes - h2d0) / steps
    eager_launches_per_step = (ops.launch_count - launches0) / steps  # sampling only: the forward is a graph

    # ---- value: inputs resident, whole-model graph + sampling kernel replayed ----
    ctx.initialize_attention_state()
    ids, pos = ctx.current_input_and_position_ids()
    inp = {"tokens": ids, "position_ids": pos, "attention_mask": None}
    # launches inside one captured forward = launches of one eager forward of the same shapes
    l0 = ops.launch_count
    wrapper._decode_rows(T)
    graph_launches = ops.launch_count - l0
    for _ in range(warmup):
        ops.argmax(wrapper.run_one_forward_step(inp).squeeze(0).contiguous())
    barrier()
    with ClockSampler(local_rank) as clk:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            ops.argmax(wrapper.run_one_forward_step(inp).squeeze(0).contiguous())
        e1.record()
        barrier()
    dev_s = e0.elapsed_time(e1) / 1e3
    times = torch.tensor([dev_s, e2e_s], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    dev_s, e2e_s = times.tolist()

    peak, peak_kind = measured_peak_hbm()
    kern = kernel_rooflines(model, ctx, T, peak)
    status = ops.device_status()
    if rank != 0:
        if world > 1:
            dist.barrier()
        return
    g = kern.pop("_gemm_total")
    gemm_us = sum(kern[k]["us"] for k in ("linear_qkv", "linear_proj", "linear_fc1", "linear_fc2"))
    layer_us = gemm_us + kern["paged_attention"]["us"]
    cpu = cpu_oracle_sample(w) if not args.no_cpu_baseline else None
    clocks = clk.summary()
    clocks["e2e_region"] = clk_e2e.summary()
    line = {
        "metric": METRIC, "value": B * steps / dev_s, "unit": UNIT, "n_gpus": world, "steps": steps, "warmup": warmup,
        "ms_per_step": dev_s / steps * 1e3, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "mxfp8 linears (fp32 accumulate), bf16 elsewhere" if w.fp8 else "bf16", "data": "synthetic",
        "config": {"workload": w.name, "concurrent_requests": B, "padded_tokens": T, "parallelism": f"tp{tp}",
                   "l2": "per-step inputs (weights + KV pool) far exceed the 126 MB L2; no flush needed",
                   "mean_context_tokens": float(ctx.kv_seq_lengths_cudagraph_only[:B].float().mean())},
        "e2e": {"value": B * steps / e2e_s, "unit": UNIT, "h2d_bytes_per_step": h2d_per_step,
                "d2h_bytes_per_step": B * 8, "ms_per_step": e2e_s / steps * 1e3,
                "p50_step_ms": statistics.median(step_ms)},
        "gpu_launches": int((graph_launches + 1) * steps),
        "launches_per_step": {"graph_forward": graph_launches, "eager_outside_graph": eager_launches_per_step},
        "roofline": {"bound": "hbm", "kernel": f"{'gemm_mxfp8_kernel' if w.fp8 else 'gemm_bf16_kernel'} (tcgen05, {len(model.decoder.layers)} layers x qkv/proj/fc1/fc2)",
                     "achieved": g["bytes"] / g["sec"] / 1e9, "peak": peak, "peak_kind": peak_kind, "unit": "GB/s",
                     "frac": g["bytes"] / g["sec"] / 1e9 / peak,
                     "algorithmic_bytes": g["bytes"], "traffic": GEMM_DRAM_TRAFFIC_PER_LAYER.get((args.workload, tp))},
        "kernels": kern,
        "kernel_share_of_layer": {"gemm": gemm_us / layer_us, "paged_attention": kern["paged_attention"]["us"] / layer_us},
        "step_vs_hbm_floor": {"bytes_per_step": step_bytes(w, ctx, B, tp), "floor_ms": step_bytes(w, ctx, B, tp) / peak / 1e6,
                              "frac": step_bytes(w, ctx, B, tp) / peak / 1e6 / (dev_s / steps * 1e3)},
        "cpu_baseline": cpu, "clocks": clocks, "prefill_s": prefill_s,
        # outside the timed region, wall clock, includes the first-use set-up of every kernel: an indication only
        "prefill": {"prompt_tokens": int(sum(len(p) for p in prompts)), "seconds": prefill_s,
                    "tokens_per_s": sum(len(p) for p in prompts) / prefill_s},
        "device_status": status,
    }
    emit(line)
    if world > 1:
        dist.barrier()


# dram__bytes_read.sum + dram__bytes_write.sum of one layer's four GEMM launches (bytes), from the ncu capture
# summarised in profiles/gemm_bf16_kernel_dram_traffic_llama3_8b_M64.md; the capture exists for the bf16 8B shapes at
# 64 tokens on one GPU only.
GEMM_DRAM_TRAFFIC_PER_LAYER = {("llama3_8b", 1): 441.8e6, ("smoke", 1): 441.8e6}


def step_bytes(w, ctx, B, tp):
    """Algorithmic HBM bytes of one decode step per GPU: every weight once + the resident KV once."""
    H, F, d = w.hidden_size, w.ffn_hidden_size, w.kv_channels
    per_layer = ((w.num_attention_heads + 2 * w.num_query_groups) * d * H + w.num_attention_heads * d * H + 3 * F * H) // tp
    bytes_per_weight = (1.0 + 1.0 / 32.0) if w.fp8 else 2.0
    weights = bytes_per_weight * w.num_layers * per_layer + 2.0 * (w.vocab_size * H // tp)
    kv = float(ctx.kv_seq_lengths_cudagraph_only[:B].sum()) * 2 * (w.num_query_groups // tp) * d * (1 if w.kv_fp8 else 2) * w.num_layers
    return weights + kv


_RESULT_FD = None


def protect_stdout():
    """Keep file descriptor 1 for the one JSON line: libraries that write to stdout themselves (NCCL prints its
    version banner there) are pointed at stderr for the rest of the run."""
    global _RESULT_FD
    sys.stdout.flush()
    _RESULT_FD = os.dup(1)
    os.dup2(2, 1)


def emit(line: dict) -> None:
    data = (json.dumps(line) + "\n").encode()
    if _RESULT_FD is None:
        sys.stdout.write(data.decode())
        sys.stdout.flush()
    else:
        os.write(_RESULT_FD, data)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="llama3_8b", choices=["llama3_8b", "llama3_8b_mxfp8", "llama3_8b_mxfp8_fp8kv", "smoke", "smoke_mxfp8", "smoke_mxfp8_fp8kv"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--nccl-allreduce", action="store_true",
                    help="ablation (TP > 1): NCCL all-reduce + separate norm kernel instead of the fused peer-load kernel")
    ap.add_argument("--fused-qkv", action="store_true",
                    help="ablation: the attention kernel sums the QKV GEMM's split-K partial sums itself")
    ap.add_argument("--no-overlap", action="store_true",
                    help="ablation (e2e): do not enqueue the next decode forward before post-processing the step")
    ap.add_argument("--unfused-swiglu", action="store_true", help="ablation: fc1 and SwiGLU as two kernels")
    ap.add_argument("--unfused-splitk", action="store_true",
                    help="ablation: reduce the split-K partial sums of out-proj / fc2 in a kernel of their own")
    args = ap.parse_args()
    protect_stdout()
    from megatron_mixtera_b200 import configs

    w = {"llama3_8b": configs.LLAMA3_8B_BF16_64REQ, "llama3_8b_mxfp8": configs.LLAMA3_8B_MXFP8_128REQ,
         "llama3_8b_mxfp8_fp8kv": configs.LLAMA3_8B_MXFP8_FP8KV_128REQ, "smoke": configs.LLAMA3_8B_SHAPE_2LAYER, "smoke_mxfp8": configs.LLAMA3_8B_MXFP8_SHAPE_2LAYER,
         "smoke_mxfp8_fp8kv": configs.LLAMA3_8B_MXFP8_FP8KV_SHAPE_2LAYER}[args.workload]
    if args.impl == "reference":
        run_reference(args, w)
    else:
        run_ours(args, w)


if __name__ == "__main__":
    main()
