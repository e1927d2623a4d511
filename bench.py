"""Decode benchmark of the dynamic-inference path (synthetic weights and prompts).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

Default workload: Llama-3-8B shape with MXFP8 linears and a bf16 KV cache, 128 concurrent requests, prompts uniform
in [256, 4096] - the FP8 configuration of the headline metric that fits one GPU and is defined for TP 1/2/4/8.
For N > 1 launch with torchrun (one rank per GPU); the model is tensor-parallel over the N GPUs.
Rank 0 prints ONE JSON line.  A "step" is one decode step of the whole batch: model forward, greedy sampling and
the context update.

  value      decode tokens/s with every input already on the device: the whole-model CUDA graph plus the
             sampling kernel replayed K times, timed with CUDA events.
  e2e        the same metric through the public API (DynamicInferenceEngine.step_modern): each step copies its
             inputs from pinned host memory, reads the sampled tokens back and updates the context on the host.
  roofline   the kernel with the largest share of a layer (paged attention or the GEMM family): algorithmic bytes /
             CUDA-event time of a sweep over the model's own layers, against the measured HBM copy bandwidth;
             the other family is reported beside it (`roofline_other`).
  cpu_baseline  the CPU oracle (a port of the reference's local-spec PyTorch decode) timed on the host cores on a
             bounded sample of the same workload, after the GPU part and with the other ranks gone.
  tp_check   (N > 1, outside every timed region) the tokens sampled in the timed engine steps are identical on all
             ranks, and the logits of a 2-layer cut of the same widths agree with the CPU oracle's restatement of
             the reference's arithmetic at this tensor-parallel size.
"""
from __future__ import annotations

import argparse
import json
import math
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


def host_threads() -> int:
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return os.cpu_count() or 1


# ---------------------------------------------------------------------------------------------
# clocks
# ---------------------------------------------------------------------------------------------
class ClockSampler:
    """One `nvidia-smi` process for the whole measured part (it needs a few hundred milliseconds to start, longer than a
    short timed region): every 20 ms a line with a timestamp; `window(t0, t1)` summarises the lines whose timestamp
    falls inside a timed region (host clock read after a synchronise on either side of it)."""

    FIELDS = ("timestamp,index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index: int):
        self.device_index = device_index
        self.proc = None
        self.path = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "20",
                 "-i", str(self.device_index)], stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None
        return self

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except Exception:
                self.proc.kill()
            self.proc = None

    def _rows(self):
        import datetime

        rows = []
        if not self.path or not os.path.exists(self.path):
            return rows
        for line in open(self.path):
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 10:
                continue
            try:
                ts = datetime.datetime.strptime(parts[0], "%Y/%m/%d %H:%M:%S.%f").timestamp()
                rows.append((ts, float(parts[2]), float(parts[3]), parts[6:10]))
            except ValueError:
                continue
        return rows

    def window(self, t0: float, t1: float, t_warm: float = None):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        rows = self._rows()
        inside = [r for r in rows if t0 <= r[0] <= t1]
        if not inside and t_warm is not None:  # a region shorter than the sampling period: include its warm-up steps,
            inside = [r for r in rows if t_warm <= r[0] <= t1]  # which run the same kernels right before it
            if inside:
                out["note"] = "no sample fell inside the timed region; its warm-up steps are included"
        if not inside and rows:
            mid = 0.5 * (t0 + t1)
            inside = sorted(rows, key=lambda r: abs(r[0] - mid))[:1]
            out["note"] = "no sample fell inside the region; the nearest sample is reported"
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = set()
        for _, _, _, flags in inside:
            for name, val in zip(names, flags):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if inside:
            out["sm_mhz"] = statistics.median(r[1] for r in inside)
            out["sm_max_mhz"] = max(r[2] for r in inside)
            out["samples"] = len(inside)
        out["reasons"] = sorted(reasons)
        return out

    def close(self):
        self.stop()
        try:
            if self.path:
                os.unlink(self.path)
        except OSError:
            pass


# ---------------------------------------------------------------------------------------------
# the CUDA stack
# ---------------------------------------------------------------------------------------------
def request_lengths(w, seed: int = 0):
    from megatron_mixtera_b200.synthetic import synthetic_prompts

    return synthetic_prompts(w.num_requests, *w.prompt_len_range, w.vocab_size, seed=seed, log_uniform=w.log_uniform_lengths)


def build_stack(w, tp: int, prompts, seed: int = 0, fuse_splitk: bool = True, fuse_tp: bool = True, fuse_swiglu: bool = True,
                fuse_qkv: bool = False, overlap: bool = True, keep_bf16_weights: bool = False):
    from megatron_mixtera_b200 import build
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
    if w.fp8 and not keep_bf16_weights:
        model.release_checkpoint_weights()  # the FP8 copies are what the GEMMs stream; frees 2 bytes per weight

    # KV pool: what the requests need at full length (+ slack), capped by the memory that is left on this GPU.
    kv_elem = 1 if w.kv_fp8 else 2
    chunk_bytes = 2 * kv_elem * w.num_layers * w.chunk_size_tokens * (w.num_query_groups // tp) * w.kv_channels
    need_chunks = sum(-(-(len(p) + w.num_tokens_to_generate) // w.chunk_size_tokens) for p in prompts)
    chunks_per_req = -(-w.max_sequence_length // w.chunk_size_tokens)
    want = int(need_chunks * 1.03) + chunks_per_req + 2
    torch.cuda.synchronize()
    torch.cuda.empty_cache()  # the released bf16 weights are still in torch's cache: hand them back before measuring
    free, _total = torch.cuda.mem_get_info()
    # headroom: activations of the largest prefill step, logits, workspaces, CUDA graphs
    prefill_tokens = w.num_requests if w.synthesize_kv else (w.max_prefill_tokens or sum(len(p) for p in prompts))
    act_bytes = prefill_tokens * (2 * w.hidden_size + 3 * (w.ffn_hidden_size // tp) + 2 * (w.num_attention_heads + 2 * w.num_query_groups) * w.kv_channels // tp) * 2
    headroom = int(act_bytes * 1.5) + (6 << 30)
    cap = max(chunks_per_req + 2, (free - headroom) // chunk_bytes)
    n_chunks = min(want, cap)
    max_tokens = w.max_prefill_tokens + w.num_requests if w.max_prefill_tokens else sum(len(p) for p in prompts) + w.num_requests
    ctx = DynamicInferenceContext(
        params_dtype=torch.bfloat16, num_layers=w.num_layers, kv_channels=w.kv_channels,
        num_attention_heads=w.num_query_groups, max_sequence_length=w.max_sequence_length,
        buffer_size_gb=n_chunks * chunk_bytes / 1024**3, buffer_guaranteed_fraction=0.02,
        chunk_size_tokens=w.chunk_size_tokens, max_requests_override=w.num_requests,
        max_tokens_override=max(max_tokens, max(len(p) for p in prompts)), tensor_model_parallel_size=tp,
        kv_cache_dtype=torch.float8_e4m3fn if w.kv_fp8 else None, kv_fp8_single_term=w.kv_fp8 == "one_term")
    if w.kv_fp8:
        ctx.kv_scales.fill_(2.0**-6)  # keys / values of the synthetic model stay below 448 * 2^-6 = 7
    wrapper = GPTInferenceWrapper(
        model, InferenceWrapperConfig(hidden_size=w.hidden_size, params_dtype=torch.bfloat16,
                                      padded_vocab_size=w.vocab_size), ctx)
    ctl = TextGenerationController(wrapper, types.SimpleNamespace(vocab_size=w.vocab_size, detokenize=lambda t: ""))
    engine = DynamicInferenceEngine(ctl, ctx, termination_id=-1, random_seed=seed, overlap_host_and_device=overlap)
    pool = {"chunks": int(n_chunks), "chunks_wanted": int(want), "chunk_bytes": int(chunk_bytes),
            "pool_gb": n_chunks * chunk_bytes / 1e9, "capped_by_memory": bool(n_chunks < want)}
    return model, ctx, wrapper, ctl, engine, pool


def fill_kv_noise(ctx, seed: int = 0) -> None:
    """Seeded N(0, 0.5) keys / values in every chunk of the pool, layer by layer (bounded temporaries)."""
    g = torch.Generator(device=ctx.memory_buffer.device).manual_seed(seed)
    buf = ctx.memory_buffer
    for kv in range(2):
        for layer in range(buf.shape[1]):
            dst = buf[kv, layer]
            step = max(1, (1 << 28) // max(1, dst[0].numel()))
            for c0 in range(0, dst.shape[0], step):
                part = dst[c0 : c0 + step]
                noise = torch.empty(part.shape, dtype=torch.bfloat16, device=buf.device).normal_(0.0, 0.5, generator=g)
                if ctx.kv_cache_fp8:
                    scale = ctx.kv_scales[layer, kv].view(1, 1, -1, 1)
                    part.copy_((noise.float() / scale).clamp_(-448.0, 448.0).to(torch.float8_e4m3fn).view(torch.uint8))
                else:
                    part.copy_(noise)


def algorithmic_gemm_bytes(M, N, K, fp8=None):
    if fp8 == "mxfp8":  # E4M3 operands + one scale byte per 32 elements, bf16 output
        return (N * K + M * K) * (1.0 + 1.0 / 32.0) + 2.0 * M * N
    if fp8 == "blockwise":  # E4M3 operands, fp32 scale per 128 x 128 weight block and per token per 128 of K
        return N * K + M * K + 4.0 * (N * K / 16384.0 + M * K / 128.0) + 2.0 * M * N
    return 2.0 * (N * K + M * K + M * N)


def kernel_rooflines(model, ctx, T, peak_gbs):
    """Per-kernel algorithmic bytes and CUDA-event time: each kernel is run once per layer on that
    layer's own weights / KV pool (so nothing is served from L2) and the sweep is timed as a whole
    (as one CUDA-graph replay, the way the kernels run inside the decode step)."""
    from megatron_mixtera_b200 import ops

    layers = list(model.decoder.layers)
    dev = layers[0].input_layernorm.weight.device
    stream_events = lambda: (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
    reps_of_stack = max(1, 16 // len(layers))  # short stacks (2-layer cuts) are swept several times per replay

    def sweep(fn, reps=3):
        # The sweep (one launch per layer) is captured into a CUDA graph and the replay is timed: issued one by
        # one from Python, launches shorter than ~15 us would measure the host's launch rate, not the kernel.
        fn()
        torch.cuda.synchronize()
        side = torch.cuda.Stream()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            with torch.cuda.graph(graph, stream=side):
                for _ in range(reps_of_stack):
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
        return best / 1e3 / (len(layers) * reps_of_stack)  # seconds per launch

    out = {}
    gemm_bytes = gemm_time = 0.0
    for name, get in (("linear_qkv", lambda l: l.self_attention.linear_qkv), ("linear_proj", lambda l: l.self_attention.linear_proj),
                      ("linear_fc1", lambda l: l.mlp.linear_fc1), ("linear_fc2", lambda l: l.mlp.linear_fc2)):
        mods = [get(l) for l in layers]
        N, K = mods[0].weight_shape
        fp8 = mods[0].fp8
        x = torch.randn(T, K, device=dev, dtype=torch.bfloat16)
        if fp8 == "mxfp8":
            x = ops.quantize_mxfp8(x)
        elif fp8 == "blockwise":
            x = ops.quantize_fp8_rowblock(x)
        interleaved = name == "linear_fc1" and getattr(mods[0], "_layout_interleaved", False)
        gated = name == "linear_fc1" and not interleaved and model.config.gated_linear_unit and hasattr(mods[0], "forward_gated")
        fused_act = interleaved or gated
        if fused_act:  # fc1 + SwiGLU (+ FP8 quantisation of the result): the output is [T, N/2]
            sec = sweep(lambda: [m.forward_swiglu(x) for m in mods]) if interleaved else sweep(lambda: [m.forward_gated(x) for m in mods])
            out_bytes = T * (N // 2) * (2.0 if not fp8 else (1.0 + 1.0 / 32.0 if fp8 == "mxfp8" else 1.0 + 4.0 / 128.0))
            b = algorithmic_gemm_bytes(T, N, K, fp8) - 2.0 * T * N + out_bytes
        else:
            sec = sweep(lambda: [m._matmul(x, m.weight, None) for m in mods])
            b = algorithmic_gemm_bytes(T, N, K, fp8)
        out[name] = {"us": sec * 1e6, "GB/s": b / sec / 1e9, "frac": b / sec / 1e9 / peak_gbs, "shape": [T, N, K],
                     "tflops": 2.0 * T * N * K / sec / 1e12}
        if fused_act:
            out[name]["fused"] = "swiglu" + ("+quantise" if fp8 else "") + ("" if interleaved else " (one kernel or GEMM + activation kernel, as the layer runs it)")
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
                              "kv_tokens": int(kv_lens.sum()), "bytes": kv_bytes}
    out["_gemm_total"] = {"bytes": gemm_bytes, "sec": gemm_time}
    # tensor parallel: the out-projection -> all-reduce -> residual add -> norm (-> quantise) edge as the layer runs it
    # (every rank executes the same sweep, so the exchange kernels meet their peers); minus the GEMM alone = what the
    # collective + norm costs.  bytes = what one rank moves over NVLink for the two-shot exchange.
    from megatron_mixtera_b200 import parallel_state

    tp = parallel_state.get_tensor_model_parallel_world_size()
    if tp > 1 and (len(layers) * reps_of_stack) % 2 == 0:  # (the one-shot form needs an even number of calls per replay)
        proj = [l.self_attention.linear_proj for l in layers]
        K = proj[0].weight_shape[1]
        fp8 = proj[0].fp8
        x = torch.randn(T, K, device=dev, dtype=torch.bfloat16)
        if fp8 == "mxfp8":
            x = ops.quantize_mxfp8(x)
        elif fp8 == "blockwise":
            x = ops.quantize_fp8_rowblock(x)
        H = proj[0].output_size
        res = torch.randn(T, H, device=dev, dtype=torch.bfloat16)

        def edge():
            for l in layers:
                y, _ = l.self_attention.linear_proj(x, defer_reduction=True)
                l.pre_mlp_layernorm.add_and_norm(y, res, quantize=fp8)

        sec = sweep(edge)
        out["proj_allreduce_norm"] = {
            "us": sec * 1e6, "gemm_alone_us": out["linear_proj"]["us"], "collective_and_norm_us": sec * 1e6 - out["linear_proj"]["us"],
            "rows": T, "hidden": H, "nvlink_bytes_per_rank": 2.0 * (tp - 1) / tp * T * H * 2}
    return out


# ---------------------------------------------------------------------------------------------
# CPU baseline: the oracle port on the host cores, bounded sample of the same workload
# ---------------------------------------------------------------------------------------------
CPU_SAMPLE_MAX_REQUESTS = 64
CPU_SAMPLE_MAX_CONTEXT = 8192


class CpuOracleSample:
    """One decode step of a bounded batch (requests at their real context lengths, capped) through `sample_layers`
    of the model's layers in fp32 on the CPU, KV pool filled with noise.  The per-step time of the full depth is the
    per-layer time scaled linearly in the layer count plus the LM head, which is timed on its own."""

    def __init__(self, w, sample_layers: int = 2, seed: int = 0):
        import numpy as np

        from megatron_mixtera_b200.synthetic import canonical_tensor
        from oracle import decode_oracle as O

        self.w, self.sample_layers, self.O, self.np = w, sample_layers, O, np
        self.threads = host_threads()
        torch.set_num_threads(self.threads)
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
        self.weights = weights
        prompts = request_lengths(w, seed)[:CPU_SAMPLE_MAX_REQUESTS]
        prompts = [p[:CPU_SAMPLE_MAX_CONTEXT] for p in prompts]
        self.batch = len(prompts)
        self.mean_context = sum(len(p) for p in prompts) / len(prompts)
        max_len = max(len(p) for p in prompts) + w.num_tokens_to_generate
        spec.max_sequence_length = max_len
        chunk_bytes = 4 * 2 * sample_layers * w.chunk_size_tokens * w.num_query_groups * d
        n_chunks = sum(-(-(len(p) + 8) // w.chunk_size_tokens) for p in prompts) + -(-max_len // w.chunk_size_tokens) + 2
        ctx = O.ContextOracle(dtype_bytes=4, num_layers=sample_layers, kv_channels=d, num_attention_heads=w.num_query_groups,
                              max_sequence_length=max_len, buffer_size_gb=n_chunks * chunk_bytes / 1024**3,
                              buffer_guaranteed_fraction=0.02, chunk_size_tokens=w.chunk_size_tokens,
                              max_requests_override=self.batch, max_tokens_override=sum(len(p) for p in prompts) + self.batch)
        self.model = O.GPTOracle(spec, weights, ctx, torch.float32)
        self.model.k_cache.normal_(0, 0.5)
        self.model.v_cache.normal_(0, 0.5)
        for i, p in enumerate(prompts):
            ctx.add_request(i, p.numpy(), w.num_tokens_to_generate)
        # jump straight to the decode phase: bookkeeping only, the KV of the prompts is the noise above
        ctx.update_requests(np.ones(self.batch, dtype=np.uint8), np.zeros(self.batch, dtype=np.int64))
        self.ctx = ctx
        with torch.inference_mode():  # LM head alone, to keep it out of the per-layer extrapolation
            x = torch.randn(self.batch, H)
            torch.matmul(x, weights["output_layer.weight"].t())
            t0 = time.perf_counter()
            torch.matmul(x, weights["output_layer.weight"].t())
            self.head_s = time.perf_counter() - t0

    def step(self) -> float:
        """Seconds of one sample step (forward of the sampled layers + LM head + greedy sampling)."""
        with torch.inference_mode():
            self.ctx.initialize_attention_state()
            t0 = time.perf_counter()
            logits = self.model.forward()
            self.O.sample(logits)
            return time.perf_counter() - t0

    def describe(self, step_s: float, n_steps: int):
        w = self.w
        per_layer = max(step_s - self.head_s, 0.0) / self.sample_layers
        full_step = per_layer * w.num_layers + self.head_s
        capped = self.batch < w.num_requests or w.prompt_len_range[1] > CPU_SAMPLE_MAX_CONTEXT
        return {"value": self.batch / full_step, "unit": UNIT, "cores": self.threads, "kind": "port",
                "sample": f"{self.sample_layers} of {w.num_layers} layers + LM head, fp32, {self.batch} requests"
                          f"{' (capped; contexts capped at %d tokens)' % CPU_SAMPLE_MAX_CONTEXT if capped else ''} at mean context "
                          f"{self.mean_context:.0f} tokens, {n_steps} decode step(s) (median), per-layer time scaled to "
                          f"{w.num_layers} layers (extrapolated)",
                "sample_step_s": step_s, "full_step_s_extrapolated": full_step}


def cpu_oracle_sample(w, reps: int = 2):
    s = CpuOracleSample(w)
    s.step()
    times = [s.step() for _ in range(reps)]
    return s.describe(statistics.median(times), reps)


def run_reference(args, w):
    """`--impl reference`: the reference's CPU implementation of the path (the oracle port; the Python reference
    itself cannot be shipped to the benchmark machine), all host threads.  A step here is one SAMPLE step (2 of the
    model's layers + LM head on a bounded batch); `steps` and `ms_per_step` describe exactly what was run, and
    `value` is the decode rate of the full depth extrapolated from it."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    s = CpuOracleSample(w)
    for _ in range(max(1, args.warmup)):
        s.step()
    t0 = time.perf_counter()
    times = [s.step() for _ in range(max(1, args.steps))]
    wall = time.perf_counter() - t0
    cpu = s.describe(statistics.median(times), len(times))
    line = {"impl": "reference", "metric": METRIC, "value": cpu["value"], "unit": UNIT, "n_gpus": args.gpus,
            "steps": len(times), "warmup": max(1, args.warmup), "ms_per_step": wall / len(times) * 1e3,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": w.name, "extrapolated": cpu["sample"],
                       "note": "ms_per_step is the measured SAMPLE step (2 layers + LM head); value is tokens/s of the "
                               "full depth extrapolated from it"},
            "cpu_baseline": cpu,
            "e2e": {"value": cpu["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    emit(line)


# ---------------------------------------------------------------------------------------------
# tensor-parallel correctness, visible in the benchmark record
# ---------------------------------------------------------------------------------------------
def tp_cut_check(w, tp: int, rank: int, with_floor: bool = True):
    """Logits of a 2-layer cut of the workload's widths at this tensor-parallel size against the CPU oracle's
    restatement of the reference's TP arithmetic (teacher forced), plus rank consistency of the logits."""
    import torch.distributed as dist

    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import width_parity as WP

    meta = WP.cut_meta(hidden_size=w.hidden_size, ffn_hidden_size=w.ffn_hidden_size, num_attention_heads=w.num_attention_heads,
                       num_query_groups=w.num_query_groups, vocab_size=w.vocab_size, fp8=w.fp8, tp=tp,
                       kv_fp8_scale=2.0**-6 if w.kv_fp8 == "two_term" else None, prompt_lengths=[37, 130, 5, 64],
                       num_tokens_to_generate=3)
    trace, floor = None, None
    if rank == 0:
        torch.set_num_threads(host_threads())  # torchrun pins OMP_NUM_THREADS to 1; the oracle may use every core
        trace = WP.oracle_trace_for(meta)
        if with_floor:  # the oracle against a twin of itself (every dot product accumulated in reverse order)
            floor = WP.oracle_floor(meta, trace)
    box = [trace, floor]
    dist.broadcast_object_list(box, src=0)
    trace, floor = box
    res = WP.run_cuda_cut(meta, trace)
    mine = torch.tensor([res["checksum"]], dtype=torch.float64, device="cuda")
    allc = [torch.zeros_like(mine) for _ in range(tp)]
    dist.all_gather(allc, mine)
    same = all(float(c) == float(allc[0]) for c in allc)
    bar = WP.bar_for(meta)
    out = {"cut": f"2 layers, hidden {w.hidden_size}, ffn {w.ffn_hidden_size}, vocab {w.vocab_size}, recipe {w.fp8 or 'bf16'}, tp{tp}",
           "logits_rel_l2_vs_tp_oracle": {"max": max(res["rel"]), "mean": sum(res["rel"]) / len(res["rel"])},
           "bar": bar, "within_bar": bool(max(res["rel"]) <= bar), "greedy_flips": len(res["flips"]),
           "flips_are_near_ties": bool(res["flips_ok"]), "logits_identical_on_all_ranks": bool(same)}
    if floor is not None:
        # the oracle itself is this far from an equally valid evaluation of the same model: where that is above the bar,
        # no implementation can meet the bar against this oracle, and the check is a stated multiple of the floor
        factor = WP.floor_factor(meta)
        out.update({"oracle_twin_floor": {"max": max(floor), "mean": sum(floor) / len(floor)}, "floor_factor_allowed": factor,
                    "within_floor_factor": bool(max(res["rel"]) <= max(bar, factor * max(floor)))})
    return out


# ---------------------------------------------------------------------------------------------
# our arm
# ---------------------------------------------------------------------------------------------
def run_ours(args, w):
    import numpy as np
    import torch.distributed as dist

    from megatron_mixtera_b200 import ops, parallel_state
    from megatron_mixtera_b200.inference.sampling_params import SamplingParams

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the decode kernels have no CPU fallback")
    torch.cuda.set_device(local_rank)
    tp = world
    if tp < w.min_tp:
        raise SystemExit(f"workload '{args.workload}' needs tensor parallel size >= {w.min_tp} (launch with torchrun)")
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    parallel_state.initialize_model_parallel(tp)
    if args.gpus != world and rank == 0:
        print(f"# note: --gpus {args.gpus} but WORLD_SIZE={world}; running tensor-parallel over {world}", file=sys.stderr)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    if args.split_policy:
        from megatron_mixtera_b200 import _lib as _l

        a_, b_, c_ = (int(v) for v in args.split_policy.split(","))
        _l.check("b200_set_gemm_split_policy", _l.load().b200_set_gemm_split_policy(a_, b_, c_))
    if args.splitk_into_exchange:
        from megatron_mixtera_b200.tensor_parallel import peer_allreduce as _pa

        _pa.SPLITK_INTO_EXCHANGE = True
    if args.one_shot_max_world is not None:
        from megatron_mixtera_b200.tensor_parallel import peer_allreduce

        peer_allreduce.ONE_SHOT_MAX_WORLD = args.one_shot_max_world
    prompts = request_lengths(w, seed=0)
    model, ctx, wrapper, ctl, engine, pool = build_stack(
        w, tp, prompts, fuse_splitk=not args.unfused_splitk, fuse_tp=not args.nccl_allreduce,
        fuse_swiglu=not args.unfused_swiglu, fuse_qkv=args.fused_qkv, overlap=not args.no_overlap)
    sp = SamplingParams(top_k=1, num_tokens_to_generate=w.num_tokens_to_generate)
    t0 = time.perf_counter()
    for i, p in enumerate(prompts):
        engine.add_request(i, p, w.num_tokens_to_generate)
    if w.synthesize_kv:
        # only the bookkeeping of the prefill runs; the pool holds seeded noise in place of the prompts' keys / values
        fill_kv_noise(ctx)
        n = ctx.total_request_count
        ctx.update_requests(np.ones(n, dtype=np.uint8), np.zeros(n, dtype=np.int64))
    prefill_steps = 0
    waiting_before = None
    while True:
        if ctx.is_decode_only():
            waiting = len(engine.waiting_request_ids)
            if waiting == 0 or waiting == waiting_before:
                break  # everybody is in, or the pool admits no more: the rest stays queued (see `concurrent_requests`)
            waiting_before = waiting
        engine.step_modern(sp)  # prefill / admission (excluded from the timed region)
        prefill_steps += 1
        if prefill_steps > 4 * w.num_requests:
            break
    torch.cuda.synchronize()
    prefill_s = time.perf_counter() - t0
    # requests that did not fit the pool stay queued (or paused): the measured batch is what is concurrently active
    B = ctx.total_request_count - ctx.paused_request_count
    if B <= 0:
        raise SystemExit("no request could be admitted: the KV pool is too small for this workload on this GPU")
    T = ctx.padded_active_token_count if ctx.padded_active_token_count else ctx.round_up_tokens(B, tp_size=tp)
    steps, warmup = args.steps, max(args.warmup, 3)
    remaining = w.num_tokens_to_generate - prefill_steps - 2
    if warmup + 2 * steps + 2 > remaining:
        raise SystemExit(f"--steps/--warmup too large for {w.num_tokens_to_generate} output tokens per request")

    # ---- e2e: the public API, host<->device copies inside the timed region ----
    sampler = ClockSampler(local_rank).start()  # runs through both timed regions
    t_e2e_warm = time.time()
    for _ in range(warmup):
        engine.step_modern(sp)
    B = ctx.total_request_count - ctx.paused_request_count
    launches0, h2d0 = ops.launch_count, ctx.h2d_bytes
    step_ms, step_tokens, sampled = [], 0, []
    barrier()
    t_e2e0 = time.time()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        r = engine.step_modern(sp)
        step_ms.append(r["step_time"] * 1e3)
        step_tokens += len(r["active_requests"]) + len(r["finished_requests"])
        sampled.append([req.generated_tokens[-1] for req in r["active_requests"]])
    e1.record()
    barrier()
    t_e2e1 = time.time()
    e2e_s = e0.elapsed_time(e1) / 1e3
    h2d_per_step = (ctx.h2d_bytes - h2d0) / steps
    eager_launches_per_step = (ops.launch_count - launches0) / steps  # sampling only: the forward is a graph
    e2e_tokens_per_step = step_tokens / steps

    # ---- value: inputs resident, whole-model graph + sampling kernel replayed ----
    ctx.initialize_attention_state()
    B = ctx.total_request_count - ctx.paused_request_count
    T = ctx.padded_active_token_count
    ids, pos = ctx.current_input_and_position_ids()
    inp = {"tokens": ids, "position_ids": pos, "attention_mask": None}
    # launches inside one captured forward = launches of one eager forward of the same shapes
    l0 = ops.launch_count
    wrapper._decode_rows(T)
    graph_launches = ops.launch_count - l0
    torch.cuda.synchronize()
    t_dev_warm = time.time()
    for _ in range(warmup):
        ctl.sample_from_logits(wrapper.run_one_forward_step(inp).squeeze(0), sp, vocab_size=w.vocab_size)
    barrier()
    torch.cuda.synchronize()
    torch.cuda.profiler.start()  # a profiler started with "--profile-from-start off" sees the timed launches only
    t_dev0 = time.time()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        ctl.sample_from_logits(wrapper.run_one_forward_step(inp).squeeze(0), sp, vocab_size=w.vocab_size)
    e1.record()
    barrier()
    torch.cuda.synchronize()
    t_dev1 = time.time()
    torch.cuda.profiler.stop()
    dev_s = e0.elapsed_time(e1) / 1e3
    times = torch.tensor([dev_s, e2e_s], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    dev_s, e2e_s = times.tolist()

    peak, peak_kind = measured_peak_hbm()
    kern = kernel_rooflines(model, ctx, T, peak)
    status = ops.device_status()
    mean_ctx = float(ctx.kv_seq_lengths_cudagraph_only[:B].float().mean())
    sbytes = step_bytes(w, ctx, B, tp)

    # ---- tensor-parallel correctness (outside every timed region) ----
    tp_check = None
    if world > 1:
        mine = torch.tensor([t for row in sampled for t in row], dtype=torch.int64, device="cuda")
        gathered = [torch.zeros_like(mine) for _ in range(world)]
        dist.all_gather(gathered, mine)
        tp_check = {"timed_steps_checked": len(sampled), "tokens_per_step": len(sampled[0]) if sampled else 0,
                    "sampled_tokens_identical_on_all_ranks": bool(all(torch.equal(g, gathered[0]) for g in gathered))}
        if not args.no_tp_check:
            tp_check.update(tp_cut_check(w, tp, rank, with_floor=not args.no_tp_floor))
        dist.barrier()
        torch.cuda.synchronize()
        # The other ranks leave now, so that rank 0 has the host cores to itself for the CPU leg; no collective is
        # issued after this point.  The process group is NOT destroyed: tearing the NCCL communicator down while
        # captured CUDA graphs still reference it blocks for ever (torch 2.11 / NCCL 2.28); the graphs are released
        # and every rank leaves through os._exit once its output is flushed.
        wrapper._graphs.clear()
        torch.cuda.synchronize()
    if rank != 0:
        leave()
    g = kern.pop("_gemm_total")
    gemm_us = sum(kern[k]["us"] for k in ("linear_qkv", "linear_proj", "linear_fc1", "linear_fc2"))
    attn = kern["paged_attention"]
    layer_us = gemm_us + attn["us"]
    clocks = sampler.window(t_dev0, t_dev1, t_dev_warm)
    clocks["e2e_region"] = sampler.window(t_e2e0, t_e2e1, t_e2e_warm)
    sampler.close()
    gemm_name = {None: "gemm_bf16_kernel", "mxfp8": "gemm_mxfp8_kernel", "blockwise": "gemm_fp8_block_kernel"}[w.fp8]
    attn_name = "paged_attention_fp8_kernel" if w.kv_fp8 else "paged_attention_kernel"
    roof_gemm = {"bound": "hbm", "kernel": f"{gemm_name} (tcgen05, {len(model.decoder.layers)} layers x qkv/proj/fc1/fc2)",
                 "achieved": g["bytes"] / g["sec"] / 1e9, "peak": peak, "peak_kind": peak_kind, "unit": "GB/s",
                 "frac": g["bytes"] / g["sec"] / 1e9 / peak, "algorithmic_bytes": g["bytes"],
                 "share_of_layer": gemm_us / layer_us, "traffic": DRAM_TRAFFIC.get((args.workload, tp, "gemm"))}
    roof_attn = {"bound": "hbm", "kernel": f"{attn_name} ({len(model.decoder.layers)} layers, {attn['kv_tokens']} resident KV tokens)",
                 "achieved": attn["GB/s"], "peak": peak, "peak_kind": peak_kind, "unit": "GB/s", "frac": attn["frac"],
                 "algorithmic_bytes": attn["bytes"], "share_of_layer": attn["us"] / layer_us,
                 "traffic": attention_traffic(args.workload, tp, attn["kv_tokens"])}
    for r_ in (roof_gemm, roof_attn):
        if r_["traffic"] is None:
            r_["traffic_note"] = "no ncu capture of this kernel on this workload / TP size is committed under profiles/"
    dominant, other = (roof_attn, roof_gemm) if attn["us"] >= gemm_us else (roof_gemm, roof_attn)
    cpu = None if args.no_cpu_baseline else cpu_oracle_sample(w)
    dtype = {None: "bf16", "mxfp8": "mxfp8 linears (E4M3 x E4M3, E8M0 scale per 32, fp32 accumulate)",
             "blockwise": "fp8 linears (E4M3, 128x128 weight / 1x128 token fp32 scales, fp32 accumulate)"}[w.fp8]
    dtype += ", E4M3 KV" if w.kv_fp8 else ", bf16 KV and activations" if w.fp8 else ""
    line = {
        "metric": METRIC, "value": B * steps / dev_s, "unit": UNIT, "n_gpus": world, "steps": steps, "warmup": warmup,
        "ms_per_step": dev_s / steps * 1e3, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": dtype, "data": "synthetic",
        "config": {"workload": w.name, "workload_key": args.workload, "concurrent_requests": B,
                   "requested_requests": w.num_requests, "padded_tokens": T, "parallelism": f"tp{tp}",
                   "l2": "per-step inputs (weights + KV pool) far exceed the 126 MB L2; no flush needed",
                   "mean_context_tokens": mean_ctx, "kv_pool": pool},
        "e2e": {"value": e2e_tokens_per_step * steps / e2e_s, "unit": UNIT, "h2d_bytes_per_step": h2d_per_step,
                "d2h_bytes_per_step": e2e_tokens_per_step * 8, "ms_per_step": e2e_s / steps * 1e3,
                "p50_step_ms": statistics.median(step_ms)},
        "gpu_launches": int((graph_launches + 1) * steps),
        "launches_per_step": {"graph_forward": graph_launches, "eager_outside_graph": eager_launches_per_step,
                              "per_layer": (graph_launches - 4) / max(1, len(model.decoder.layers))},
        "roofline": dominant, "roofline_other": other,
        "kernels": kern,
        "kernel_share_of_layer": {"gemm": gemm_us / layer_us, "paged_attention": attn["us"] / layer_us},
        "step_vs_hbm_floor": {"bytes_per_step": sbytes, "floor_ms": sbytes / peak / 1e6,
                              "frac": sbytes / peak / 1e6 / (dev_s / steps * 1e3)},
        "tp_check": tp_check, "cpu_baseline": cpu, "clocks": clocks, "prefill_s": prefill_s,
        # outside the timed region, wall clock, includes the first-use set-up of every kernel: an indication only
        "prefill": {"prompt_tokens": int(sum(len(p) for p in prompts)), "seconds": prefill_s, "steps": prefill_steps,
                    "synthesized_kv": bool(w.synthesize_kv)},
        "device_status": status,
    }
    emit(line)
    if world > 1:
        leave()


def leave():
    sys.stdout.flush()
    sys.stderr.flush()
    os._exit(0)


# dram__bytes_read.sum + dram__bytes_write.sum per launch (bytes) from the ncu captures summarised under profiles/,
# keyed by (workload, tensor-parallel size, kernel family).  "gemm" = the four GEMM launches of one layer together.
# A 2-layer cut has the same per-launch shapes, batch and contexts as its full workload, so its figure carries over.
DRAM_TRAFFIC = {
    ("llama3_8b", 1, "gemm"): 441.8e6,   # profiles/gemm_bf16_kernel_dram_traffic_llama3_8b_M64.md
    ("smoke", 1, "gemm"): 441.8e6,
    ("llama3_8b_mxfp8", 1, "gemm"): 228.8e6,   # profiles/dram_traffic_llama3_8b_mxfp8_decode_128req.md
    ("smoke_mxfp8", 1, "gemm"): 228.8e6,
}
# Attention traffic grows with the resident KV tokens: bytes per token from the same capture (1164.3 MB / 279 237 tokens;
# 4096 of them are the token's K and V in bf16 over 8 KV heads x 128).
DRAM_TRAFFIC_PER_KV_TOKEN = {
    ("llama3_8b_mxfp8", 1): 4169.5,
    ("smoke_mxfp8", 1): 4169.5,
}


def attention_traffic(workload: str, tp: int, kv_tokens: int):
    per_token = DRAM_TRAFFIC_PER_KV_TOKEN.get((workload, tp))
    return None if per_token is None else per_token * kv_tokens


def step_bytes(w, ctx, B, tp):
    """Algorithmic HBM bytes of one decode step per GPU: every weight once + the resident KV once."""
    H, F, d = w.hidden_size, w.ffn_hidden_size, w.kv_channels
    per_layer = ((w.num_attention_heads + 2 * w.num_query_groups) * d * H + w.num_attention_heads * d * H + 3 * F * H) // tp
    bytes_per_weight = {None: 2.0, "mxfp8": 1.0 + 1.0 / 32.0, "blockwise": 1.0 + 4.0 / 16384.0}[w.fp8]
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
    from megatron_mixtera_b200 import configs

    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=configs.DEFAULT_WORKLOAD, choices=sorted(configs.WORKLOADS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-tp-check", action="store_true",
                    help="N > 1: skip the 2-layer cut against the CPU oracle (the token comparison across ranks stays)")
    ap.add_argument("--no-tp-floor", action="store_true",
                    help="N > 1: skip the oracle-against-its-twin run that puts the cut's distance into context")
    ap.add_argument("--one-shot-max-world", type=int, default=None,
                    help="ablation (TP > 1): largest group that uses the one-shot fused all-reduce (larger ones: two-shot)")
    ap.add_argument("--nccl-allreduce", action="store_true",
                    help="ablation (TP > 1): NCCL all-reduce + separate norm kernel instead of the fused peer-memory kernel")
    ap.add_argument("--fused-qkv", action="store_true",
                    help="ablation: the attention kernel sums the QKV GEMM's split-K partial sums itself")
    ap.add_argument("--no-overlap", action="store_true",
                    help="ablation (e2e): do not enqueue the next decode forward before post-processing the step")
    ap.add_argument("--unfused-swiglu", action="store_true", help="ablation: fc1 and SwiGLU as two kernels")
    ap.add_argument("--unfused-splitk", action="store_true",
                    help="ablation: reduce the split-K partial sums of out-proj / fc2 in a kernel of their own")
    ap.add_argument("--split-policy", default=None,
                    help="GEMM split-K policy 'CTAs per SM wanted,min K blocks per split,max splits' (default 2,4,32)")
    ap.add_argument("--splitk-into-exchange", action="store_true",
                    help="ablation: the two-shot exchange kernel sums the row-parallel GEMMs' split-K partial sums itself")
    ap.add_argument("--synthesize-kv", action="store_true",
                    help="skip the prefill forward passes: admit the requests through the bookkeeping only and fill the KV "
                         "pool with seeded noise (decode timing does not depend on the pool's contents)")
    ap.add_argument("--deadline", type=int, default=1500,
                    help="seconds after which a stuck run dumps every thread's stack and exits instead of waiting to be killed")
    args = ap.parse_args()
    import faulthandler

    faulthandler.dump_traceback_later(args.deadline, exit=True)
    protect_stdout()
    w = configs.WORKLOADS[args.workload]
    if args.synthesize_kv and not w.synthesize_kv:
        import dataclasses

        w = dataclasses.replace(w, synthesize_kv=True, max_prefill_tokens=0,
                                name=w.name + " (KV pool filled with seeded noise instead of a prefill)")
    if args.impl == "reference":
        run_reference(args, w)
    else:
        run_ours(args, w)


if __name__ == "__main__":
    main()
