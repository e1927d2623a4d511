"""Helpers for model-level parity at the benchmark's real layer widths (not a test file).

A "cut" is a 2-layer model with the hidden / FFN / head / vocabulary sizes of one of the benchmark workloads.
The CPU oracle produces a trace on seeded prompts; the CUDA stack is then driven through the same scenario
teacher-forced on the oracle's tokens (`test_model_gpu.run_teacher_forced`).  `oracle_floor` measures how far
apart two equally valid CPU evaluations of the same model are (the second one accumulates every dot product in
the opposite order): no implementation can be expected to sit closer to the oracle than the oracle sits to itself.

Used by tests/test_width_parity_gpu.py and, for tensor-parallel runs, by bench.py's `tp_check`.
"""
from __future__ import annotations

import numpy as np
import torch

BF16_BAR = 5e-3  # stated tolerance for bf16 logits (relative L2)
FP8_BAR = 2e-2   # stated tolerance for FP8 logits (relative L2)


def cut_meta(*, hidden_size, ffn_hidden_size, num_attention_heads, num_query_groups, vocab_size, fp8=None, tp=1,
             kv_fp8_scale=None, prompt_lengths=(37, 130, 5, 64), num_tokens_to_generate=3, num_layers=2,
             chunk_size_tokens=128, weight_seed=0):
    max_seq = 512
    return dict(
        llama=True, num_layers=num_layers, hidden_size=hidden_size, num_attention_heads=num_attention_heads,
        num_query_groups=num_query_groups, kv_channels=128, ffn_hidden_size=ffn_hidden_size, vocab_size=vocab_size,
        max_sequence_length=max_seq, rotary_base=500000, weight_seed=weight_seed, prompt_lengths=list(prompt_lengths),
        num_tokens_to_generate=num_tokens_to_generate, rounder=8, chunk_size_tokens=chunk_size_tokens, max_requests=8,
        max_tokens=1024, fp8=fp8, tp=tp, kv_fp8_scale=kv_fp8_scale,
        # pool of 40 chunks whatever the widths: chunk bytes = dtype * 2 * L * chunk * kv heads * 128
        buffer_size_gb=40 * (1 if kv_fp8_scale else 2) * 2 * num_layers * chunk_size_tokens * num_query_groups * 128 / 1024**3)


def bar_for(meta) -> float:
    return FP8_BAR if (meta.get("fp8") or meta.get("kv_fp8_scale")) else BF16_BAR


def floor_factor(meta) -> float:
    """Allowed multiple of the oracle-twin floor (what each is made of: tests/test_width_parity_gpu.py)."""
    if meta.get("kv_fp8_scale"):
        return 2.75
    return 1.75 if meta.get("fp8") == "mxfp8" else 1.2


def cut_prompts(meta):
    g = torch.Generator().manual_seed(1234)
    return [torch.randint(0, meta["vocab_size"], (n,), generator=g, dtype=torch.int64).numpy() for n in meta["prompt_lengths"]]


def _oracle_meta(meta):
    """The oracle's pool is sized in its own dtype (an fp32 copy of an E4M3 pool holds the same chunks)."""
    return meta


def oracle_trace_for(meta, reverse_k: bool = False, forced=None, split_k: int = 1):
    """Trace of the CPU oracle on the cut (`forced`: teacher-force the tokens of an earlier trace)."""
    from oracle import decode_oracle as O
    from test_oracle_golden import build_oracle_model

    model, _ = build_oracle_model(_oracle_meta(meta), torch.bfloat16, fp8=meta.get("fp8"), kv_fp8_scale=meta.get("kv_fp8_scale"),
                                  tp=meta.get("tp", 1))
    model.reverse_k = reverse_k
    model.split_k = split_k
    prompts = cut_prompts(meta)
    trace = {f"prompt_{i}": p for i, p in enumerate(prompts)}

    def on_step(step, c, logits, new, ids):
        if forced is not None:
            new[:] = forced[f"s{step}_sample"]
        trace[f"s{step}_logits"] = logits.float().numpy().copy()
        trace[f"s{step}_sample"] = new.copy()
        trace[f"s{step}_active_request_ids"] = ids.astype(np.int64)
        seq = c.get_active_sequence_lengths() + 1
        trace[f"s{step}_finished_request_ids"] = ids[~((new != -1) & (seq < c.get_max_sequence_lengths()))].astype(np.int64)

    with torch.inference_mode():
        O.decode_loop(model, prompts, meta["num_tokens_to_generate"], on_step=on_step)
    trace["num_steps"] = max(int(k[1:].split("_")[0]) for k in trace if k.startswith("s") and k.endswith("_logits")) + 1
    return trace


def oracle_floor(meta, trace, twins=((True, 1),)):
    """Relative L2 per step between the oracle and "twins" of it - the same model, the same rounding points, every dot
    product accumulated in another order (reversed; in split-K fashion) - on the same token trajectory: the distance
    that separates two correct evaluations of this model in this arithmetic.  Per step the largest over the twins."""
    rel = [0.0] * trace["num_steps"]
    for reverse_k, split_k in twins:
        other = oracle_trace_for(meta, reverse_k=reverse_k, forced=trace, split_k=split_k)
        for s in range(trace["num_steps"]):
            a, b = torch.from_numpy(trace[f"s{s}_logits"]), torch.from_numpy(other[f"s{s}_logits"])
            rel[s] = max(rel[s], float((a - b).norm() / a.norm()))
    return rel


def unquantised_reference(meta, trace):
    """Logits of the same model WITHOUT any FP8 (bf16 oracle), teacher-forced on `trace`'s tokens: the ground truth that
    an FP8 evaluation approximates.  Returns {step: logits}."""
    plain = dict(meta, fp8=None, kv_fp8_scale=None)
    ref = oracle_trace_for(plain, forced=trace)
    return {s: torch.from_numpy(ref[f"s{s}_logits"]) for s in range(trace["num_steps"])}


def run_cuda_cut(meta, trace, enable_cuda_graph: bool = True):
    """The CUDA stack on the cut, teacher-forced on `trace`.  Returns rel-L2 per step, greedy flips, whether every
    flip sits on a near-tie of the oracle's own logits, and a checksum of the logits (rank consistency)."""
    from test_model_gpu import assert_flips_are_near_ties, run_teacher_forced

    state, gen, wrapper = run_teacher_forced(meta, trace, enable_cuda_graph=enable_cuda_graph)
    n_dec = sum(len(v) for k, v in trace.items() if k.endswith("_sample"))
    fp8 = bool(meta.get("fp8") or meta.get("kv_fp8_scale"))
    try:
        # With an E4M3 KV pool the logits of these random-weight cuts sit ~7e-2 (relative L2) from the oracle's, i.e.
        # ~0.1 absolute on logits whose top-1/top-2 margins are often below 0.15: up to a third of the decisions may
        # flip, each still only on such a near-tie (the margin rule above is what catches a wrong kernel).
        assert_flips_are_near_ties(state["flips"], n_dec, resolution=2.0**-4 if fp8 else 2.0**-7,
                                   max_fraction=1 / 3 if meta.get("kv_fp8_scale") else 0.1)
        flips_ok = True
    except AssertionError:
        flips_ok = False
    checksum = float(sum(v.double().sum() for v in state["logits"].values()))
    return {"rel": state["rel"], "flips": state["flips"], "flips_ok": flips_ok, "decisions": n_dec, "checksum": checksum,
            "graph_replays": wrapper.graph_replays, "logits": state["logits"]}
