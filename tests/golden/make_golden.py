"""Generate the committed golden fixtures by running the REFERENCE itself on CPU.

Run from the repository root, in a container that has the reference checkout:

    TORCHDYNAMO_DISABLE=1 python tests/golden/make_golden.py --ref /path/to/reference

Nothing here is needed at test time; the tests only read the ``*.npz`` files this
script wrote.  The reference needs three shims to run without a GPU:

1. ``torch.cuda.current_device`` returns the CPU device (the reference hard-codes it
   as the device of every bookkeeping tensor);
2. the CUDA RNG tracker's ``fork`` becomes a null context (eval-mode dropout);
3. ``Attention.flash_decode_and_prefill`` (a flash-attn call with no CPU kernel) is
   replaced by a dense fp32-softmax restatement of the same contract: paged K/V gathered
   through the block table, query head h reads KV head h // group, causal mask aligned
   bottom-right, all-masked rows give zeros.

Weights are not the reference's own initialisation: they come from
``megatron_mixtera_b200.synthetic.canonical_tensor`` (seeded per state-dict key), loaded
with ``load_state_dict``, so the tests can rebuild exactly the same model.
"""
from __future__ import annotations

import argparse
import contextlib
import json
import math
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))


def _shim_and_import(ref_path: str):
    sys.path.insert(0, ref_path)
    sys.path.insert(0, ROOT)
    os.environ.setdefault("TORCHDYNAMO_DISABLE", "1")
    torch.cuda.current_device = lambda: torch.device("cpu")
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29533")
    import torch.distributed as dist

    if not dist.is_initialized():
        dist.init_process_group("gloo", rank=0, world_size=1)
    from megatron.core import parallel_state as ps

    ps.initialize_model_parallel(1, 1)
    from megatron.core.tensor_parallel import random as _r

    _r.CudaRNGStatesTracker.fork = lambda self, name=None: contextlib.nullcontext()
    from megatron.core.transformer import attention as A

    def dense_paged_attention(self, q, k, v, max_seqlen_q, max_seqlen_k, cu_q, cu_k, seqlens_k, block_table):
        T, _, H, D = q.shape
        Hkv = k.shape[2]
        g = H // Hkv
        cs = k.shape[1]
        out = torch.zeros(T, 1, H, D, dtype=q.dtype)
        if max_seqlen_q == 1:
            qlens = [1] * block_table.shape[0]
        else:
            qlens = (cu_q[1:] - cu_q[:-1]).tolist()
        off = 0
        for r, ql in enumerate(qlens):
            kl = int(seqlens_k[r])
            if kl == 0 or ql == 0:
                off += ql
                continue
            nblk = math.ceil(kl / cs)
            ids = block_table[r, :nblk].long()
            kk = k[ids].reshape(-1, Hkv, D)[:kl].float().repeat_interleave(g, 1)
            vv = v[ids].reshape(-1, Hkv, D)[:kl].float().repeat_interleave(g, 1)
            qq = q[off : off + ql, 0].float()
            s = torch.einsum("qhd,khd->hqk", qq, kk) * (D**-0.5)
            mask = torch.ones(ql, kl, dtype=torch.bool).tril(kl - ql)
            s = s.masked_fill(~mask, float("-inf"))
            o = torch.einsum("hqk,khd->qhd", s.softmax(-1), vv)
            out[off : off + ql, 0] = o.to(q.dtype)
            off += ql
        return out

    A.Attention.flash_decode_and_prefill = dense_paged_attention


def _snap_ctx(ctx, prefix, out):
    """Bookkeeping snapshot (everything the kernels or the parity tests consume)."""
    n_act = ctx.active_token_count
    n_pad = ctx.padded_active_token_count or 0
    out[prefix + "counts"] = np.array(
        [
            ctx.total_request_count,
            ctx.paused_request_count,
            n_act,
            n_pad,
            ctx.padded_active_request_count or 0,
            int(ctx.is_decode_only()),
            ctx.chunk_allocator.chunk_count_avail,
        ],
        dtype=np.int64,
    )
    out[prefix + "input_ids"] = ctx.token_to_input_ids[:n_act].numpy().copy()
    out[prefix + "pos_ids"] = ctx.token_to_pos_ids[:n_act].numpy().copy()
    out[prefix + "request_idx"] = ctx.token_to_request_idx[:n_act].numpy().copy()
    out[prefix + "chunk_idx"] = ctx.token_to_chunk_idx[:n_pad].numpy().copy()
    out[prefix + "local_pos"] = ctx.token_to_local_position_within_kv_chunk[:n_pad].numpy().copy()
    out[prefix + "pos_in_request"] = ctx.token_to_position_in_request[:n_pad].numpy().copy()
    p, t = ctx.paused_request_count, ctx.total_request_count
    out[prefix + "request_ids"] = ctx.request_ids[:t].numpy().copy()
    out[prefix + "request_query_lengths"] = ctx.request_query_lengths[:t].numpy().copy()
    out[prefix + "request_output_lengths"] = ctx.request_output_lengths[:t].numpy().copy()
    out[prefix + "request_kv_length_offsets"] = ctx.request_kv_length_offsets[:t].numpy().copy()
    out[prefix + "request_kv_chunk_counts"] = ctx.request_kv_chunk_counts[:t].numpy().copy()
    out[prefix + "request_last_kv_chunk_id"] = ctx.request_last_kv_chunk_id[:t].numpy().copy()
    out[prefix + "request_last_kv_chunk_offset"] = ctx.request_last_kv_chunk_offset[:t].numpy().copy()
    out[prefix + "request_to_kv_chunk_ids"] = ctx.request_to_kv_chunk_ids[:t].numpy().copy()
    out[prefix + "chunk_bag"] = ctx.chunk_allocator.chunk_bag.numpy().copy()
    if ctx.kv_seq_lengths is not None:
        out[prefix + "kv_seq_lengths"] = ctx.kv_seq_lengths.numpy().copy()
        out[prefix + "block_table"] = ctx.block_table.numpy().copy()
        out[prefix + "max_seqlen"] = np.array([ctx.max_seqlen_q, ctx.max_seqlen_k], dtype=np.int64)
        if ctx.cu_query_seq_lengths is not None:
            out[prefix + "cu_query_seq_lengths"] = ctx.cu_query_seq_lengths.numpy().copy()
            out[prefix + "cu_kv_seq_lengths"] = ctx.cu_kv_seq_lengths.numpy().copy()


# --------------------------------------------------------------------------------------
# Context-only scenario: random admissions / terminations with a tight chunk budget so
# that pausing, resuming, chunk release and row compaction are all exercised.
# --------------------------------------------------------------------------------------
def case_context_scenario(path, *, seed, chunk, max_seq, buffer_gb, steps, max_requests, rounder=4):
    from megatron.core.inference.contexts.dynamic_context import (
        ContextOverflowError,
        DynamicInferenceContext as C,
    )

    C.TOKEN_ROUNDER = rounder
    C.REQUEST_ROUNDER = rounder
    cfg = dict(
        num_layers=2,
        kv_channels=8,
        num_attention_heads=2,
        max_sequence_length=max_seq,
        buffer_size_gb=buffer_gb,
        buffer_guaranteed_fraction=0.1,
        chunk_size_tokens=chunk,
        max_requests_override=max_requests,
        max_tokens_override=max_requests * max_seq // 4,
        tensor_model_parallel_size=1,
    )
    ctx = C(params_dtype=torch.float32, **cfg)
    rng = np.random.RandomState(seed)
    out = {}
    events = []
    next_id = 0
    out["init"] = np.array(
        [
            ctx.max_requests,
            ctx.max_tokens,
            ctx.chunk_allocator.chunk_count_total,
            ctx.gtd_chunk_count,
            ctx.gtd_request_count,
            ctx.max_kv_chunk_count,
            ctx.chunk_size_bytes,
        ],
        dtype=np.int64,
    )
    for step in range(steps):
        # admissions
        n_add = int(rng.randint(0, 4)) if step < steps * 2 // 3 else 0
        for _ in range(n_add):
            plen = int(rng.randint(1, max_seq // 2))
            ngen = int(rng.randint(1, max_seq - plen))
            toks = torch.from_numpy(rng.randint(0, 1000, size=plen).astype(np.int64))
            try:
                ctx.add_request(next_id, toks, ngen)
                events.append(["add", step, next_id, plen, ngen, "ok"])
            except ContextOverflowError as e:
                events.append(["add", step, next_id, plen, ngen, type(e).__name__])
            next_id += 1
        if ctx.active_token_count == 0:
            events.append(["idle", step])
            continue
        ctx.initialize_attention_state()
        _snap_ctx(ctx, f"s{step}_", out)
        n_active = ctx.total_request_count - ctx.paused_request_count
        new_tokens = torch.from_numpy(rng.randint(0, 1000, size=n_active).astype(np.int64))
        seq = ctx.get_active_sequence_lengths() + 1
        mx = ctx.get_max_sequence_lengths()
        early = torch.from_numpy((rng.rand(n_active) < 0.05))
        mask = (torch.less(seq, mx) & ~early).byte()
        out[f"s{step}_new_tokens"] = new_tokens.numpy().copy()
        out[f"s{step}_mask"] = mask.numpy().copy()
        newly_paused = ctx.update_requests(mask, new_tokens.clone())
        out[f"s{step}_newly_paused"] = (
            np.zeros(0, dtype=np.int64) if newly_paused is None else newly_paused.numpy().astype(np.int64)
        )
        events.append(["step", step])
    out["meta"] = np.array(json.dumps({"cfg": cfg, "rounder": rounder, "events": events, "seed": seed}))
    np.savez_compressed(path, **out)
    print("wrote", path, "steps", steps, "requests", next_id)


# --------------------------------------------------------------------------------------
# Model decode cases
# --------------------------------------------------------------------------------------
def _build_reference_model(spec):
    from megatron.core.models.gpt.gpt_layer_specs import get_gpt_layer_local_spec
    from megatron.core.models.gpt.gpt_model import GPTModel
    from megatron.core.transformer.transformer_config import TransformerConfig
    from megatron_mixtera_b200.synthetic import canonical_tensor

    dtype = getattr(torch, spec["dtype"])
    kw = dict(
        num_layers=spec["num_layers"],
        hidden_size=spec["hidden_size"],
        num_attention_heads=spec["num_attention_heads"],
        kv_channels=spec["kv_channels"],
        ffn_hidden_size=spec["ffn_hidden_size"],
        use_cpu_initialization=True,
        params_dtype=dtype,
        hidden_dropout=0.0,
        attention_dropout=0.0,
        init_method_std=0.02,
        inference_sampling_seed=0,
        bf16=(dtype == torch.bfloat16),
    )
    if spec["llama"]:
        kw.update(
            num_query_groups=spec["num_query_groups"],
            normalization="RMSNorm",
            gated_linear_unit=True,
            activation_func=torch.nn.functional.silu,
            add_bias_linear=False,
            bias_activation_fusion=True,
        )
    cfg = TransformerConfig(**kw)
    if spec["llama"]:
        m = GPTModel(
            config=cfg,
            transformer_layer_spec=get_gpt_layer_local_spec(normalization="RMSNorm"),
            vocab_size=spec["vocab_size"],
            max_sequence_length=spec["max_sequence_length"],
            parallel_output=True,
            position_embedding_type="rope",
            rotary_base=spec["rotary_base"],
            share_embeddings_and_output_weights=False,
        )
    else:
        m = GPTModel(
            config=cfg,
            transformer_layer_spec=get_gpt_layer_local_spec(),
            vocab_size=spec["vocab_size"],
            max_sequence_length=spec["max_sequence_length"],
            parallel_output=True,
        )
    m = m.eval()
    sd = {}
    for k, v in m.state_dict().items():
        if k.endswith("_extra_state") or v is None:
            continue
        sd[k] = canonical_tensor(k, v.shape, seed=spec["weight_seed"], dtype=dtype)
    missing = m.load_state_dict(sd, strict=False)
    assert not [k for k in missing.missing_keys if not k.endswith("_extra_state")], missing
    return m, sd


def case_model_decode(path, spec):
    from megatron.core.inference.contexts.dynamic_context import DynamicInferenceContext as C
    from megatron.core.inference.model_inference_wrappers.gpt.gpt_inference_wrapper import GPTInferenceWrapper
    from megatron.core.inference.model_inference_wrappers.inference_wrapper_config import InferenceWrapperConfig
    from megatron.core.inference.sampling_params import SamplingParams
    from megatron.core.inference.text_generation_controllers.text_generation_controller import (
        TextGenerationController,
    )

    dtype = getattr(torch, spec["dtype"])
    m, sd = _build_reference_model(spec)
    C.TOKEN_ROUNDER = spec["rounder"]
    C.REQUEST_ROUNDER = spec["rounder"]
    ctx = C(
        params_dtype=dtype,
        num_layers=spec["num_layers"],
        kv_channels=spec["kv_channels"],
        num_attention_heads=spec.get("num_query_groups", spec["num_attention_heads"]),
        max_sequence_length=spec["max_sequence_length"],
        buffer_size_gb=spec["buffer_size_gb"],
        buffer_guaranteed_fraction=0.1,
        chunk_size_tokens=spec["chunk_size_tokens"],
        max_requests_override=spec["max_requests"],
        max_tokens_override=spec["max_tokens"],
        tensor_model_parallel_size=1,
    )
    icfg = InferenceWrapperConfig(
        hidden_size=spec["hidden_size"],
        inference_batch_times_seqlen_threshold=-1,
        fp32_residual_connection=False,
        params_dtype=dtype,
        padded_vocab_size=spec["vocab_size"],
    )
    w = GPTInferenceWrapper(m, icfg, ctx)
    w.model_is_pipeline_parallel = False
    ctl = TextGenerationController(w, types.SimpleNamespace(vocab_size=spec["vocab_size"]))

    g = torch.Generator().manual_seed(spec["prompt_seed"])
    lens = spec["prompt_lengths"]
    prompts = [torch.randint(0, spec["vocab_size"], (n,), generator=g, dtype=torch.int64) for n in lens]
    ngen = spec["num_tokens_to_generate"]
    # Late arrivals: ``arrival_step[i]`` is the step before which request i is added.
    arrival = spec.get("arrival_step", [0] * len(lens))

    out = {}
    state = {"step": 0}
    orig = w.run_one_forward_step

    def hooked(inp):
        _snap_ctx(ctx, f"s{state['step']}_", out)
        logits = orig(inp)
        out[f"s{state['step']}_logits"] = logits.squeeze(0).float().numpy().copy()
        return logits

    w.run_one_forward_step = hooked
    sp = SamplingParams(top_k=1, num_tokens_to_generate=ngen)
    gen = {i: [] for i in range(len(lens))}
    step = 0
    added = 0
    while added < len(lens) or ctx.has_unfinished_requests():
        for i in range(len(lens)):
            if arrival[i] == step:
                ctx.add_request(i, prompts[i], ngen)
                added += 1
        if ctx.active_token_count > 0:
            state["step"] = step
            r = ctl.generate_output_tokens_dynamic_batch(sp, spec.get("termination_id", -1))
            ids = r["active_request_ids"].tolist()
            smp = r["sample"].tolist()
            out[f"s{step}_active_request_ids"] = np.array(ids, dtype=np.int64)
            out[f"s{step}_sample"] = np.array(smp, dtype=np.int64)
            out[f"s{step}_finished_request_ids"] = r["finished_request_ids"].numpy().astype(np.int64)
            for rid, tok in zip(ids, smp):
                gen[rid].append(tok)
        step += 1
        assert step < 10000
    out["num_steps"] = np.array(step)
    for i in range(len(lens)):
        out[f"prompt_{i}"] = prompts[i].numpy()
        out[f"generated_{i}"] = np.array(gen[i], dtype=np.int64)
    # A few rows of the KV pool of request 0 would need its chunk ids after release; instead
    # record a checksum of every weight so that a drifting weight recipe is detected.
    out["weight_checksums"] = np.array(
        json.dumps({k: float(v.double().abs().sum()) for k, v in sd.items()})
    )
    out["meta"] = np.array(json.dumps(spec))
    np.savez_compressed(path, **out)
    print("wrote", path, "steps", step, "gen[0][:8]", gen[0][:8])


C0 = dict(
    llama=False, dtype="float32", num_layers=2, hidden_size=256, num_attention_heads=4, kv_channels=64,
    ffn_hidden_size=1024, vocab_size=1024, max_sequence_length=64, weight_seed=0, prompt_seed=0,
    prompt_lengths=[32, 32, 32, 32], num_tokens_to_generate=16, rounder=4, buffer_size_gb=0.05,
    chunk_size_tokens=16, max_requests=4, max_tokens=256,
)

LLAMA_TINY = dict(
    llama=True, dtype="bfloat16", num_layers=2, hidden_size=512, num_attention_heads=4, num_query_groups=2,
    kv_channels=128, ffn_hidden_size=1024, vocab_size=1024, max_sequence_length=512, rotary_base=500000,
    weight_seed=0, prompt_seed=1, prompt_lengths=[250, 37, 129, 64, 200, 5], num_tokens_to_generate=24,
    arrival_step=[0, 0, 0, 3, 3, 9], rounder=8, buffer_size_gb=0.02, chunk_size_tokens=64,
    max_requests=8, max_tokens=1024,
)


LOG_PROB_CFG = dict(num_layers=2, kv_channels=8, num_attention_heads=2, max_sequence_length=64, buffer_size_gb=0.0002,
                    buffer_guaranteed_fraction=0.1, chunk_size_tokens=16, max_requests_override=8, max_tokens_override=64,
                    tensor_model_parallel_size=1)
LOG_PROB_VOCAB = 48
# (prompt lengths admitted before the step, then the step is taken): a prefill step, a decode step, a mixed step
LOG_PROB_STEPS = [[5, 3], [], [6]]


def case_log_probs(path):
    """The reference context's `calculate_log_probs` (dynamic_context.py:1300-1365) before each `update_requests`: all
    tokens' logits on a prefill step and on a mixed step (per-request lists, prompt tokens shifted by one), last-token
    logits on a decode step and with ``only_last_token_logits``."""
    from megatron.core.inference.contexts.dynamic_context import DynamicInferenceContext as C

    C.TOKEN_ROUNDER = 4
    C.REQUEST_ROUNDER = 4
    ctx = C(params_dtype=torch.float32, **LOG_PROB_CFG)
    gen = torch.Generator().manual_seed(5)
    out, next_id = {}, 0
    for step, prompts in enumerate(LOG_PROB_STEPS):
        for plen in prompts:
            ctx.add_request(next_id, torch.randint(0, LOG_PROB_VOCAB, (plen,), generator=gen), 8)
            next_id += 1
        ctx.initialize_attention_state()
        n_req = ctx.total_request_count - ctx.paused_request_count
        new_tokens = torch.randint(0, LOG_PROB_VOCAB, (n_req,), generator=gen)
        logits = torch.randn(1, ctx.padded_active_token_count, LOG_PROB_VOCAB, generator=gen)
        out[f"s{step}_input_ids"] = ctx.token_to_input_ids[: ctx.active_token_count].numpy().copy()
        out[f"s{step}_new_tokens"] = new_tokens.numpy()
        out[f"s{step}_logits"] = logits.numpy()
        full = ctx.calculate_log_probs(logits, new_tokens)
        out[f"s{step}_lengths"] = np.array([len(x) for x in full], dtype=np.int64)
        out[f"s{step}_log_probs"] = np.array([v for x in full for v in x], dtype=np.float64)
        last = ctx.last_token_logits(logits)
        only_last = ctx.calculate_log_probs(last.unsqueeze(0), new_tokens, only_last_token_logits=True)
        out[f"s{step}_last_log_probs"] = np.array([v for x in only_last for v in x], dtype=np.float64)
        ctx.update_requests(torch.ones(n_req, dtype=torch.uint8), new_tokens.clone())
    np.savez_compressed(path, **out)


SAMPLING_CASES = [  # (top_k, top_p, temperature)
    (1, 0.0, 1.0), (4, 0.0, 1.0), (50, 0.0, 0.7), (0, 0.9, 1.0), (0, 0.5, 1.3), (0, 0.0, 0.8),
]


def case_sampling(path):
    """The reference's `sample_from_logits` (text_generation_controller.py:172-315) on seeded logits: the token of the
    greedy case and, for the others, the probability vector it hands to `torch.multinomial` (captured by wrapping that
    one call; the draw itself is torch's and needs no pin)."""

    from megatron.core.inference.sampling_params import SamplingParams
    from megatron.core.inference.text_generation_controllers.text_generation_controller import TextGenerationController

    gen = torch.Generator().manual_seed(11)
    out = {}
    for dtype in ("float32", "bfloat16"):
        logits = (torch.randn(6, 512, generator=gen) * 3.0).to(getattr(torch, dtype))
        out[f"{dtype}_logits"] = logits.float().numpy()
        stub = types.SimpleNamespace(sampling_rng=torch.Generator().manual_seed(0))
        for i, (top_k, top_p, temperature) in enumerate(SAMPLING_CASES):
            seen = []
            real = torch.multinomial

            def capture(probabilities, num_samples=1, generator=None, _seen=seen):
                _seen.append(probabilities.clone())
                return real(probabilities, num_samples=num_samples, generator=generator)

            torch.multinomial = capture
            try:
                tokens = TextGenerationController.sample_from_logits(
                    stub, logits.clone(), SamplingParams(top_k=top_k, top_p=top_p, temperature=temperature), vocab_size=512)
            finally:
                torch.multinomial = real
            out[f"{dtype}_case{i}_params"] = np.array([top_k, top_p, temperature], dtype=np.float64)
            if top_k == 1:
                assert not seen
                out[f"{dtype}_case{i}_tokens"] = tokens.numpy()
            else:
                out[f"{dtype}_case{i}_probs"] = seen[0].float().numpy()
    np.savez_compressed(path, **out)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", required=True, help="checkout of the reference (the directory that holds megatron/)")
    ap.add_argument("--only", default=None)
    args = ap.parse_args()
    _shim_and_import(args.ref)
    cases = {
        "ctx_scenario_a": lambda p: case_context_scenario(
            p, seed=0, chunk=16, max_seq=128, buffer_gb=0.00016, steps=140, max_requests=16
        ),
        "ctx_scenario_b": lambda p: case_context_scenario(
            p, seed=1, chunk=32, max_seq=256, buffer_gb=0.0006, steps=180, max_requests=24, rounder=8
        ),
        "c0_fp32": lambda p: case_model_decode(p, C0),
        "llama_tiny_bf16": lambda p: case_model_decode(p, LLAMA_TINY),
        "llama_tiny_fp32": lambda p: case_model_decode(p, dict(LLAMA_TINY, dtype="float32")),
        "sampling": case_sampling,
        "log_probs": case_log_probs,
    }
    for name, fn in cases.items():
        if args.only and name != args.only:
            continue
        with torch.inference_mode():
            fn(os.path.join(HERE, name + ".npz"))


if __name__ == "__main__":
    main()
