"""The CPU oracle must reproduce what the reference itself produced (fixtures in tests/golden)."""
import json
import os
import re

import numpy as np
import pytest
import torch

from conftest import GOLDEN
from oracle import decode_oracle as O

CTX_KEYS = [
    "input_ids", "pos_ids", "request_idx", "chunk_idx", "local_pos", "pos_in_request", "request_ids",
    "request_query_lengths", "request_output_lengths", "request_kv_length_offsets", "request_kv_chunk_counts",
    "request_last_kv_chunk_id", "request_last_kv_chunk_offset", "request_to_kv_chunk_ids", "kv_seq_lengths",
    "block_table",
]


def snapshot(c):
    a, pa, t = c.active_token_count, c.padded_active_token_count, c.total_request_count
    d = {
        "counts": np.array([t, c.paused_request_count, a, pa, c.padded_active_request_count,
                            int(c.is_decode_only()), c.chunk_allocator.chunk_count_avail]),
        "input_ids": c.token_to_input_ids[:a], "pos_ids": c.token_to_pos_ids[:a],
        "request_idx": c.token_to_request_idx[:a], "chunk_idx": c.token_to_chunk_idx[:pa],
        "local_pos": c.token_to_local_position_within_kv_chunk[:pa],
        "pos_in_request": c.token_to_position_in_request[:pa],
        "kv_seq_lengths": c.kv_seq_lengths, "block_table": c.block_table,
    }
    for k in CTX_KEYS[6:14]:
        d[k] = getattr(c, k)[:t]
    return d


def check_snapshot(z, step, c):
    d = snapshot(c)
    for k, v in d.items():
        ref = z[f"s{step}_{k}"]
        assert np.array_equal(np.asarray(v).astype(np.int64), ref.astype(np.int64)), (step, k, v, ref)
    avail = c.chunk_allocator.chunk_count_avail
    assert np.array_equal(c.chunk_allocator.chunk_bag[:avail], z[f"s{step}_chunk_bag"][:avail]), step


@pytest.mark.parametrize("name", ["ctx_scenario_a", "ctx_scenario_b"])
def test_context_oracle_matches_reference_scenario(name):
    z = np.load(os.path.join(GOLDEN, name + ".npz"))
    meta = json.loads(str(z["meta"]))
    cfg = meta["cfg"]
    c = O.ContextOracle(dtype_bytes=4, token_rounder=meta["rounder"], request_rounder=meta["rounder"], **cfg)
    init = z["init"]
    assert [c.max_requests, c.max_tokens, c.chunk_count_total, c.gtd_chunk_count, c.gtd_request_count,
            c.max_kv_chunk_count, c.chunk_size_bytes] == init.tolist()
    rng = np.random.RandomState(meta["seed"])
    events = iter(meta["events"])
    # replay the generator's random stream so that prompts / masks are identical
    steps = max(int(m.group(1)) for k in z.files if (m := re.match(r"s(\d+)_counts$", k))) + 1
    total_steps = max(e[1] for e in meta["events"]) + 1
    next_id = 0
    for step in range(total_steps):
        n_add = int(rng.randint(0, 4)) if step < total_steps * 2 // 3 else 0
        for _ in range(n_add):
            plen = int(rng.randint(1, cfg["max_sequence_length"] // 2))
            ngen = int(rng.randint(1, cfg["max_sequence_length"] - plen))
            toks = rng.randint(0, 1000, size=plen).astype(np.int64)
            ev = next(events)
            assert ev[:5] == ["add", step, next_id, plen, ngen]
            try:
                c.add_request(next_id, toks, ngen)
                assert ev[5] == "ok", ev
            except O.OverflowOracle as e:
                assert ev[5].lower().startswith(e.kind.replace("_", "")[:5]), (ev, e.kind)
            next_id += 1
        ev = next(events)
        if c.active_token_count == 0:
            assert ev[0] == "idle"
            continue
        assert ev[0] == "step"
        c.initialize_attention_state()
        check_snapshot(z, step, c)
        n_active = c.total_request_count - c.paused_request_count
        new_tokens = rng.randint(0, 1000, size=n_active).astype(np.int64)
        early = rng.rand(n_active) < 0.05
        assert np.array_equal(new_tokens, z[f"s{step}_new_tokens"])
        mask = z[f"s{step}_mask"]
        seq = c.get_active_sequence_lengths() + 1
        assert np.array_equal(((seq < c.get_max_sequence_lengths()) & ~early).astype(np.uint8), mask)
        newly = c.update_requests(mask, new_tokens)
        ref = z[f"s{step}_newly_paused"]
        got = np.zeros(0, np.int64) if newly is None else newly.astype(np.int64)
        assert np.array_equal(got, ref), step
    assert steps <= total_steps


def _reference_unit_test_context():
    # configuration of the reference's tests/unit_tests/inference/contexts/test_dynamic_context.py:66-87
    return O.ContextOracle(dtype_bytes=4, num_layers=4, kv_channels=8, num_attention_heads=2, max_sequence_length=512,
                           buffer_size_gb=0.03, buffer_guaranteed_fraction=0.1, chunk_size_tokens=128,
                           token_rounder=64, request_rounder=64)


def test_context_oracle_reference_unit_goldens():
    c = _reference_unit_test_context()
    # test_dynamic_context.py:83-87
    assert (c.gtd_chunk_count, c.gtd_request_count, c.chunk_count_total, c.max_requests, c.max_tokens) == (
        48, 12, 491, 128, 62848)
    # :263-279
    assert c.chunk_allocator.allocate(4).tolist() == [486, 487, 488, 489]
    c.chunk_allocator.release(np.array([488, 489]))
    assert c.chunk_allocator.chunk_count_avail == 488
    assert c.chunk_allocator.allocate(1).item() == 489
    assert c.chunk_allocator.allocate(c.chunk_allocator.chunk_count_avail + 100) is None
    # :283-345
    c = _reference_unit_test_context()
    c.add_request(0, np.arange(144))
    assert c.request_to_kv_chunk_ids[0].tolist() == [488, 489, -1, -1]
    assert c.request_last_kv_chunk_offset[0] == 15 and c.request_last_kv_chunk_id[0] == 489
    assert np.all(c.token_to_chunk_idx[:128] == 488) and np.all(c.token_to_chunk_idx[128:144] == 489)


def test_context_oracle_reference_update_requests_golden():
    # test_dynamic_context.py:386-515: paused 0,1; finished 3,7,8; 5,6 cross a chunk boundary
    c = _reference_unit_test_context()
    mask = np.array([1, 0, 1, 1, 1, 0, 0, 1])
    nxt = np.arange(2, 10)
    c.paused_request_count = 2
    c.paused_tokens = np.array([0, 1])
    n = 10
    c.chunk_allocator.chunk_count_avail -= 11
    c.total_request_count = n
    avail = c.chunk_allocator.chunk_count_avail
    c.request_to_kv_chunk_ids[:n, 0] = np.arange(avail, avail + 10)
    c.request_to_kv_chunk_ids[3][1] = avail
    c.request_kv_length_offsets[:n] = 10
    c.request_kv_length_offsets[0:2] = 127
    c.request_kv_length_offsets[5:7] = 127
    c.request_kv_length_offsets[3] = c.chunk_size_bytes + 10
    c.request_query_lengths[:n] = 1
    c.request_ids[:n] = np.arange(n)
    c.request_kv_chunk_counts[:n] = 1
    c.request_kv_chunk_counts[3] = 2
    c.request_last_kv_chunk_id[:n] = np.arange(n)
    c.request_last_kv_chunk_id[3] = 11
    c.request_last_kv_chunk_offset[:n] = 10
    c.request_last_kv_chunk_offset[0:2] = 127
    c.request_last_kv_chunk_offset[5:7] = 127
    c.update_requests(mask, nxt)
    assert (c.paused_request_count, c.total_request_count, c.active_token_count) == (0, 7, 7)
    assert c.request_last_kv_chunk_offset[:10].tolist() == [0, 0, 0, 0, 11, 11, 11, 10, 10, 10]
    assert c.token_to_input_ids[:7].tolist() == [0, 1, 5, 6, 4, 2, 9]
    assert c.token_to_pos_ids[:7].tolist() == [128, 128, 128, 128, 11, 11, 11]
    assert c.request_to_kv_chunk_ids[:10].tolist() == [
        [479, 482, -1, -1], [480, 479, -1, -1], [484, 486, -1, -1], [485, 487, -1, -1], [483, -1, -1, -1],
        [481, -1, -1, -1], [488, -1, -1, -1], [-1, -1, -1, -1], [-1, -1, -1, -1], [-1, -1, -1, -1]]


def build_oracle_model(meta, dtype, fp8=None, kv_fp8_scale=None, tp=1):
    from megatron_mixtera_b200.synthetic import canonical_tensor

    spec = O.ModelSpec(
        num_layers=meta["num_layers"], hidden_size=meta["hidden_size"], num_attention_heads=meta["num_attention_heads"],
        num_query_groups=meta.get("num_query_groups", meta["num_attention_heads"]), kv_channels=meta["kv_channels"],
        ffn_hidden_size=meta["ffn_hidden_size"], vocab_size=meta["vocab_size"],
        max_sequence_length=meta["max_sequence_length"], llama=meta["llama"],
        rotary_base=meta.get("rotary_base", 10000))
    shapes = oracle_weight_shapes(spec)
    w = {k: canonical_tensor(k, s, seed=meta["weight_seed"], dtype=dtype) for k, s in shapes.items()}
    ctx = O.ContextOracle(
        dtype_bytes=1 if kv_fp8_scale is not None else torch.empty(0, dtype=dtype).element_size(), num_layers=spec.num_layers, kv_channels=spec.kv_channels,
        num_attention_heads=spec.num_query_groups, max_sequence_length=spec.max_sequence_length,
        buffer_size_gb=meta["buffer_size_gb"], buffer_guaranteed_fraction=0.1, chunk_size_tokens=meta["chunk_size_tokens"],
        max_requests_override=meta["max_requests"], max_tokens_override=meta["max_tokens"],
        token_rounder=meta["rounder"], request_rounder=meta["rounder"])
    return O.GPTOracle(spec, w, ctx, dtype, fp8=fp8, kv_fp8_scale=kv_fp8_scale, tp=tp), w


def oracle_weight_shapes(s):
    """state_dict keys and full shapes of the reference's local-spec GPTModel."""
    H, F_, d = s.hidden_size, s.ffn_hidden_size, s.kv_channels
    qkv = (s.num_attention_heads + 2 * s.num_query_groups) * d
    sh = {"embedding.word_embeddings.weight": (s.vocab_size, H)}
    if not s.llama:
        sh["embedding.position_embeddings.weight"] = (s.max_sequence_length, H)
    for l in range(s.num_layers):
        p = f"decoder.layers.{l}."
        sh[p + "input_layernorm.weight"] = (H,)
        sh[p + "self_attention.linear_qkv.weight"] = (qkv, H)
        sh[p + "self_attention.linear_proj.weight"] = (H, s.num_attention_heads * d)
        sh[p + "pre_mlp_layernorm.weight"] = (H,)
        sh[p + "mlp.linear_fc1.weight"] = (F_ * (2 if s.llama else 1), H)
        sh[p + "mlp.linear_fc2.weight"] = (H, F_)
        if not s.llama:
            sh[p + "input_layernorm.bias"] = (H,)
            sh[p + "self_attention.linear_qkv.bias"] = (qkv,)
            sh[p + "self_attention.linear_proj.bias"] = (H,)
            sh[p + "pre_mlp_layernorm.bias"] = (H,)
            sh[p + "mlp.linear_fc1.bias"] = (F_,)
            sh[p + "mlp.linear_fc2.bias"] = (H,)
    sh["decoder.final_layernorm.weight"] = (H,)
    if not s.llama:
        sh["decoder.final_layernorm.bias"] = (H,)
    sh["output_layer.weight"] = (s.vocab_size, H)
    return sh


@pytest.mark.parametrize("name", ["c0_fp32", "llama_tiny_fp32", "llama_tiny_bf16"])
def test_model_oracle_matches_reference(name):
    z = np.load(os.path.join(GOLDEN, name + ".npz"))
    meta = json.loads(str(z["meta"]))
    dtype = getattr(torch, meta["dtype"])
    model, w = build_oracle_model(meta, dtype)
    sums = json.loads(str(z["weight_checksums"]))
    assert set(sums) == set(w), set(sums) ^ set(w)
    for k, v in w.items():
        assert abs(float(v.double().abs().sum()) - sums[k]) <= 1e-9 * max(1.0, sums[k]), k
    prompts = [z[f"prompt_{i}"] for i in range(len(meta["prompt_lengths"]))]
    worst = {"rel": 0.0}

    def on_step(step, c, logits, new, ids):
        check_snapshot(z, step, c)
        ref = torch.from_numpy(z[f"s{step}_logits"])
        assert np.array_equal(ids, z[f"s{step}_active_request_ids"])
        rel = float((logits.float() - ref).norm() / ref.norm())
        worst["rel"] = max(worst["rel"], rel)
        assert np.array_equal(new, z[f"s{step}_sample"]), (step, rel)

    with torch.inference_mode():
        gen = O.decode_loop(model, prompts, meta["num_tokens_to_generate"], meta.get("arrival_step"), on_step=on_step)
    for i in range(len(prompts)):
        assert gen[i] == z[f"generated_{i}"].tolist()
    # same torch ops in the same order on the same CPU: bit-identical in practice, 1e-6 allowed
    assert worst["rel"] <= 1e-6, worst


def test_quantisers_roundtrip():
    g = torch.Generator().manual_seed(0)
    x = torch.randn(64, 256, generator=g) * 0.02
    q, e = O.quantize_mxfp8(x)
    xd = O.dequantize_mxfp8(q, e)
    assert float((xd - x).norm() / x.norm()) < 0.04
    # scale choice puts every block's amax into the top binade of E4M3 without saturating
    assert float(q.float().abs().max()) <= 448
    qw, s = O.quantize_fp8_block_weight(x, 128)
    assert float((O.dequantize_fp8_block_weight(qw, s) - x).norm() / x.norm()) < 0.04
    qa, sa = O.quantize_fp8_rowblock(x, 128)
    assert float((O.dequantize_fp8_rowblock(qa, sa) - x).norm() / x.norm()) < 0.04


def test_oracle_tensor_parallel_arithmetic_is_a_small_perturbation():
    # tp=2 rounds the two partial products of every row-parallel linear to bf16 before adding them - the reference's
    # own TP arithmetic.  In fp32 that is exact up to summation order; in bf16 it moves the logits by < 1e-2.
    z = np.load(os.path.join(GOLDEN, "llama_tiny_bf16.npz"))
    meta = json.loads(str(z["meta"]))
    for dtype, bound in ((torch.float32, 1e-5), (torch.bfloat16, 1.2e-2)):
        logits = {}
        for tp in (1, 2):
            model, _ = build_oracle_model(meta, dtype, tp=tp)
            c = model.ctx
            for i in range(2):
                c.add_request(i, z[f"prompt_{i}"], 4)
            c.initialize_attention_state()
            with torch.inference_mode():
                logits[tp] = model.forward().float()
        rel = float((logits[1] - logits[2]).norm() / logits[1].norm())
        assert rel < bound, (dtype, rel)
        assert dtype == torch.float32 or rel > 0  # bf16: the partial roundings are really there


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_sampling_oracle_matches_reference(dtype):
    """`O.sample` / `O.filtered_probabilities` against the reference's `sample_from_logits`: the greedy token and the
    exact probability vector handed to `torch.multinomial` (top-k, top-p with its shift-by-one, plain temperature)."""
    z = np.load(os.path.join(GOLDEN, "sampling.npz"))
    logits = torch.from_numpy(z[f"{dtype}_logits"]).to(getattr(torch, dtype))
    cases = 0
    while f"{dtype}_case{cases}_params" in z.files:
        top_k, top_p, temperature = z[f"{dtype}_case{cases}_params"].tolist()
        if int(top_k) == 1:
            assert np.array_equal(O.sample(logits, top_k=1).numpy(), z[f"{dtype}_case{cases}_tokens"])
        else:
            probs = O.filtered_probabilities(logits, int(top_k), float(top_p), float(temperature))
            ref = z[f"{dtype}_case{cases}_probs"]
            got = probs.float().numpy()
            if np.array_equal(got, ref):
                cases += 1
                continue
            # Only where equal logits straddle the nucleus boundary may the two differ: the reference's sort is not
            # stable, so WHICH of the tied tokens it keeps is arbitrary; the oracle keeps the lower index.  The kept
            # values are the same multiset, and every token whose state differs is tied with one in the opposite state.
            assert dtype == "bfloat16" and top_p > 0, (dtype, cases, np.abs(got - ref).max())
            assert np.array_equal(np.sort(got, axis=1), np.sort(ref, axis=1)), (dtype, cases)
            x = logits.float().numpy()
            for r, c in zip(*np.nonzero((got > 0) != (ref > 0))):
                opposite = ((got[r] > 0) != (got[r, c] > 0)) & (x[r] == x[r, c])
                assert opposite.any(), (dtype, cases, r, c)
        cases += 1
    assert cases == 6
