"""Host bookkeeping of the shipped DynamicInferenceContext against the reference's own fixtures
(bit-exact block tables, KV slots, chunk stack) and the reference's unit-test goldens."""
import json
import os

import numpy as np
import pytest
import torch

from conftest import GOLDEN
from megatron_mixtera_b200.inference.contexts.dynamic_context import (
    ChunkOverflowError,
    ContextOverflowError,
    DynamicInferenceContext,
    MaxSequenceLengthOverflowError,
    RequestOverflowError,
    TokenOverflowError,
)


def set_rounder(v):
    DynamicInferenceContext.TOKEN_ROUNDER = v
    DynamicInferenceContext.REQUEST_ROUNDER = v


@pytest.fixture(autouse=True)
def _restore_rounders():
    yield
    DynamicInferenceContext.TOKEN_ROUNDER = 64
    DynamicInferenceContext.REQUEST_ROUNDER = 4


def make_ctx(**kw):
    base = dict(params_dtype=torch.float32, num_layers=4, kv_channels=8, num_attention_heads=2,
                max_sequence_length=512, buffer_size_gb=0.03, buffer_guaranteed_fraction=0.1, chunk_size_tokens=128,
                tensor_model_parallel_size=1, device="cpu", allocate_memory_buffer=False)
    base.update(kw)
    return DynamicInferenceContext(**base)


def snapshot(c):
    a, pa, t = c.active_token_count, c.padded_active_token_count, c.total_request_count
    d = {
        "counts": np.array([t, c.paused_request_count, a, pa, c.padded_active_request_count, int(c.is_decode_only()),
                            c.chunk_allocator.chunk_count_avail]),
        "input_ids": c.token_to_input_ids[:a], "pos_ids": c.token_to_pos_ids[:a],
        "request_idx": c.token_to_request_idx[:a], "chunk_idx": c.token_to_chunk_idx[:pa],
        "local_pos": c.token_to_local_position_within_kv_chunk[:pa],
        "pos_in_request": c.token_to_position_in_request[:pa],
        "kv_seq_lengths": c.kv_seq_lengths, "block_table": c.block_table,
    }
    for k in ("request_ids", "request_query_lengths", "request_output_lengths", "request_kv_length_offsets",
              "request_kv_chunk_counts", "request_last_kv_chunk_id", "request_last_kv_chunk_offset",
              "request_to_kv_chunk_ids"):
        d[k] = getattr(c, k)[:t]
    return {k: np.asarray(torch.as_tensor(v).cpu()) for k, v in d.items()}


def check_snapshot(z, step, c):
    for k, v in snapshot(c).items():
        ref = z[f"s{step}_{k}"]
        assert np.array_equal(v.astype(np.int64), ref.astype(np.int64)), (step, k, v, ref)
    avail = c.chunk_allocator.chunk_count_avail
    assert np.array_equal(c.chunk_allocator.chunk_bag.numpy()[:avail], z[f"s{step}_chunk_bag"][:avail]), step
    if not c.is_decode_only():
        assert np.array_equal(c.cu_query_seq_lengths.cpu().numpy(), z[f"s{step}_cu_query_seq_lengths"])
        assert np.array_equal(c.cu_kv_seq_lengths.cpu().numpy(), z[f"s{step}_cu_kv_seq_lengths"])
        # the per-token view used by the token-as-row prefill attention
        a = c.active_token_count
        rows = c.token_to_block_table_row[:a].cpu().numpy()
        assert np.array_equal(rows, z[f"s{step}_request_idx"] - c.paused_request_count)
        assert np.array_equal(c.token_kv_lengths[:a].cpu().numpy(), z[f"s{step}_pos_in_request"][:a] + 1)
    assert [c.max_seqlen_q, c.max_seqlen_k] == z[f"s{step}_max_seqlen"].tolist()


@pytest.mark.parametrize("name", ["ctx_scenario_a", "ctx_scenario_b"])
def test_context_matches_reference_scenario(name):
    z = np.load(os.path.join(GOLDEN, name + ".npz"))
    meta = json.loads(str(z["meta"]))
    cfg = meta["cfg"]
    set_rounder(meta["rounder"])
    c = DynamicInferenceContext(params_dtype=torch.float32, device="cpu", allocate_memory_buffer=False, **cfg)
    assert [c.max_requests, c.max_tokens, c.chunk_allocator.chunk_count_total, c.gtd_chunk_count, c.gtd_request_count,
            c.max_kv_chunk_count, c.chunk_size_bytes] == z["init"].tolist()
    rng = np.random.RandomState(meta["seed"])
    events = iter(meta["events"])
    total_steps = max(e[1] for e in meta["events"]) + 1
    names = {"ok": None, "RequestOverflowError": RequestOverflowError, "ChunkOverflowError": ChunkOverflowError,
             "TokenOverflowError": TokenOverflowError}
    next_id = 0
    for step in range(total_steps):
        n_add = int(rng.randint(0, 4)) if step < total_steps * 2 // 3 else 0
        for _ in range(n_add):
            plen = int(rng.randint(1, cfg["max_sequence_length"] // 2))
            ngen = int(rng.randint(1, cfg["max_sequence_length"] - plen))
            toks = torch.from_numpy(rng.randint(0, 1000, size=plen).astype(np.int64))
            ev = next(events)
            assert ev[:5] == ["add", step, next_id, plen, ngen]
            try:
                c.add_request(next_id, toks, ngen)
                assert ev[5] == "ok", ev
            except ContextOverflowError as e:
                assert type(e) is names[ev[5]], (ev, e)
                assert e.is_transient
            next_id += 1
        ev = next(events)
        if c.active_token_count == 0:
            assert ev[0] == "idle"
            continue
        c.initialize_attention_state()
        check_snapshot(z, step, c)
        n_active = c.total_request_count - c.paused_request_count
        new_tokens = rng.randint(0, 1000, size=n_active).astype(np.int64)
        _ = rng.rand(n_active)
        newly = c.update_requests(torch.from_numpy(z[f"s{step}_mask"]), torch.from_numpy(new_tokens))
        got = np.zeros(0, np.int64) if newly is None else newly.numpy().astype(np.int64)
        assert np.array_equal(got, z[f"s{step}_newly_paused"]), step


def test_initialize_dynamic_context():
    # reference tests/unit_tests/inference/contexts/test_dynamic_context.py:66-90
    set_rounder(64)
    c = make_ctx()
    assert c.gtd_chunk_count == 48
    assert c.gtd_request_count == 12
    assert c.chunk_allocator.chunk_count_total == 491
    assert c.max_requests == 128
    assert c.max_tokens == 62848
    assert torch.all(c.request_ids == -1)
    assert not c.is_static_batching()


def test_is_memory_available():
    # :108-133
    c = make_ctx(num_layers=2, kv_channels=64, num_attention_heads=8, buffer_size_gb=1.0)
    c.chunk_allocator.chunk_count_avail = 10
    assert c.chunk_allocator.is_memory_available(10)
    assert not c.chunk_allocator.is_memory_available(11)
    assert c.chunk_allocator.is_memory_available(1)
    c.chunk_allocator.chunk_count_avail = 0
    assert not c.chunk_allocator.is_memory_available(1)
    c.chunk_allocator.chunk_count_avail = 10
    c.chunk_allocator.gtd_chunk_count = 5
    assert c.chunk_allocator.is_memory_available(6)
    assert not c.chunk_allocator.is_memory_available(6, safe=True)


def test_request_overflow():
    # :136-153
    set_rounder(1)
    c = make_ctx(num_layers=2, kv_channels=64, num_attention_heads=8, max_sequence_length=128, buffer_size_gb=0.01,
                 chunk_size_tokens=32)
    with pytest.raises(RequestOverflowError):
        for i in range(c.max_requests + 1):
            c.add_request(i, torch.zeros(10, dtype=torch.int64))


def test_token_overflow_error():
    # :156-178
    set_rounder(1)
    c = make_ctx(num_layers=2, kv_channels=64, num_attention_heads=8, buffer_size_gb=0.1, buffer_overflow_factor=1.0,
                 max_requests_override=2, max_tokens_override=20)
    with pytest.raises(TokenOverflowError):
        c.add_request(1, torch.arange(0, 25))


def test_max_sequence_length_overflow_is_permanent_and_leaks_nothing():
    c = make_ctx()
    avail = c.chunk_allocator.chunk_count_avail
    with pytest.raises(MaxSequenceLengthOverflowError) as e:
        c.add_request(0, torch.arange(0, 500), 100)
    assert not e.value.is_transient
    assert c.chunk_allocator.chunk_count_avail == avail


def test_reset():
    # :181-243
    c = make_ctx(num_layers=2, kv_channels=64, num_attention_heads=8, max_sequence_length=128, buffer_size_gb=1.0)
    c.add_request(0, torch.arange(0, 100), 10)
    c.initialize_attention_state()
    c.total_request_count = 10
    c.active_token_count = 10
    c.paused_request_count = 5
    c.paused_tokens = torch.tensor([1, 2, 3])
    for t in (c.request_ids, c.request_query_lengths, c.request_kv_length_offsets, c.request_kv_chunk_counts,
              c.request_last_kv_chunk_id, c.request_last_kv_chunk_offset, c.request_to_kv_chunk_ids):
        t.fill_(1)
    c.chunk_allocator.chunk_count_avail = 5
    c.reset()
    assert c.total_request_count == 0 and c.active_token_count == 0 and c.paused_request_count == 0
    assert c.padded_active_token_count == 0 and c.padded_active_request_count == 0
    assert c.paused_tokens is None
    assert torch.all(c.request_ids == -1)
    assert torch.all(c.request_query_lengths == 0)
    assert torch.all(c.request_kv_length_offsets == 0)
    assert torch.all(c.request_kv_chunk_counts == 0)
    assert torch.all(c.request_last_kv_chunk_id == -1)
    assert torch.all(c.request_last_kv_chunk_offset == 0)
    assert torch.all(c.token_to_input_ids == 0) and torch.all(c.token_to_pos_ids == 0)
    assert torch.all(c.token_to_request_idx == -1) and torch.all(c.token_to_chunk_idx == -1)
    assert torch.all(c.token_to_position_in_request == 0)
    assert torch.all(c.token_to_local_position_within_kv_chunk == 0)
    assert c.chunk_allocator.chunk_count_avail == c.chunk_allocator.chunk_count_total - 1
    assert torch.all(c.request_to_kv_chunk_ids == -1)


def test_allocate_and_release_memory_chunks():
    # :246-279
    set_rounder(64)
    c = make_ctx()
    assert c.chunk_allocator.allocate_memory_chunks(4).tolist() == [486, 487, 488, 489]
    assert c.chunk_allocator.chunk_count_avail == 486
    c.chunk_allocator.release_memory_chunks(torch.tensor([488, 489]))
    assert c.chunk_allocator.chunk_count_avail == 488
    assert c.chunk_allocator.allocate_memory_chunks(1).item() == 489
    assert c.chunk_allocator.chunk_count_avail == 487
    assert c.chunk_allocator.allocate_memory_chunks(c.chunk_allocator.chunk_count_avail + 100) is None


def test_add_request():
    # :282-345
    set_rounder(64)
    c = make_ctx()
    n = 144
    c.add_request(request_id=0, tokens=torch.arange(0, n, dtype=torch.long))
    assert c.total_request_count == 1 and c.active_token_count == n
    assert c.request_ids[0] == 0 and torch.all(c.request_ids[1:] == -1)
    assert c.request_query_lengths[0] == n and c.request_kv_length_offsets[0] == 0
    assert c.request_to_kv_chunk_ids[0].tolist() == [488, 489, -1, -1]
    assert c.request_kv_chunk_counts[0] == 2 and c.request_last_kv_chunk_id[0] == 489
    assert c.request_last_kv_chunk_offset[0].item() == 15
    ar = torch.arange(0, n, dtype=torch.long)
    assert torch.all(c.token_to_pos_ids[:n] == ar) and torch.all(c.token_to_input_ids[:n] == ar)
    assert torch.all(c.token_to_position_in_request[:n] == ar)
    assert torch.all(c.token_to_chunk_idx[:128] == 488) and torch.all(c.token_to_chunk_idx[128:n] == 489)
    assert torch.all(c.token_to_local_position_within_kv_chunk[:n] == ar % 128)


def test_update_request():
    # :348-515
    set_rounder(64)
    c = make_ctx()
    c.paused_request_count = 0
    c.total_request_count = 3
    c.request_kv_chunk_counts[0:3] = 1
    c.request_to_kv_chunk_ids[0:3, 0] = c.chunk_allocator.allocate_memory_chunks(3, safe=True)
    c.update_requests(active_requests_mask=torch.Tensor([0, 0, 0]), new_tokens=torch.tensor([0, 1, 2]))
    assert c.total_request_count == 0

    c = make_ctx()
    mask = torch.Tensor([1, 0, 1, 1, 1, 0, 0, 1]).int()
    next_tokens = torch.arange(2, 10).int()
    c.paused_request_count = 2
    c.paused_tokens = torch.Tensor([0, 1]).int()
    c.total_request_count = 5
    with pytest.raises(AssertionError):
        c.update_requests(active_requests_mask=mask, new_tokens=next_tokens)
    n = 10
    c.chunk_allocator.chunk_count_avail -= 11
    c.total_request_count = n
    avail = c.chunk_allocator.chunk_count_avail
    c.request_to_kv_chunk_ids[0:n, 0] = torch.arange(avail, avail + 10, dtype=torch.int32)
    c.request_to_kv_chunk_ids[3][1] = avail
    c.request_kv_length_offsets[0:n] = 10
    c.request_kv_length_offsets[0:2] = c.chunk_size_tokens - 1
    c.request_kv_length_offsets[5:7] = c.chunk_size_tokens - 1
    c.request_kv_length_offsets[3] = c.chunk_size_bytes + 10
    c.request_query_lengths[0:n] = 1
    c.request_ids[0:n] = torch.arange(0, n, dtype=torch.int32)
    c.request_kv_chunk_counts[0:n] = 1
    c.request_kv_chunk_counts[3] = 2
    c.request_last_kv_chunk_id[0:n] = torch.arange(0, n, dtype=torch.int32)
    c.request_last_kv_chunk_id[3] = 11
    c.request_last_kv_chunk_offset[0:n] = 10
    c.request_last_kv_chunk_offset[0:2] = c.chunk_size_tokens - 1
    c.request_last_kv_chunk_offset[5:7] = c.chunk_size_tokens - 1
    c.update_requests(active_requests_mask=mask, new_tokens=next_tokens)
    assert c.paused_request_count == 0 and c.total_request_count == 7 and c.active_token_count == 7
    assert c.request_last_kv_chunk_offset[0:10].tolist() == [0, 0, 0, 0, 11, 11, 11, 10, 10, 10]
    assert c.token_to_input_ids[:7].tolist() == [0, 1, 5, 6, 4, 2, 9]
    assert c.token_to_pos_ids[:7].tolist() == [128, 128, 128, 128, 11, 11, 11]
    assert c.request_to_kv_chunk_ids[0:10].tolist() == [
        [479, 482, -1, -1], [480, 479, -1, -1], [484, 486, -1, -1], [485, 487, -1, -1], [483, -1, -1, -1],
        [481, -1, -1, -1], [488, -1, -1, -1], [-1, -1, -1, -1], [-1, -1, -1, -1], [-1, -1, -1, -1]]


def test_release_memory_chunks_for_finished_requests():
    # :517-571 and :573-630
    c = make_ctx()
    chunks = c.chunk_allocator.allocate_memory_chunks(5, safe=True)
    c.total_request_count = 5
    avail0 = c.chunk_allocator.chunk_count_avail
    for i in range(5):
        c.request_to_kv_chunk_ids[i, 0] = chunks[i]
        c.request_query_lengths[i] = 1
        c.request_ids[i] = i
    c.update_requests(torch.tensor([0, 1, 0, 1, 0]), torch.tensor([10, 11, 12, 13, 14]))
    assert c.total_request_count == 2 and c.active_token_count == 2
    assert c.chunk_allocator.chunk_count_avail == avail0 + 3

    c = make_ctx()
    chunks = c.chunk_allocator.allocate_memory_chunks(6, safe=True)
    c.total_request_count = 3
    avail0 = c.chunk_allocator.chunk_count_avail
    c.request_to_kv_chunk_ids[0, 0] = chunks[0]
    c.request_to_kv_chunk_ids[1, :2] = chunks[1:3]
    c.request_to_kv_chunk_ids[2, :3] = chunks[3:6]
    c.request_kv_chunk_counts[:3] = torch.tensor([1, 2, 3], dtype=torch.int32)
    c.request_query_lengths[:3] = 1
    c.request_ids[:3] = torch.arange(3, dtype=torch.int32)
    c.update_requests(torch.tensor([0, 0, 0]), torch.tensor([10, 11, 12]))
    assert c.total_request_count == 0 and c.active_token_count == 0
    assert c.chunk_allocator.chunk_count_avail == avail0 + 6


def test_cuda_graph_token_counts():
    # size tables of the reference's engine tests (tests/unit_tests/inference/engines/test_dynamic_engine.py:496-522)
    set_rounder(4)
    c = make_ctx(max_requests_override=64, num_cuda_graphs=4)
    assert c.cuda_graph_token_counts == [64, 48, 32, 16]
    c = make_ctx(max_requests_override=64, num_cuda_graphs=1)
    assert c.cuda_graph_token_counts == [64]
    c = make_ctx(max_requests_override=60, num_cuda_graphs=16)
    assert c.cuda_graph_token_counts == [60, 56, 48, 40, 32, 24, 16, 8]


def test_prefill_work_list_covers_every_token_once():
    # blocks of `prefill_q_block` consecutive tokens, never across two requests; decode requests are blocks of one
    set_rounder(1)
    ctx = make_ctx()
    ctx.set_prefill_q_block(16)
    lens = [40, 1, 16, 33]
    for i, n in enumerate(lens):
        ctx.add_request(i, torch.arange(n))
    ctx.initialize_attention_state()
    assert not ctx.is_decode_only()
    n_units = ctx.prefill_unit_count
    units = ctx.prefill_units[:n_units].numpy()
    assert n_units == 3 + 1 + 1 + 3
    seen = np.zeros(sum(lens), dtype=int)
    row_of_token = ctx.token_to_block_table_row[: sum(lens)].numpy()
    for row, t0, n, pad in units:
        assert 1 <= n <= 16 and pad == 0
        seen[t0 : t0 + n] += 1
        assert (row_of_token[t0 : t0 + n] == row).all()
    assert (seen == 1).all()
    assert ctx.token_kv_lengths[: sum(lens)].tolist() == [p + 1 for n in lens for p in range(n)]
    # the next step is decode only: no list is built, the old one is not used
    ctx.update_requests(torch.ones(4, dtype=torch.uint8), torch.arange(4))
    ctx.initialize_attention_state()
    assert ctx.is_decode_only()


def test_gate_up_interleave_is_a_permutation_with_an_inverse():
    from megatron_mixtera_b200 import ops

    w = torch.arange(2 * 192 * 3, dtype=torch.float32).view(2 * 192, 3)
    wi = ops.interleave_gate_up(w)
    assert torch.equal(ops.deinterleave_gate_up(wi), w)
    # tile j: gate rows 64j..64j+63, then up rows 64j..64j+63
    assert torch.equal(wi[128:192], w[64:128]) and torch.equal(wi[192:256], w[192 + 64 : 192 + 128])


def test_steady_state_shortcut_of_update_requests_equals_the_general_path():
    # two contexts driven identically, one with the decode shortcut switched off: every host array stays equal
    set_rounder(1)
    a, b = make_ctx(chunk_size_tokens=16, max_sequence_length=96), make_ctx(chunk_size_tokens=16, max_sequence_length=96)
    b.FAST_DECODE_UPDATE = False
    rng = np.random.RandomState(7)
    lens = [5, 17, 30, 9]
    for c in (a, b):
        for i, n in enumerate(lens):
            c.add_request(i, torch.arange(n), 40)
    for step in range(45):
        n = a.total_request_count - a.paused_request_count
        if n == 0:
            break
        toks = rng.randint(0, 100, size=n)
        seq = a.get_active_sequence_lengths() + 1
        mask = torch.less(seq, a.get_max_sequence_lengths()).byte()
        if step == 20:
            mask[0] = 0  # an early finish in the middle
        for c in (a, b):
            c.initialize_attention_state()
            c.update_requests(mask.clone(), torch.from_numpy(toks.copy()))
        for name in ("request_ids", "request_query_lengths", "request_kv_length_offsets", "request_kv_chunk_counts",
                     "request_last_kv_chunk_id", "request_last_kv_chunk_offset", "request_to_kv_chunk_ids", "_h_tok"):
            assert torch.equal(getattr(a, name), getattr(b, name)), (step, name)
        assert (a.total_request_count, a.paused_request_count, a.active_token_count) == (
            b.total_request_count, b.paused_request_count, b.active_token_count)
        assert torch.equal(a.chunk_allocator.chunk_bag, b.chunk_allocator.chunk_bag)


def test_rejected_admission_leaves_the_state_version_alone():
    # A request that does not fit (and is retried by the engine after every step) must not look like a change of the
    # set of requests: the version guards the block table on the device and the forward that is enqueued early.
    set_rounder(1)
    c = make_ctx(num_layers=2, kv_channels=64, num_attention_heads=8, max_sequence_length=128, buffer_size_gb=0.01,
                 chunk_size_tokens=32, max_requests_override=2)
    c.add_request(0, torch.zeros(10, dtype=torch.int64))
    c.add_request(1, torch.zeros(10, dtype=torch.int64))
    v = c.state_version
    for _ in range(3):
        with pytest.raises(RequestOverflowError):
            c.add_request(2, torch.zeros(10, dtype=torch.int64))
        assert c.state_version == v
    c.update_requests(np.array([1, 0], dtype=np.uint8), np.array([7, 8]))  # request 1 finishes: a row is free again
    v = c.state_version
    with pytest.raises(MaxSequenceLengthOverflowError):
        c.add_request(3, torch.zeros(10, dtype=torch.int64), 1000)
    assert c.state_version == v
    c.add_request(2, torch.zeros(10, dtype=torch.int64))
    assert c.state_version == v + 1


def test_debug_validation_accepts_real_steps_and_names_corruptions():
    from megatron_mixtera_b200.inference.contexts.dynamic_context import AttentionStateError

    set_rounder(4)
    c = make_ctx(debug_validate=True, max_requests_override=8, max_tokens_override=600)
    rng = np.random.RandomState(0)
    for i, n in enumerate((130, 5, 127)):
        c.add_request(i, torch.from_numpy(rng.randint(0, 50, size=n)), 40)
    for step in range(12):  # prefill, then decode steps that cross a chunk boundary: every step validates itself
        c.initialize_attention_state()
        n = c.total_request_count - c.paused_request_count
        c.update_requests(np.ones(n, dtype=np.uint8), rng.randint(0, 50, size=n))
    c.initialize_attention_state()
    c.validate_attention_state()

    def corrupted(mutate, match):
        c.initialize_attention_state()
        saved = [a.copy() for a in (c._h_bt_np, c._h_len_np, c._h_tok_np)]
        mutate()
        with pytest.raises(AttentionStateError, match=match):
            c.validate_attention_state()
        for a, b in zip((c._h_bt_np, c._h_len_np, c._h_tok_np), saved):  # (an unchanged block table is not staged again)
            a[...] = b

    corrupted(lambda: c._h_bt_np.__setitem__((0, 0), c.chunk_allocator.chunk_count_total), "chunk id")
    corrupted(lambda: c._h_bt_np.__setitem__((1, 0), -1), "chunk id")
    corrupted(lambda: c._h_len_np.__setitem__((1, 0), c.max_sequence_length + 1), "kv_seq_lengths")
    corrupted(lambda: c._h_len_np.__setitem__((2, 0), c._h_len_np[2, 1]), "permutation")
    corrupted(lambda: c._h_tok_np.__setitem__((5, 0), c.chunk_size_tokens), "KV slot")
    corrupted(lambda: c._h_tok_np.__setitem__((3, 0), c.dummy_chunk_idx), "dummy chunk")
    c.initialize_attention_state()  # a fresh step is clean again


@pytest.mark.parametrize("tp", [1, 2, 4, 8])
def test_checkpoint_shards_merge_back_to_the_full_tensors(tp):
    # the partition rules of the reference (QKV by KV group, gated fc1 as [gate_r ; up_r], row-parallel along the
    # input, vocabulary contiguous): sharding for `tp` ranks and merging the ranks' state dicts is the identity
    from megatron_mixtera_b200.gpt.gpt_model import merge_tensor_parallel_shards, shard_for_rank

    g = torch.Generator().manual_seed(tp)
    H, F, V = 64, 32 * 8, 16 * 8
    full = {
        "embedding.word_embeddings.weight": torch.randn(V, H, generator=g),
        "decoder.layers.0.input_layernorm.weight": torch.randn(H, generator=g),
        "decoder.layers.0.self_attention.linear_qkv.weight": torch.randn(8 * 3 * 16, H, generator=g),
        "decoder.layers.0.self_attention.linear_proj.weight": torch.randn(H, 8 * 16, generator=g),
        "decoder.layers.0.mlp.linear_fc1.weight": torch.randn(2 * F, H, generator=g),
        "decoder.layers.0.mlp.linear_fc2.weight": torch.randn(H, F, generator=g),
        "output_layer.weight": torch.randn(V, H, generator=g),
    }
    shards = [{k: shard_for_rank(k, v, r, tp, gated=True) for k, v in full.items()} for r in range(tp)]
    if tp > 1:
        gate_r = shards[1]["decoder.layers.0.mlp.linear_fc1.weight"][: F // tp]
        assert torch.equal(gate_r, full["decoder.layers.0.mlp.linear_fc1.weight"][F // tp: 2 * F // tp])
    merged = merge_tensor_parallel_shards(shards, gated=True)
    assert set(merged) == set(full)
    for k in full:
        assert torch.equal(merged[k], full[k]), k
    # re-sharding a checkpoint written at another size: merge the `tp` shards, cut for 2 ranks
    again = [shard_for_rank(k, merged[k], 1, 2, gated=True) for k in full]
    direct = [shard_for_rank(k, full[k], 1, 2, gated=True) for k in full]
    assert all(torch.equal(a, b) for a, b in zip(again, direct))


def test_sharded_state_dict_pieces_tile_the_full_tensors():
    # every rank's `sharded_state_dict` says where its pieces sit in the unsharded tensors (a gated fc1: two pieces, the
    # rank's gate rows and its up rows); pasting the pieces of both ranks reproduces the checkpoint
    from megatron_mixtera_b200 import parallel_state
    from megatron_mixtera_b200.gpt.gpt_model import GPTModel
    from megatron_mixtera_b200.synthetic import canonical_tensor
    from megatron_mixtera_b200.transformer.transformer_config import TransformerConfig

    tp = 2
    pasted, full = {}, None
    try:
        for rank in range(tp):
            parallel_state._TP_SIZE, parallel_state._TP_RANK, parallel_state._INITIALIZED = tp, rank, True
            cfg = TransformerConfig(num_layers=1, hidden_size=128, num_attention_heads=4, num_query_groups=2, kv_channels=32,
                                    ffn_hidden_size=256, normalization="RMSNorm", gated_linear_unit=True, activation="silu",
                                    add_bias_linear=False, tensor_model_parallel_size=tp)
            model = GPTModel(cfg, vocab_size=64, max_sequence_length=32, position_embedding_type="rope")
            if full is None:
                full = {k: canonical_tensor(k, s, dtype=torch.bfloat16) for k, s in model.full_parameter_shapes().items()}
            model.load_full_state_dict(full)
            assert model.decoder.layers[0].mlp.linear_fc1._layout_interleaved  # stored rearranged, exported canonical
            for k, pieces in model.sharded_state_dict().items():
                dst = pasted.setdefault(k, torch.zeros(pieces[0].global_shape, dtype=torch.bfloat16))
                assert len(pieces) == (2 if k.endswith("linear_fc1.weight") else 1)
                for pc in pieces:
                    assert pc.global_shape == tuple(full[k].shape)
                    idx = tuple(slice(o, o + n) for o, n in zip(pc.global_offset, pc.data.shape))
                    if pc.replica_id == 0 or rank == 0:
                        dst[idx] = pc.data
    finally:
        parallel_state.destroy_model_parallel()
    assert set(pasted) == set(full)
    for k in full:
        assert torch.equal(pasted[k], full[k]), k


def test_log_probs_match_the_reference_context():
    """`calculate_log_probs` / `last_token_logits` before each `update_requests` of a prefill, a decode and a mixed step
    (fixture: the reference context's own results on the same prompts, logits and sampled tokens)."""
    z = np.load(os.path.join(GOLDEN, "log_probs.npz"))
    set_rounder(4)
    ctx = make_ctx(num_layers=2, max_sequence_length=64, buffer_size_gb=0.0002, chunk_size_tokens=16,
                   max_requests_override=8, max_tokens_override=64)
    gen = torch.Generator().manual_seed(5)
    next_id = 0
    for step, prompts in enumerate([[5, 3], [], [6]]):
        for plen in prompts:
            ctx.add_request(next_id, torch.randint(0, 48, (plen,), generator=gen), 8)
            next_id += 1
        ctx.initialize_attention_state()
        n_req = ctx.total_request_count - ctx.paused_request_count
        new_tokens = torch.randint(0, 48, (n_req,), generator=gen)
        logits = torch.randn(1, ctx.padded_active_token_count, 48, generator=gen)
        assert np.array_equal(ctx.token_to_input_ids[: ctx.active_token_count].numpy(), z[f"s{step}_input_ids"])
        assert np.array_equal(new_tokens.numpy(), z[f"s{step}_new_tokens"]) and np.array_equal(logits.numpy(), z[f"s{step}_logits"])
        full = ctx.calculate_log_probs(logits, new_tokens)
        assert [len(x) for x in full] == z[f"s{step}_lengths"].tolist()
        assert np.array_equal(np.array([v for x in full for v in x]), z[f"s{step}_log_probs"]), step
        last = ctx.last_token_logits(logits)
        only_last = ctx.calculate_log_probs(last.unsqueeze(0), new_tokens, only_last_token_logits=True)
        assert np.array_equal(np.array([v for x in only_last for v in x]), z[f"s{step}_last_log_probs"]), step
        ctx.update_requests(np.ones(n_req, dtype=np.uint8), new_tokens.numpy())
    assert z["s2_lengths"].tolist() == [1, 1, 6]  # the mixed step: two decoding requests and one prompt
