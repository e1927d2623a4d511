"""Kernel-level parity: every C-ABI entry point against the CPU oracle on seeded inputs."""
import math

import numpy as np
import pytest
import torch
import torch.nn.functional as F
from torch.nn.functional import silu as F_silu

from oracle import decode_oracle as O

pytestmark = pytest.mark.gpu

BF16 = torch.bfloat16


@pytest.fixture(scope="module")
def ops():
    from megatron_mixtera_b200 import build, ops as _ops

    build.build()
    yield _ops
    torch.cuda.synchronize()
    assert _ops.device_status() == 0, "a kernel abandoned a bounded wait"


def rel_l2(a, b):
    a, b = a.float().cpu(), b.float().cpu()
    return float((a - b).norm() / b.norm().clamp_min(1e-30))


def randn(shape, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(BF16)


# ------------------------------------------------------------------------------------------
# GEMM
# ------------------------------------------------------------------------------------------
@pytest.mark.parametrize(
    "M,N,K,bias",
    [
        (8, 256, 256, False),      # one tile, BT=32 with zero-filled token rows
        (64, 1024, 512, True),     # split-K (8 tiles only)
        (64, 1000, 576, False),    # ragged N tile, K not a multiple of the split
        (40, 998, 512, True),      # N not a multiple of 4: scalar reduction path
        (33, 384, 1024, True),     # BT=64 with ragged M
        (128, 512, 256, False),    # BT=128
        (300, 640, 512, True),     # BT=256, two token blocks, ragged
        (64, 6144, 4096, False),   # Llama-3-8B QKV projection at decode
        (64, 4096, 14336, False),  # Llama-3-8B fc2 at decode (long K, deep split)
        (16, 20000, 512, False),   # many tiles: no split
        (1, 130, 72, True),        # a single token; K tail inside the first 64-wide block; ragged N
        (256, 128, 4096, False),   # the largest token block, one weight tile, deep split
    ],
)
def test_gemm_matches_fp32_matmul(ops, M, N, K, bias):
    x = randn((M, K), 1)
    w = randn((N, K), 2, 0.05)
    b = randn((N,), 3) if bias else None
    y = ops.gemm(x.cuda(), w.cuda(), None if b is None else b.cuda())
    ref = x.float() @ w.float().t()
    if b is not None:
        ref = ref.to(BF16).float() + b.float()  # layers.py:333-335: bf16 matmul result, then bias add
    assert y.shape == (M, N) and y.dtype == BF16
    err = rel_l2(y, ref)
    assert err < 3e-3, err
    # run again: the split-K tile counters must have been left at zero
    y2 = ops.gemm(x.cuda(), w.cuda(), None if b is None else b.cuda())
    assert torch.equal(y, y2)


def test_gemm_is_deterministic_and_linear(ops):
    # size-independent properties at a full-size shape: repeatability and y(2x) = 2 y(x) exactly
    x = randn((64, 4096), 5).cuda()
    w = randn((4096, 4096), 6, 0.02).cuda()
    y1 = ops.gemm(x, w)
    y2 = ops.gemm(x * 2, w)
    assert torch.equal(ops.gemm(x, w), y1)
    assert torch.equal(y2.float(), y1.float() * 2)


@pytest.mark.parametrize(
    "M,N,K,norm",
    [
        (64, 4096, 4096, "rms"),     # Llama-3-8B out-projection at decode: 8 splits
        (64, 4096, 14336, "rms"),    # fc2: long K
        (33, 1024, 256, "rms"),      # a single split: the partial sums are the whole product
        (16, 1024, 512, "layer"),    # LayerNorm with beta and a linear bias
        (130, 8192, 1024, "rms"),    # two token blocks of 128, widest supported row
        (5, 264, 640, "layer"),      # row not a multiple of 256 elements
    ],
)
def test_splitk_partials_into_add_norm_equal_unfused(ops, M, N, K, norm):
    # the fused pair (GEMM leaves fp32 partial sums, residual-add + norm reduces them) is bit-identical to
    # GEMM -> reduction kernel -> residual-add + norm
    x, w = randn((M, K), 1).cuda(), randn((N, K), 2, 0.05).cuda()
    r = randn((M, N), 3).cuda()
    g = (1 + randn((N,), 4, 0.02).float()).to(BF16).cuda()
    beta = randn((N,), 5, 0.1).cuda() if norm == "layer" else None
    bias = randn((N,), 6).cuda() if norm == "layer" else None
    y = ops.gemm(x, w)
    h_ref, n_ref = ops.add_norm(y, g, bias=bias, residual=r, beta=beta, want_hidden=True)
    p = ops.gemm_splitk(x, w)
    assert p.num_splits >= 1 and p.shape == (M, N)
    h, n = ops.add_norm_splitk(p, g, bias=bias, residual=r, beta=beta, want_hidden=True)
    assert torch.equal(h, h_ref) and torch.equal(n, n_ref)
    # hidden only (the last layer of a model without a final norm)
    p = ops.gemm_splitk(x, w)
    h2, none = ops.add_norm_splitk(p, None, bias=bias, residual=r, want_hidden=True, want_normed=False)
    assert none is None and torch.equal(h2, h_ref)
    assert ops.device_status() == 0


def test_workspace_growth_after_graph_capture_leaves_the_captured_buffer_alive(ops):
    # A captured graph has the split-K workspace address baked in.  A later, larger eager GEMM makes the workspace
    # grow; the old buffer must stay allocated, or replays would write partial sums into memory that the caching
    # allocator has handed to someone else.
    x, w = randn((64, 4096), 1).cuda(), randn((4096, 4096), 2, 0.05).cuda()
    ref = ops.gemm(x, w)  # eager warm-up sizes the workspace for this shape
    torch.cuda.synchronize()
    small = ops._workspace._buf[(x.device.index, "gemm")]
    out = torch.empty_like(ref)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        ops.gemm(x, w, out=out)
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(out, ref)
    big_bytes = small.numel() * 4 + (8 << 20)
    ops._workspace.reserve(x.device, "gemm", big_bytes)  # what an eager prefill GEMM of many rows does
    assert ops._workspace._buf[(x.device.index, "gemm")].numel() >= big_bytes
    assert any(b is small for b in ops._workspace._retired)
    # whatever is allocated now must not land on the old buffer: fill fresh tensors of that size with a pattern
    canaries = [torch.full((small.numel(),), 0x5A, dtype=torch.uint8, device="cuda") for _ in range(4)]
    out.zero_()
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(out, ref)
    for c in canaries:
        assert bool((c == 0x5A).all())


def test_splitk_partials_are_invalidated_by_the_next_gemm(ops):
    x, w = randn((8, 256), 1).cuda(), randn((256, 256), 2, 0.05).cuda()
    g = torch.ones(256, dtype=BF16, device="cuda")
    p = ops.gemm_splitk(x, w)
    ops.gemm(x, w)  # reuses the workspace that holds p
    with pytest.raises(ops.B200Error):
        ops.add_norm_splitk(p, g)


@pytest.mark.parametrize("M,F,K", [(64, 14336, 4096), (8, 10240, 256), (128, 14336, 1024), (200, 19200, 512), (5, 64 * 300, 128)])
def test_fc1_with_swiglu_epilogue_equals_gemm_then_activation(ops, M, F, K):
    # fc1 weight [gate ; up] rearranged per 64 rows; fused kernel, unfused kernels on the rearranged columns and the
    # plain pair on the canonical weight all give the same bits
    x = randn((M, K), 1).cuda()
    w = randn((2 * F, K), 2, 0.05).cuda()
    ref = ops.activation(ops.gemm(x, w), "swiglu")
    wi = ops.interleave_gate_up(w)
    assert torch.equal(ops.deinterleave_gate_up(wi), w)
    assert torch.equal(ops.activation(ops.gemm(x, wi), "swiglu_interleaved"), ref)
    assert ops.gemm_swiglu_supported(M, 2 * F, K)
    out = ops.gemm_swiglu(x, wi)
    assert out.shape == (M, F) and torch.equal(out, ref)
    g, u = torch.chunk(x.float() @ w.float().t(), 2, dim=-1)
    assert rel_l2(out, F_silu(g.to(BF16)).float() * u.to(BF16).float()) < 6e-3
    assert ops.device_status() == 0


def test_fc1_with_swiglu_epilogue_is_refused_for_split_k_shapes(ops):
    M, F, K = 64, 1024, 4096  # 16 output tiles: the GEMM is split along K
    assert not ops.gemm_swiglu_supported(M, 2 * F, K)
    with pytest.raises(ops.B200Error):
        ops.gemm_swiglu(randn((M, K), 1).cuda(), randn((2 * F, K), 2, 0.05).cuda())


def test_gemm_rejects_bad_arguments(ops):
    x = randn((8, 100), 1).cuda()  # K not a multiple of 8
    w = randn((16, 100), 2).cuda()
    with pytest.raises(ops.B200Error):
        ops.gemm(x, w)
    with pytest.raises(ops.B200Error):
        ops.gemm(randn((8, 128), 1), randn((16, 128), 2))  # CPU tensors: no fallback


# ------------------------------------------------------------------------------------------
# Norm / activation / gather
# ------------------------------------------------------------------------------------------
@pytest.mark.parametrize("rows,hidden", [(5, 256), (64, 4096), (3, 8192), (7, 512)])
def test_rmsnorm_with_residual(ops, rows, hidden):
    x, r = randn((rows, hidden), 1), randn((rows, hidden), 2)
    g = (1 + randn((hidden,), 3, 0.02).float()).to(BF16)
    h, y = ops.add_norm(x.cuda(), g.cuda(), residual=r.cuda(), want_hidden=True)
    h_ref = x + r
    y_ref = F.rms_norm(h_ref, (hidden,), g, 1e-5)
    assert torch.equal(h.cpu(), h_ref)
    mism = (y.cpu() != y_ref).float().mean().item()
    assert mism < 2e-3 and rel_l2(y, y_ref) < 1e-3, (mism, rel_l2(y, y_ref))
    _, y0 = ops.add_norm(x.cuda(), g.cuda())
    assert rel_l2(y0, F.rms_norm(x, (hidden,), g, 1e-5)) < 1e-3


def test_layernorm_with_bias_and_residual(ops):
    rows, hidden = 9, 256
    x, r, b = randn((rows, hidden), 1), randn((rows, hidden), 2), randn((hidden,), 3, 0.1)
    g, beta = (1 + randn((hidden,), 4, 0.02).float()).to(BF16), randn((hidden,), 5, 0.1)
    h, y = ops.add_norm(x.cuda(), g.cuda(), bias=b.cuda(), residual=r.cuda(), beta=beta.cuda(), want_hidden=True)
    h_ref = (x + b) + r
    assert torch.equal(h.cpu(), h_ref)
    assert rel_l2(y, F.layer_norm(h_ref, (hidden,), g, beta, 1e-5)) < 2e-3


def test_swiglu_and_gelu(ops):
    x = randn((17, 2 * 1024), 1, 2.0)
    y = ops.activation(x.cuda(), "swiglu")
    a, b = torch.chunk(x, 2, dim=-1)
    ref = F.silu(a) * b
    assert (y.cpu() != ref).float().mean().item() < 2e-3 and rel_l2(y, ref) < 1e-3
    x = randn((17, 1024), 2, 2.0)
    bias = randn((1024,), 3, 0.1)
    y = ops.activation(x.cuda(), "gelu", bias.cuda())
    assert rel_l2(y, F.gelu(x + bias)) < 2e-3


def test_gather_rows(ops):
    table = randn((100, 256), 1)
    pos = randn((64, 256), 2)
    ids = torch.tensor([0, 99, 5, 5, 42, 77], dtype=torch.int64)
    pid = torch.tensor([0, 1, 2, 3, 63, 10], dtype=torch.int64)
    assert torch.equal(ops.gather_rows(table.cuda(), ids.cuda()).cpu(), table[ids])
    out = ops.gather_rows(table.cuda(), ids.cuda(), add_table=pos.cuda(), add_ids=pid.cuda())
    assert torch.equal(out.cpu(), table[ids] + pos[pid])
    # vocab shard [40, 80): ids outside give zero rows (layers.py:262-295)
    out = ops.gather_rows(table[40:80].contiguous().cuda(), ids.cuda(), vocab_start=40, vocab_end=80)
    ref = torch.zeros(6, 256, dtype=BF16)
    ref[4], ref[5] = table[42], table[77]
    assert torch.equal(out.cpu(), ref)


# ------------------------------------------------------------------------------------------
# Sampling
# ------------------------------------------------------------------------------------------
def test_argmax_ties_pick_first(ops):
    g = torch.Generator().manual_seed(0)
    logits = torch.randn((9, 128256), generator=g).to(BF16)
    logits[0, 1000] = logits[0, 77000] = 50.0   # tie: the smaller index wins
    logits[1, :] = 0.0                           # all equal
    logits[2, -1] = 60.0                         # last element
    got = ops.argmax(logits.cuda()).cpu()
    assert got.tolist() == torch.argmax(logits.float(), dim=-1).tolist()
    assert got[0] == 1000 and got[1] == 0 and got[2] == 128255
    # strided rows (a slice of padded logits)
    wide = torch.randn((4, 1100), generator=g).to(BF16).cuda()
    assert ops.argmax(wide[:, :1000].contiguous()).tolist() == torch.argmax(wide[:, :1000].float(), -1).tolist()


@pytest.mark.parametrize("top_k,temperature", [(2, 1.0), (40, 0.7), (1000, 1.3)])
def test_topk_probabilities(ops, top_k, temperature):
    g = torch.Generator().manual_seed(1)
    logits = (torch.randn((5, 32000), generator=g) * 3).to(BF16)
    probs = ops.topk_probs(logits.cuda(), top_k, temperature).cpu()
    ref = O.filtered_probabilities(logits, top_k, 0.0, temperature, softmax_dtype=torch.float32)
    assert torch.equal(probs > 0, ref > 0)  # exact support
    assert int((ref > 0).sum(-1).min()) >= top_k
    assert float((probs - ref).abs().max()) < 1e-5
    # and within bf16 rounding of what the reference hands to multinomial
    assert float((probs - O.filtered_probabilities(logits, top_k, 0.0, temperature).float()).abs().max()) < 2.5e-3
    assert torch.allclose(probs.sum(-1), torch.ones(5), atol=1e-4)


def _nucleus_reference(x_bf16, top_p):
    """Oracle probabilities (fp32 restatement of the reference's sort / cumsum / shift rule) and, per token, the
    mass strictly ahead of it in float64 - the quantity the keep decision compares with top_p."""
    ref = O.filtered_probabilities(x_bf16.float(), 0, top_p, 1.0)
    sl, si = torch.sort(x_bf16.double(), descending=True, stable=True)
    excl = sl.softmax(-1).cumsum(-1) - sl.softmax(-1)
    ahead = torch.empty_like(excl).scatter_(1, si, excl)
    return ref, ahead


@pytest.mark.parametrize("vocab", [1000, 32000, 128256])
@pytest.mark.parametrize("top_p,temperature", [(0.1, 1.0), (0.5, 0.7), (0.9, 1.0), (0.97, 1.3), (1.0, 1.0)])
def test_topp_probabilities(ops, vocab, top_p, temperature):
    g = torch.Generator().manual_seed(2)
    logits = (torch.randn((6, vocab), generator=g) * 3).to(BF16)
    logits[5] = (logits[5] * 2).round() / 2  # a row with few distinct values: many ties around the cut
    probs = ops.topp_probs(logits.cuda(), top_p, temperature).cpu()
    x = logits.clone()
    if temperature != 1.0:
        x.div_(temperature)  # in bf16, like the reference's in-place division
    ref, ahead = _nucleus_reference(x, top_p)
    assert torch.allclose(probs.sum(-1), torch.ones(6), atol=1e-4)
    if top_p == 1.0:
        # In exact arithmetic nothing is filtered.  (The fp32 restatement drops a tail whose cumulative sum rounds
        # above 1.0; what it drops carries no mass.)
        assert float((probs - x.float().softmax(-1)).abs().max()) < 1e-6
        assert float(probs[ref == 0].sum()) < 1e-4
        return
    differ = (probs > 0) != (ref > 0)
    # a keep/drop decision may only differ where the mass ahead of the token equals top_p to the rounding of an
    # fp32 sum over the row (ours and the restatement's own): a few 1e-6 at 128 k entries
    # (in a flat 128 k row that band can hold a hundred tokens of 1e-7 each, so their number is not bounded here)
    assert bool(((ahead[differ] - top_p).abs() < 5e-5).all()), (int(differ.sum()), ahead[differ])
    assert bool((probs > 0)[torch.arange(6), x.float().argmax(-1)].all())  # the top token always survives
    # a token that flips at the cut of a 128 k row carries ~1e-5 of mass, so the vectors agree everywhere to 1e-4;
    # rows whose support is identical agree to fp32 rounding
    assert float((probs - ref).abs().max()) < 1e-4
    same = ~differ.any(-1)
    if bool(same.any()):
        assert float((probs[same] - ref[same]).abs().max()) < 1e-5


def test_topp_equal_logits_keep_the_lowest_indices(ops):
    # all tokens tie: the kept ones are the first floor(top_p / p) + 1 by index
    logits = torch.full((2, 1000), 1.5).to(BF16)
    probs = ops.topp_probs(logits.cuda(), 0.2995, 1.0).cpu()
    assert int((probs > 0).sum(-1)[0]) == 300 and bool((probs[:, :300] > 0).all()) and bool((probs[:, 300:] == 0).all())
    assert torch.allclose(probs[:, :300], torch.full((2, 300), 1 / 300), atol=1e-7)
    # one dominant token: it alone survives whatever top_p is
    logits[:, 7] = 40.0
    probs = ops.topp_probs(logits.cuda(), 0.9, 1.0).cpu()
    assert bool((probs[:, 7] == 1).all()) and int((probs > 0).sum()) == 2
    with pytest.raises(ops.B200Error):
        ops.topp_probs(logits.cuda(), 0.0, 1.0)


# ------------------------------------------------------------------------------------------
# Paged attention
# ------------------------------------------------------------------------------------------
def make_paged_case(*, T, nkv, G, D, chunk, kv_lens, seed, rope=True, max_pos=None):
    """Random pool + block tables with shuffled chunk ids; the last token of every row is 'new'."""
    g = torch.Generator().manual_seed(seed)
    nq = nkv * G
    max_chunks = max(1, max(math.ceil(k / chunk) for k in kv_lens)) + 1
    n_chunks = sum(math.ceil(k / chunk) for k in kv_lens) + 3
    perm = torch.randperm(n_chunks - 1, generator=g).tolist()  # last chunk = dummy
    k_cache = (torch.randn((n_chunks, chunk, nkv, D), generator=g)).to(BF16)
    v_cache = (torch.randn((n_chunks, chunk, nkv, D), generator=g)).to(BF16)
    block_table = torch.zeros((T, max_chunks), dtype=torch.int32)
    chunk_idx = torch.full((T,), n_chunks - 1, dtype=torch.int64)
    local = torch.zeros((T,), dtype=torch.int64)
    pos = torch.zeros((T,), dtype=torch.int64)
    it = iter(perm)
    for r, kl in enumerate(kv_lens):
        nb = math.ceil(kl / chunk)
        ids = [next(it) for _ in range(nb)]
        block_table[r, :nb] = torch.tensor(ids, dtype=torch.int32)
        if kl > 0:
            chunk_idx[r] = ids[(kl - 1) // chunk]
            local[r] = (kl - 1) % chunk
            pos[r] = kl - 1
    qkv = torch.randn((T, nkv, (G + 2) * D), generator=g).to(BF16)
    max_pos = max_pos or (max(kv_lens) + 1)
    freqs = O.rope_freqs(max_pos, D, 500000.0) if rope else None
    return dict(T=T, nkv=nkv, G=G, D=D, nq=nq, chunk=chunk, kv_lens=torch.tensor(kv_lens, dtype=torch.int32),
                k_cache=k_cache, v_cache=v_cache, block_table=block_table, chunk_idx=chunk_idx, local=local, pos=pos,
                qkv=qkv, freqs=freqs)


def oracle_decode_attention(c):
    """dynamic_context.py:511-631 + attention.py:588-600 restated: rope, append, paged attention."""
    T, nkv, G, D = c["T"], c["nkv"], c["G"], c["D"]
    qkv = c["qkv"]
    q = qkv[..., : G * D].reshape(T, nkv * G, D)
    k = qkv[..., G * D : (G + 1) * D]
    v = qkv[..., (G + 1) * D :]
    if c["freqs"] is not None:
        k = O.apply_rope(k, c["freqs"][c["pos"]])
        q = O.apply_rope(q, c["freqs"][c["pos"]])
    kc, vc = c["k_cache"].clone(), c["v_cache"].clone()
    kc[c["chunk_idx"], c["local"]] = k
    vc[c["chunk_idx"], c["local"]] = v
    out = O.paged_attention(q, kc, vc, c["kv_lens"], c["block_table"].numpy())
    return out, kc, vc


def run_cuda_attention(ops, c, *, num_splits, fused, row_of_token=None, row_order=None, qkv_from=None, out_quantized=None):
    dev = "cuda"
    D = c["D"]
    cos = sin = None
    if c["freqs"] is not None:
        half = c["freqs"][:, : D // 2]
        cos, sin = torch.cos(half).to(BF16).to(dev), torch.sin(half).to(BF16).to(dev)
    kc, vc = c["k_cache"].clone().to(dev), c["v_cache"].clone().to(dev)
    out = torch.full((c["T"], c["nq"] * D), float("nan"), dtype=BF16, device=dev)
    # the argument struct holds raw pointers only: keep every device tensor alive in `d`
    d = {k: c[k].to(dev) for k in ("qkv", "block_table", "kv_lens", "pos", "chunk_idx", "local")}
    d["row"] = None if row_of_token is None else row_of_token.to(dev)
    d["order"] = None if row_order is None else row_order.to(dev)
    if qkv_from is not None:  # (x, w): the QKV GEMM's un-reduced split-K partial sums instead of its bf16 output
        d["qkv"] = ops.gemm_splitk(*qkv_from)
    args = ops.make_attention_args(
        qkv=d["qkv"], k_cache=kc, v_cache=vc, block_table=d["block_table"], kv_seq_lengths=d["kv_lens"], out=out,
        num_q_heads=c["nq"], num_kv_heads=c["nkv"], head_dim=D, chunk_size=c["chunk"], token_to_pos_ids=d["pos"],
        token_to_pos_in_request=d["pos"], token_to_chunk_idx=d["chunk_idx"], token_to_local_pos=d["local"],
        rope_cos=cos, rope_sin=sin, num_splits=num_splits, fuse_rope_append=fused, row_of_token=d["row"], row_order=d["order"],
        out_quantized=out_quantized)
    if not fused:
        ops.rope_append(args)
    ops.paged_attention(args)
    torch.cuda.synchronize()
    return out.cpu().view(c["T"], c["nq"], D), kc.cpu(), vc.cpu()


@pytest.mark.parametrize("nkv,G,D,chunk,kv_lens,splits", [
    (2, 4, 128, 64, [1, 64, 65, 130, 0, 300, 17, 256], 1),
    (2, 4, 128, 64, [1, 64, 65, 130, 0, 300, 17, 256], 4),
    (8, 4, 128, 256, [2304, 128, 700, 1216, 0, 0], 4),
    (4, 2, 64, 64, [33, 200, 64, 0], 1),
    (4, 2, 64, 64, [33, 200, 64, 0], 2),
])
@pytest.mark.parametrize("recipe", ["mxfp8", "blockwise"])
def test_decode_attention_writes_quantised_output(ops, nkv, G, D, chunk, kv_lens, splits, recipe):
    # the kernel that finishes an output row quantises it for the out-projection: same bytes and scales as the
    # stand-alone quantiser applied to the kernel's bf16 output
    if recipe == "blockwise" and D != 128:
        pytest.skip("the 128-block recipe takes one scale per head of 128 dims")
    T = len(kv_lens)
    c = make_paged_case(T=T, nkv=nkv, G=G, D=D, chunk=chunk, kv_lens=kv_lens, seed=21)
    out, _, _ = run_cuda_attention(ops, c, num_splits=splits, fused=True)
    width = c["nq"] * D
    ref_in = out.reshape(T, width).cuda()
    ref = ops.quantize_mxfp8(ref_in) if recipe == "mxfp8" else ops.quantize_fp8_rowblock(ref_in)
    got = ops.quantized_like(recipe, T, width, "cuda")
    got.q.fill_(0x7F)
    nan_out, _, _ = run_cuda_attention(ops, c, num_splits=splits, fused=True, out_quantized=got)
    assert torch.isnan(nan_out.float()).all()  # the bf16 output was not written
    assert torch.equal(got.q[:T].cpu(), ref.q[:T].cpu())
    if recipe == "mxfp8":
        r = torch.arange(T)[:, None]
        b = torch.arange(width // 32)[None, :]
        idx = ((r // 128) * (width // 128) * 512 + (b // 4) * 512 + (r % 32) * 16 + ((r % 128) // 32) * 4 + (b % 4)).reshape(-1)
        assert torch.equal(got.sf.cpu()[idx], ref.sf.cpu()[idx])
    else:
        assert torch.equal(got.scale[:, :T].cpu(), ref.scale[:, :T].cpu())


@pytest.mark.parametrize(
    "nkv,G,D,chunk,kv_lens,splits",
    [
        (2, 4, 128, 64, [1, 64, 65, 130, 0, 300, 17, 256], 1),
        (2, 4, 128, 64, [1, 64, 65, 130, 0, 300, 17, 256], 4),
        (1, 8, 128, 256, [1000, 257, 512, 3], 3),
        (8, 4, 128, 256, [2304, 128, 700, 1216, 0, 0], 4),     # Llama-3-8B head geometry
        (4, 1, 64, 64, [33, 200, 64], 2),                       # MHA, head dim 64
        (2, 2, 64, 128, [129, 5], 1),
        (1, 16, 128, 64, [70, 1, 640], 2),                      # the widest group the kernel takes (16 query heads)
        (3, 3, 64, 64, [5, 0, 191, 64], 1),                     # odd group size, three KV heads
    ],
)
@pytest.mark.parametrize("fused", [True, False])
def test_paged_decode_attention(ops, nkv, G, D, chunk, kv_lens, splits, fused):
    c = make_paged_case(T=len(kv_lens), nkv=nkv, G=G, D=D, chunk=chunk, kv_lens=kv_lens, seed=11)
    ref, kc_ref, vc_ref = oracle_decode_attention(c)
    out, kc, vc = run_cuda_attention(ops, c, num_splits=splits, fused=fused)
    # KV-slot indexing and contents: bit-exact (bf16 RoPE rounding points reproduced)
    live = [r for r, kl in enumerate(kv_lens) if kl > 0]
    for r in live:
        ci, lp = int(c["chunk_idx"][r]), int(c["local"][r])
        assert torch.equal(kc[ci, lp], kc_ref[ci, lp]), r
        assert torch.equal(vc[ci, lp], vc_ref[ci, lp]), r
    if fused:
        # nothing but the new slots was written
        mask = torch.ones(kc.shape[:2], dtype=torch.bool)
        mask[c["chunk_idx"][live], c["local"][live]] = False
        assert torch.equal(kc[mask], c["k_cache"][mask]) and torch.equal(vc[mask], c["v_cache"][mask])
    assert not torch.isnan(out.float()).any()
    for r, kl in enumerate(kv_lens):
        if kl == 0:
            assert torch.all(out[r] == 0)
    # P is carried as hi + lo bf16 terms: close to an fp32 softmax, far inside flash-attn's own bf16-P error
    err = rel_l2(out, ref)
    assert err < 1.5e-3, err


def test_paged_attention_prefill_rows_via_row_of_token(ops):
    # One request of 70 prompt tokens processed as 70 rows sharing block-table row 1: row t sees t+1 keys.
    nkv, G, D, chunk, n = 2, 4, 128, 64, 70
    c = make_paged_case(T=n, nkv=nkv, G=G, D=D, chunk=chunk, kv_lens=[n] * n, seed=3, max_pos=128)
    ids = c["block_table"][0].clone()
    c["block_table"] = torch.stack([torch.zeros_like(ids), ids])
    pos = torch.arange(n, dtype=torch.int64)
    c["pos"], c["local"] = pos, pos % chunk
    c["chunk_idx"] = ids[(pos // chunk)].long()
    c["kv_lens"] = (pos + 1).int()
    row_of_token = torch.ones(n, dtype=torch.int32)
    out, kc, vc = run_cuda_attention(ops, c, num_splits=2, fused=False, row_of_token=row_of_token)
    # oracle: same thing expressed as one varlen request (cu_q = [0, n]) over block-table row 1
    T = n
    qkv = c["qkv"]
    q = O.apply_rope(qkv[..., : G * D].reshape(T, nkv * G, D), c["freqs"][pos])
    k = O.apply_rope(qkv[..., G * D : (G + 1) * D], c["freqs"][pos])
    kc_ref, vc_ref = c["k_cache"].clone(), c["v_cache"].clone()
    kc_ref[c["chunk_idx"], c["local"]] = k
    vc_ref[c["chunk_idx"], c["local"]] = qkv[..., (G + 1) * D :]
    ref = O.paged_attention(q, kc_ref, vc_ref, torch.tensor([n]), c["block_table"][1:2].numpy(),
                            cu_q=torch.tensor([0, n]))
    assert torch.equal(kc, kc_ref) and torch.equal(vc, vc_ref)
    assert rel_l2(out, ref) < 5e-3


@pytest.mark.parametrize("nkv,G,D", [(2, 4, 128), (1, 8, 128), (2, 1, 64), (1, 16, 64), (2, 2, 128)])
def test_paged_prefill_attention_mixed_step(ops, nkv, G, D):
    # A mixed step: request 0 prefills 70 tokens, request 1 decodes one token on a context of 37, request 2
    # prefills 150 tokens.  The prefill kernel (blocks of 64 / G query tokens share the K/V tiles) must agree with
    # the oracle and with the one-CTA-per-token path.
    chunk = 64
    q_lens, kv_total = [70, 1, 150], [70, 38, 150]
    c = make_paged_case(T=3, nkv=nkv, G=G, D=D, chunk=chunk, kv_lens=kv_total, seed=21, max_pos=256)
    bt = c["block_table"]
    row_of_token = torch.cat([torch.full((n,), r, dtype=torch.int32) for r, n in enumerate(q_lens)])
    pos = torch.cat([torch.arange(kv - n, kv, dtype=torch.int64) for n, kv in zip(q_lens, kv_total)])
    T = int(row_of_token.numel())
    g = torch.Generator().manual_seed(22)
    c.update(T=T, qkv=torch.randn((T, nkv, (G + 2) * D), generator=g).to(BF16), pos=pos, local=pos % chunk,
             chunk_idx=bt[row_of_token.long(), (pos // chunk)].long(), kv_lens=(pos + 1).int())
    ref_rows, kc_ref, vc_ref = run_cuda_attention(ops, c, num_splits=1, fused=False, row_of_token=row_of_token)

    qb = 64 // G
    units, t0 = [], 0
    for r, n in enumerate(q_lens):
        units += [(r, t0 + b, min(qb, n - b), 0) for b in range(0, n, qb)]
        t0 += n
    units += [(0, 0, 0, 0)] * 3  # padding entries are skipped
    dev = "cuda"
    half = c["freqs"][:, : D // 2]
    d = {k: c[k].to(dev) for k in ("qkv", "block_table", "kv_lens", "pos", "chunk_idx", "local")}
    d.update(kc=c["k_cache"].clone().to(dev), vc=c["v_cache"].clone().to(dev), row=row_of_token.to(dev),
             cos=torch.cos(half).to(BF16).to(dev), sin=torch.sin(half).to(BF16).to(dev),
             units=torch.tensor(units, dtype=torch.int32, device=dev),
             out=torch.full((T, c["nq"] * D), float("nan"), dtype=BF16, device=dev))
    args = ops.make_attention_args(
        qkv=d["qkv"], k_cache=d["kc"], v_cache=d["vc"], block_table=d["block_table"], kv_seq_lengths=d["kv_lens"],
        out=d["out"], num_q_heads=c["nq"], num_kv_heads=nkv, head_dim=D, chunk_size=chunk, token_to_pos_ids=d["pos"],
        token_to_pos_in_request=d["pos"], token_to_chunk_idx=d["chunk_idx"], token_to_local_pos=d["local"],
        rope_cos=d["cos"], rope_sin=d["sin"], num_splits=1, fuse_rope_append=False, row_of_token=d["row"])
    assert ops.prefill_q_block(c["nq"], nkv) == qb
    ops.rope_append(args)
    ops.paged_prefill_attention(args, d["units"], len(units))
    torch.cuda.synchronize()
    out = d["out"].cpu().view(T, c["nq"], D)
    assert not torch.isnan(out.float()).any()  # every token belongs to a unit
    assert torch.equal(d["kc"].cpu(), kc_ref) and torch.equal(d["vc"].cpu(), vc_ref)
    assert rel_l2(out, ref_rows) < 2e-3  # same arithmetic, different summation order

    q = O.apply_rope(c["qkv"][..., : G * D].reshape(T, nkv * G, D), c["freqs"][pos])
    cu_q = torch.tensor([0, 70, 71, 221])
    ref = O.paged_attention(q, kc_ref, vc_ref, torch.tensor(kv_total), bt.numpy(), cu_q=cu_q)
    assert rel_l2(out, ref) < 5e-3
    assert ops.device_status() == 0


@pytest.mark.parametrize("nkv,G,D,K", [(8, 4, 128, 4096), (2, 8, 128, 512), (4, 1, 64, 1024)])
@pytest.mark.parametrize("splits", [1, 2])
def test_decode_attention_reads_qkv_split_k_partials(ops, nkv, G, D, K, splits):
    # the decode kernel sums the QKV GEMM's partial sums itself: same output, same pool as with the reduced bf16 qkv
    kv_lens = [300, 1, 64, 129, 0, 77]
    T = len(kv_lens)
    c = make_paged_case(T=T, nkv=nkv, G=G, D=D, chunk=64, kv_lens=kv_lens, seed=31)
    x = randn((T, K), 32).cuda()
    w = randn((nkv * (G + 2) * D, K), 33, 0.05).cuda()
    c["qkv"] = ops.gemm(x, w).view(T, nkv, (G + 2) * D).cpu()
    base = run_cuda_attention(ops, c, num_splits=splits, fused=True)
    got = run_cuda_attention(ops, c, num_splits=splits, fused=True, qkv_from=(x, w))
    for a, b in zip(got, base):
        assert torch.equal(torch.nan_to_num(a.float()), torch.nan_to_num(b.float()))
    assert ops.device_status() == 0


@pytest.mark.parametrize("splits", [1, 3])
def test_attention_row_order_changes_nothing(ops, splits):
    # the order in which rows are started is a scheduling hint: outputs and pool are bit-identical
    kv_lens = [5, 700, 64, 1, 1300, 257, 0, 90]
    c = make_paged_case(T=8, nkv=2, G=4, D=128, chunk=64, kv_lens=kv_lens, seed=11)
    base = run_cuda_attention(ops, c, num_splits=splits, fused=True)
    order = torch.argsort(-torch.tensor(kv_lens), stable=True).int()
    for ro in (order, order.flip(0)):
        got = run_cuda_attention(ops, c, num_splits=splits, fused=True, row_order=ro)
        for a, b in zip(got, base):
            assert torch.equal(torch.nan_to_num(a.float()), torch.nan_to_num(b.float()))
    # an entry outside 0..T-1 is skipped, never used as an index
    bad = order.clone()
    bad[0] = 1000
    run_cuda_attention(ops, c, num_splits=splits, fused=True, row_order=bad)
    assert ops.device_status() == 0


def test_attention_split_invariance_at_long_context(ops):
    # size-independent property at a long context: the result does not depend on the split count
    kv_lens = [32768 + 77, 9000]
    c = make_paged_case(T=2, nkv=1, G=4, D=128, chunk=256, kv_lens=kv_lens, seed=5)
    o1, _, _ = run_cuda_attention(ops, c, num_splits=1, fused=True)
    o16, _, _ = run_cuda_attention(ops, c, num_splits=16, fused=True)
    assert rel_l2(o16, o1) < 4e-3  # two bf16 roundings of outputs that differ only in summation order
    ref, _, _ = oracle_decode_attention(c)
    assert rel_l2(o16, ref) < 5e-3


# ------------------------------------------------------------------------------------------
# FP8 (E4M3) KV pool with one scale per KV head (an extension beyond the reference)
# ------------------------------------------------------------------------------------------
@pytest.mark.parametrize(
    "nkv,G,chunk,kv_lens,splits",
    [(2, 4, 128, [1, 64, 65, 130, 0, 300, 17, 256, 128, 129], 1), (2, 4, 128, [1, 64, 65, 130, 0, 300, 17, 256], 3),
     (8, 4, 256, [2304, 128, 700, 1216, 0], 2), (1, 8, 256, [5000, 257], 4), (2, 1, 128, [33, 500], 1),
     (1, 16, 128, [700, 129, 1], 2),  # a group of more than 8 heads: the two terms as separate tensor-core instructions
     (1, 4, 256, [131072, 33000, 40001], 16)],  # the long-context stress: 513-column block table, 16 context splits
)
@pytest.mark.parametrize("fused,single_term", [(True, False), (False, False), (True, True)])
def test_paged_attention_fp8_pool(ops, nkv, G, chunk, kv_lens, splits, fused, single_term):
    D = 128
    c = make_paged_case(T=len(kv_lens), nkv=nkv, G=G, D=D, chunk=chunk, kv_lens=kv_lens, seed=21)
    g = torch.Generator().manual_seed(5)
    k_scale = 0.01 + 0.02 * torch.rand(nkv, generator=g)
    v_scale = 0.01 + 0.02 * torch.rand(nkv, generator=g)
    # the pool as E4M3 bytes
    kq = O._to_e4m3(c["k_cache"].float() / k_scale[None, None, :, None])
    vq = O._to_e4m3(c["v_cache"].float() / v_scale[None, None, :, None])
    T = c["T"]
    qkv = c["qkv"]
    q = O.apply_rope(qkv[..., : G * D].reshape(T, nkv * G, D), c["freqs"][c["pos"]])
    k = O.apply_rope(qkv[..., G * D : (G + 1) * D], c["freqs"][c["pos"]])
    kq_ref, vq_ref = kq.clone(), vq.clone()
    kq_ref[c["chunk_idx"], c["local"]] = O.quantize_kv_fp8(k, k_scale)
    vq_ref[c["chunk_idx"], c["local"]] = O.quantize_kv_fp8(qkv[..., (G + 1) * D :], v_scale)
    ref = O.paged_attention(q, kq_ref, vq_ref, c["kv_lens"], c["block_table"].numpy(), k_scale=k_scale, v_scale=v_scale)

    dev = "cuda"
    half = c["freqs"][:, : D // 2]
    cos, sin = torch.cos(half).to(BF16).to(dev), torch.sin(half).to(BF16).to(dev)
    # keys as they are; values in the pool's own byte order (transposed inside a chunk, positions permuted)
    kc = kq.view(torch.uint8).to(dev)
    vc = ops.fp8_values_to_pool_layout(vq.view(torch.uint8)).to(dev)
    assert torch.equal(ops.fp8_values_from_pool_layout(vc.cpu()), vq.view(torch.uint8))
    out = torch.full((T, c["nq"] * D), float("nan"), dtype=BF16, device=dev)
    d = {k_: c[k_].to(dev) for k_ in ("qkv", "block_table", "kv_lens", "pos", "chunk_idx", "local")}
    ks, vs = k_scale.to(dev), v_scale.to(dev)
    args = ops.make_attention_args(
        qkv=d["qkv"], k_cache=kc, v_cache=vc, block_table=d["block_table"], kv_seq_lengths=d["kv_lens"], out=out,
        num_q_heads=c["nq"], num_kv_heads=nkv, head_dim=D, chunk_size=chunk, token_to_pos_ids=d["pos"],
        token_to_pos_in_request=d["pos"], token_to_chunk_idx=d["chunk_idx"], token_to_local_pos=d["local"],
        rope_cos=cos, rope_sin=sin, num_splits=splits, fuse_rope_append=fused, k_scale=ks, v_scale=vs,
        fp8_single_term=single_term)
    if not fused:
        ops.rope_append(args)
    ops.paged_attention(args)
    torch.cuda.synchronize()
    live = [r for r, kl in enumerate(kv_lens) if kl > 0]
    v_now = ops.fp8_values_from_pool_layout(vc.cpu())
    for r in live:  # appended bytes: bit-exact
        ci, lp = int(c["chunk_idx"][r]), int(c["local"][r])
        assert torch.equal(kc[ci, lp].cpu(), kq_ref.view(torch.uint8)[ci, lp]), r
        assert torch.equal(v_now[ci, lp], vq_ref.view(torch.uint8)[ci, lp]), r
    if fused:  # nothing else in the pool was touched
        mask = torch.ones(kc.shape[:2], dtype=torch.bool)
        mask[c["chunk_idx"][live], c["local"][live]] = False
        assert torch.equal(kc.cpu()[mask], kq.view(torch.uint8)[mask])
        assert torch.equal(v_now[mask], vq.view(torch.uint8)[mask])
    o = out.cpu().view(T, c["nq"], D)
    assert not torch.isnan(o.float()).any()
    # same E4M3 pool on both sides; the kernel feeds queries and probabilities to the fp8 tensor cores as two
    # E4M3 terms each (~7 significant bits), far inside the 2^-4 resolution of the pool itself
    # (one term each: E4M3 queries and probabilities, 2^-4 resolution like the pool's own)
    assert rel_l2(o, ref) < (6e-2 if single_term else 6e-3), rel_l2(o, ref)


@pytest.mark.parametrize("shards,vocab", [(2, 1000), (8, 128256), (4, 4096)])
def test_shardwise_argmax_equals_argmax_of_the_gathered_rows(ops, shards, vocab):
    rows = 37
    g = torch.Generator().manual_seed(5)
    logits = torch.randn((rows, vocab), generator=g).to(BF16)
    per = vocab // shards
    logits[0, :] = 1.5                      # all equal: index 0
    logits[1, per - 1] = 9.0                # the maximum twice, in two shards: the smaller index wins
    logits[1, per + 3] = 9.0
    logits[2, :] = -0.0                     # signed zeros compare equal
    logits[2, vocab - 1] = 0.0
    logits[3, :] = float("-inf")
    logits[4, vocab - 1] = 50.0             # last element of the last shard
    ref = ops.argmax(logits.cuda())
    keys = torch.stack([ops.argmax_shard(logits[:, s * per:(s + 1) * per].contiguous().cuda(), s * per) for s in range(shards)])
    got = ops.argmax_merge(keys)
    assert torch.equal(got, ref)
    assert got[0] == 0 and got[1] == per - 1 and got[2] == 0 and got[3] == 0 and got[4] == vocab - 1
    assert torch.equal(got.cpu(), torch.argmax(logits.float(), dim=-1))
