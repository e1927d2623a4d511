"""MXFP8 path: quantisers and the block-scaled tcgen05 GEMM against the CPU oracle's restatement
(E4M3 values, E8M0 scale per 32 elements, scale = smallest power of two >= amax / 448)."""
import pytest
import torch
import torch.nn.functional as F

from oracle import decode_oracle as O

pytestmark = pytest.mark.gpu
BF16 = torch.bfloat16


@pytest.fixture(scope="module")
def ops():
    from megatron_mixtera_b200 import build, ops as _ops

    build.build()
    yield _ops
    torch.cuda.synchronize()
    assert _ops.device_status() == 0


def randn(shape, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(BF16)


def rel_l2(a, b):
    a, b = a.float().cpu(), b.float().cpu()
    return float((a - b).norm() / b.norm().clamp_min(1e-30))


def check_quantised(t, x_ref_bf16, exact=True):
    """`t` (Mxfp8Tensor on the device) against the oracle's quantisation of `x_ref_bf16` [rows, K]."""
    rows, K = x_ref_bf16.shape
    q_ref, e_ref = O.quantize_mxfp8(x_ref_bf16)
    q = t.q.cpu().view(torch.float8_e4m3fn)
    tiles = O.mxfp8_scales_to_tile_layout(e_ref)
    sf = t.sf.cpu()
    assert sf.numel() == tiles.numel()
    # compare only the bytes that belong to real rows (the rest of a tile is never read for real outputs)
    mask = O.mxfp8_scales_to_tile_layout(torch.ones_like(e_ref)).bool()
    if exact:
        assert torch.equal(sf[mask], tiles[mask])
        assert torch.equal(q.view(torch.uint8), q_ref.view(torch.uint8))
    else:
        assert (sf[mask] != tiles[mask]).float().mean() < 2e-3
        assert (q.view(torch.uint8) != q_ref.view(torch.uint8)).float().mean() < 5e-3
    return q_ref, e_ref


@pytest.mark.parametrize("rows,K", [(1, 128), (64, 4096), (130, 512), (300, 1024)])
def test_quantize_mxfp8_bit_exact(ops, rows, K):
    x = randn((rows, K), 1, 3.0)
    x[0, :32] = 0            # an all-zero block
    x[-1, -32:] = 448.0      # exactly the E4M3 maximum: scale 2^0, no saturation
    if rows > 2:
        x[1, 0] = 1000.0     # forces the round-up of the scale exponent
    t = ops.quantize_mxfp8(x.cuda())
    q_ref, e_ref = check_quantised(t, x)
    assert float(O.dequantize_mxfp8(q_ref, e_ref)[-1, -1]) == 448.0
    assert rel_l2(O.dequantize_mxfp8(q_ref, e_ref), x) < 0.04


@pytest.mark.parametrize(
    "M,N,K,bias",
    [
        (8, 256, 256, False),
        (64, 1024, 512, True),      # split-K
        (33, 384, 1024, True),
        (128, 512, 256, False),     # BT = 128
        (200, 384, 1024, False),    # BT = 256: two scale tiles per stage
        (300, 640, 512, True),      # two token blocks
        (64, 6144, 4096, False),    # Llama-3-8B qkv at decode
        (64, 4096, 14336, False),   # Llama-3-8B fc2 at decode
        (16, 20000, 512, False),
    ],
)
def test_gemm_mxfp8_matches_dequantised_product(ops, M, N, K, bias):
    x, w = randn((M, K), 1), randn((N, K), 2, 0.05)
    b = randn((N,), 3) if bias else None
    xq, wq = ops.quantize_mxfp8(x.cuda()), ops.quantize_mxfp8_weight(w.cuda())
    y = ops.gemm_mxfp8(xq, wq, None if b is None else b.cuda())
    xd = O.dequantize_mxfp8(*O.quantize_mxfp8(x))
    wd = O.dequantize_mxfp8(*O.quantize_mxfp8(w))
    ref = xd @ wd.t()
    if b is not None:
        ref = ref.to(BF16).float() + b.float()
    assert y.shape == (M, N) and y.dtype == BF16
    # exact products of exactly representable operands, fp32 accumulation: only the output rounding differs
    assert rel_l2(y, ref) < 3e-3, rel_l2(y, ref)
    assert (y.cpu() != ref.to(BF16)).float().mean() < 2e-3
    # and the FP8 format itself stays within the stated 2e-2 of the bf16 product
    assert rel_l2(y, x.float() @ w.float().t() + (0 if b is None else b.float())) < 4e-2
    assert torch.equal(ops.gemm_mxfp8(xq, wq, None if b is None else b.cuda()), y)


@pytest.mark.parametrize("N,K", [(128, 128), (300, 512), (1024, 4096)])
def test_mxfp8_weight_quantiser_is_the_row_quantiser_with_tile_major_bytes(ops, N, K):
    w = randn((N, K), 4, 0.05).cuda()
    rows, tiles = ops.quantize_mxfp8(w), ops.quantize_mxfp8_weight(w)
    assert tiles.packed and not rows.packed
    assert torch.equal(ops.weight_tiles_to_rows(tiles.q, N, K), rows.q)
    idx = _sf_indices(N, K).to(rows.sf.device)
    assert torch.equal(tiles.sf[idx], rows.sf[idx])
    with pytest.raises(ops.B200Error):
        ops.gemm_mxfp8(ops.quantize_mxfp8(randn((8, K), 5).cuda()), rows)  # row-major bytes are not a weight


def test_fused_norm_and_activation_quantisers(ops):
    rows, hidden = 64, 4096
    x, r = randn((rows, hidden), 1), randn((rows, hidden), 2)
    g = (1 + randn((hidden,), 3, 0.02).float()).to(BF16)
    h, t = ops.add_norm_mxfp8(x.cuda(), g.cuda(), residual=r.cuda(), want_hidden=True)
    assert torch.equal(h.cpu(), x + r)
    check_quantised(t, F.rms_norm(x + r, (hidden,), g, 1e-5), exact=False)
    y = randn((17, 2 * 1024), 4, 2.0)
    a, b = torch.chunk(y, 2, dim=-1)
    t = ops.activation_mxfp8(y.cuda(), "swiglu")
    check_quantised(t, F.silu(a) * b, exact=False)
    assert t.shape == (17, 1024)


# ------------------------------------------------------------------------------------------
# 128-block recipe (fp32 scales: 128 x 128 weight blocks, 1 x 128 per-token activation blocks)
# ------------------------------------------------------------------------------------------
@pytest.mark.parametrize("rows,K", [(3, 128), (64, 4096), (130, 512)])
def test_rowblock_quantiser_bit_exact(ops, rows, K):
    x = randn((rows, K), 1, 3.0)
    x[0, :128] = 0
    t = ops.quantize_fp8_rowblock(x.cuda())
    q_ref, s_ref = O.quantize_fp8_rowblock(x, 128)
    assert torch.equal(t.q.cpu(), q_ref.view(torch.uint8))
    assert torch.equal(t.scale.cpu()[:, :rows].t().contiguous(), s_ref)


@pytest.mark.parametrize("N,K", [(128, 128), (300, 512), (4096, 4096)])
def test_weight_block_quantiser_bit_exact(ops, N, K):
    w = randn((N, K), 2, 0.05)
    t = ops.quantize_fp8_weight_block128(w.cuda())
    q_ref, s_ref = O.quantize_fp8_block_weight(w, 128)
    assert torch.equal(t.scale.cpu(), s_ref)
    assert torch.equal(ops.weight_tiles_to_rows(t.q, N, K).cpu(), q_ref.view(torch.uint8))  # bytes are tile-major


@pytest.mark.parametrize(
    "M,N,K,bias",
    [(8, 256, 256, False), (64, 1024, 512, True), (33, 384, 1024, True), (128, 512, 256, False), (300, 640, 512, True),
     (64, 6144, 4096, False), (64, 4096, 14336, False), (256, 8192 // 8 * 10 // 8 * 8, 8192, False)],
)
def test_gemm_fp8_block_matches_dequantised_product(ops, M, N, K, bias):
    x, w = randn((M, K), 1), randn((N, K), 2, 0.05)
    b = randn((N,), 3) if bias else None
    xq, wq = ops.quantize_fp8_rowblock(x.cuda()), ops.quantize_fp8_weight_block128(w.cuda())
    y = ops.gemm_fp8_block(xq, wq, None if b is None else b.cuda())
    xd = O.dequantize_fp8_rowblock(*O.quantize_fp8_rowblock(x, 128), 128)
    wd = O.dequantize_fp8_block_weight(*O.quantize_fp8_block_weight(w, 128), 128)
    ref = xd @ wd.t()
    if b is not None:
        ref = ref.to(BF16).float() + b.float()
    assert rel_l2(y, ref) < 3e-3, rel_l2(y, ref)
    assert rel_l2(y, x.float() @ w.float().t() + (0 if b is None else b.float())) < 4e-2
    assert torch.equal(ops.gemm_fp8_block(xq, wq, None if b is None else b.cuda()), y)


def test_fused_rowblock_quantisers(ops):
    rows, hidden = 64, 4096
    x, r = randn((rows, hidden), 1), randn((rows, hidden), 2)
    g = (1 + randn((hidden,), 3, 0.02).float()).to(BF16)
    h, t = ops.add_norm_fp8_rowblock(x.cuda(), g.cuda(), residual=r.cuda(), want_hidden=True)
    assert torch.equal(h.cpu(), x + r)
    q_ref, s_ref = O.quantize_fp8_rowblock(F.rms_norm(x + r, (hidden,), g, 1e-5), 128)
    assert (t.q.cpu() != q_ref.view(torch.uint8)).float().mean() < 5e-3
    assert torch.allclose(t.scale.cpu()[:, :rows].t(), s_ref, rtol=1e-2)
    y = randn((17, 2 * 1024), 4, 2.0)
    a, b = torch.chunk(y, 2, dim=-1)
    t = ops.activation_fp8_rowblock(y.cuda(), "swiglu")
    q_ref, s_ref = O.quantize_fp8_rowblock(F.silu(a) * b, 128)
    assert (t.q.cpu() != q_ref.view(torch.uint8)).float().mean() < 5e-3


# ------------------------------------------------------------------------------------------
# Split-K partial sums of the FP8 GEMMs consumed by the residual-add + norm (+ quantise) kernel
# ------------------------------------------------------------------------------------------
@pytest.mark.parametrize("recipe", ["mxfp8", "blockwise"])
@pytest.mark.parametrize("M,N,K", [(64, 4096, 4096), (128, 4096, 14336), (20, 1024, 512)])
def test_fp8_splitk_partials_into_add_norm_equal_unfused(ops, recipe, M, N, K):
    x, w = randn((M, K), 1).cuda(), randn((N, K), 2, 0.05).cuda()
    r = randn((M, N), 3).cuda()
    g = (1 + randn((N,), 4, 0.02).float()).to(BF16).cuda()
    if recipe == "mxfp8":
        xq, wq = ops.quantize_mxfp8(x), ops.quantize_mxfp8_weight(w)
        y = ops.gemm_mxfp8(xq, wq)
        h_ref, t_ref = ops.add_norm_mxfp8(y, g, residual=r, want_hidden=True)
    else:
        xq, wq = ops.quantize_fp8_rowblock(x), ops.quantize_fp8_weight_block128(w)
        y = ops.gemm_fp8_block(xq, wq)
        h_ref, t_ref = ops.add_norm_fp8_rowblock(y, g, residual=r, want_hidden=True)
    p = ops.gemm_splitk(xq, wq)
    h, t = ops.add_norm_splitk(p, g, residual=r, want_hidden=True, quantize=recipe)
    assert torch.equal(h, h_ref) and torch.equal(t.q, t_ref.q)
    if recipe == "mxfp8":
        # scale bytes of the rows that exist (the buffers are padded to whole 256-row groups and never cleared)
        rr = torch.arange(M).view(-1, 1)
        bb = torch.arange(N // 32).view(1, -1)
        off = ((rr // 128) * (N // 128) + bb // 4) * 512 + (rr % 32) * 16 + ((rr % 128) // 32) * 4 + bb % 4
        off = off.flatten().cuda()
        assert torch.equal(t.sf[off], t_ref.sf[off])
    else:
        assert torch.equal(t.scale[:, :M], t_ref.scale[:, :M])
    # bf16 output of the same partial sums
    p = ops.gemm_splitk(xq, wq)
    h2, n2 = ops.add_norm_splitk(p, g, residual=r, want_hidden=True)
    _, n_ref = ops.add_norm(y, g, residual=r, want_hidden=True)
    assert torch.equal(h2, h_ref) and torch.equal(n2, n_ref)
    assert ops.device_status() == 0


@pytest.mark.parametrize("M,F,K", [(128, 512, 1024), (64, 256, 512), (17, 128, 256), (200, 384, 640), (128, 14336 // 8, 4096)])
@pytest.mark.parametrize("quantize", [True, False])
def test_mxfp8_gate_up_pair_gemm_equals_gemm_then_activation(M, F, K, quantize):
    # fc1 + SwiGLU (+ quantisation) in one kernel against the unfused pair: the same bits whenever the unfused GEMM
    # accumulates K in one piece too (a split-K GEMM adds its partial sums in another order: fp32 rounding noise)
    from megatron_mixtera_b200 import ops

    exact = ops.gemm_num_splits("mxfp8", M, 2 * F, K) == 1

    x = ops.quantize_mxfp8(randn((M, K), 5).cuda())
    w = ops.quantize_mxfp8_weight(randn((2 * F, K), 6, 0.05).cuda())
    y = ops.gemm_mxfp8(x, w)
    if quantize:
        ref = ops.activation_mxfp8(y, "swiglu")
        got = ops.gemm_mxfp8_swiglu(x, w)
        torch.cuda.synchronize()
        # scale bytes of the rows that exist (the tile layout pads rows to 256)
        assert got.sf.numel() == ref.sf.numel()
        idx = _sf_indices(M, F).to(got.sf.device)
        if exact:
            assert torch.equal(got.q[:M], ref.q[:M])
            assert torch.equal(got.sf[idx], ref.sf[idx])
        else:
            assert float((got.q[:M] != ref.q[:M]).float().mean()) < 2e-3
            assert float((got.sf[idx] != ref.sf[idx]).float().mean()) < 2e-3
    else:
        ref = ops.activation(y, "swiglu")
        got = ops.gemm_mxfp8_swiglu(x, w, quantize=False)
        torch.cuda.synchronize()
        if exact:
            assert torch.equal(got, ref)
        else:
            assert float((got != ref).float().mean()) < 2e-3 and rel_l2(got, ref) < 1e-3
    assert ops.device_status() == 0


def _sf_indices(rows, K):
    """Flat positions, in the tile layout, of the scale bytes of rows [0, rows) x K / 32 blocks."""
    r = torch.arange(rows)[:, None]
    b = torch.arange(K // 32)[None, :]
    off = (r // 128) * (K // 128) * 512 + (b // 4) * 512 + (r % 32) * 16 + ((r % 128) // 32) * 4 + (b % 4)
    return off.reshape(-1)


@pytest.mark.parametrize("recipe", [None, "mxfp8", "blockwise"])
@pytest.mark.parametrize("M,F,K", [(64, 256, 4096), (128, 512, 2048)])
def test_activation_reduces_fc1_split_k_partials(recipe, M, F, K):
    # fc1 split along K: the activation kernel sums the partial sums itself (no reduction launch); same bits
    from megatron_mixtera_b200 import ops

    xb, wb = randn((M, K), 7).cuda(), randn((2 * F, K), 8, 0.05).cuda()
    if recipe == "mxfp8":
        x, w = ops.quantize_mxfp8(xb), ops.quantize_mxfp8_weight(wb)
        ref = ops.activation_mxfp8(ops.gemm_mxfp8(x, w), "swiglu")
    elif recipe == "blockwise":
        x, w = ops.quantize_fp8_rowblock(xb), ops.quantize_fp8_weight_block128(wb)
        ref = ops.activation_fp8_rowblock(ops.gemm_fp8_block(x, w), "swiglu")
    else:
        x, w = xb, wb
        ref = ops.activation(ops.gemm(x, w), "swiglu")
    assert ops.gemm_num_splits(recipe, M, 2 * F, K) > 1
    got = ops.activation_splitk(ops.gemm_splitk(x, w), "swiglu", quantize=recipe)
    torch.cuda.synchronize()
    if recipe is None:
        assert torch.equal(got, ref)
    else:
        assert torch.equal(got.q[:M], ref.q[:M])
        if recipe == "blockwise":
            assert torch.equal(got.scale[:, :M], ref.scale[:, :M])
        else:
            idx = _sf_indices(M, F).to(got.sf.device)
            assert torch.equal(got.sf[idx], ref.sf[idx])
    assert ops.device_status() == 0


@pytest.mark.parametrize("M,N,K", [(256, 256, 256), (256, 512, 1024), (200, 2560, 4096), (130, 1024, 2048), (256, 8192, 2048)])
def test_blockwise_gemm_as_cta_pairs_equals_the_single_cta_kernel(ops, M, N, K):
    """The opt-in `tcgen05.mma.cta_group::2` form of the 256-token blockwise GEMM (csrc/gemm_fp8_block_pair.cu: two CTAs
    on two SMs share one 256 x 256 output tile) accumulates and promotes every 128-wide K block exactly like the
    single-CTA kernel: outputs and split-K partial sums must be identical bit for bit."""
    from megatron_mixtera_b200 import _lib

    lib = _lib.load()
    x = randn((M, K), 31).cuda()
    w = randn((N, K), 32, 0.05).cuda()
    bias = randn((N,), 33).cuda()
    xq, wq = ops.quantize_fp8_rowblock(x), ops.quantize_fp8_weight_block128(w)
    got = {}
    try:
        for pairs in (0, 1):
            assert lib.b200_set_fp8_block_cta_pairs(pairs) == 0
            y = ops.gemm_fp8_block(xq, wq, bias)
            p = ops.gemm_splitk(xq, wq)
            parts = p.buf[: p.num_splits * M * N * 4].view(torch.float32).clone()
            got[pairs] = (y, parts, p.num_splits)
    finally:
        lib.b200_set_fp8_block_cta_pairs(0)
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    assert got[0][2] == got[1][2]
    assert torch.equal(got[0][0], got[1][0])
    assert torch.equal(got[0][1], got[1][1])
