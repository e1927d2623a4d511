"""Seeded synthetic weights and request sets.

There are no checkpoints or datasets to load, so both the parity fixtures and the
benchmark use weights drawn N(0, std) per tensor from a generator whose seed is
derived from the tensor's ``state_dict`` key.  Deriving the seed from the key makes
the values independent of module construction order and of the tensor-parallel size:
every rank materialises the *full* tensor and slices its own shard
(`shard_for_rank`), which is how the parity harness keeps TP=1 and TP>1 models the
same function.
"""
from __future__ import annotations

import zlib
from typing import Dict, Iterable, List, Optional, Tuple

import torch

_NORM_MARKERS = ("layernorm.weight", "layer_norm_weight", "norm.weight")


def _is_norm_scale(name: str) -> bool:
    return any(name.endswith(m) for m in _NORM_MARKERS)


def canonical_tensor(
    name: str,
    shape: Iterable[int],
    *,
    seed: int = 0,
    std: float = 0.02,
    dtype: torch.dtype = torch.float32,
    device: str | torch.device = "cpu",
) -> torch.Tensor:
    """Full (unsharded) tensor for ``state_dict`` key ``name``.

    Values are generated in fp32 and then cast.  Norm scales are ``1 + N(0, std)`` so
    that a kernel that forgets the scale is caught; everything else, biases included,
    is ``N(0, std)``.  With ``device='cpu'`` the values are reproducible bit-for-bit
    (this is what the committed fixtures use); on a CUDA device a CUDA generator is
    used, which gives the same distribution much faster for multi-billion-parameter
    benchmark models.
    """
    shape = tuple(int(s) for s in shape)
    dev = torch.device(device)
    g = torch.Generator(device=dev)
    g.manual_seed((int(seed) * 1000003 + zlib.crc32(name.encode())) & 0x7FFFFFFFFFFF)
    t = torch.empty(shape, dtype=torch.float32, device=dev)
    t.normal_(0.0, std, generator=g)
    if _is_norm_scale(name):
        t += 1.0
    return t.to(dtype)


def canonical_state_dict(
    shapes: Dict[str, Tuple[int, ...]],
    *,
    seed: int = 0,
    std: float = 0.02,
    dtype: torch.dtype = torch.float32,
    device: str | torch.device = "cpu",
) -> Dict[str, torch.Tensor]:
    """Canonical full tensors for every ``name -> full shape`` entry."""
    return {
        k: canonical_tensor(k, s, seed=seed, std=std, dtype=dtype, device=device)
        for k, s in shapes.items()
    }


def synthetic_prompts(
    num_requests: int,
    min_len: int,
    max_len: int,
    vocab_size: int,
    *,
    seed: int = 0,
    log_uniform: bool = False,
) -> List[torch.Tensor]:
    """Prompt token ids: lengths uniform (or log-uniform) in [min_len, max_len], ids uniform in vocab."""
    g = torch.Generator().manual_seed(seed)
    if log_uniform:
        import math

        u = torch.rand(num_requests, generator=g)
        lens = torch.exp(math.log(min_len) + u * (math.log(max_len) - math.log(min_len))).long()
        lens = lens.clamp(min_len, max_len)
    else:
        lens = torch.randint(min_len, max_len + 1, (num_requests,), generator=g)
    return [
        torch.randint(0, vocab_size, (int(n),), generator=g, dtype=torch.int64) for n in lens.tolist()
    ]
