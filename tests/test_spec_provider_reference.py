"""`B200SpecProvider` handed to the REFERENCE's own layer-spec assembly.

The reference picks its operator classes through a `BackendSpecProvider` (megatron/core/models/backends.py:26-70)
inside `get_gpt_layer_local_spec` (megatron/core/models/gpt/gpt_layer_specs.py:200-309).  This test runs that
function with this repository's provider in place of `LocalSpecProvider`, lets the reference's `GPTModel` /
`TransformerLayer` / `SelfAttention` / `MLP` build themselves from the resulting spec (on the CPU), and compares the
module tree and the `state_dict` keys and shapes with the reference's plain local spec: what a checkpoint of one
loads into is what the other has.  Needs the reference checkout; skipped where it is absent (it cannot travel).
It runs in a child process because importing the reference on a CPU-only machine needs two patches of torch / the
reference's RNG tracker that must not leak into the other tests.
"""
import os
import subprocess
import sys

import pytest

from conftest import ROOT

REFERENCE = os.environ.get("MEGATRON_REFERENCE", os.path.join(os.path.dirname(ROOT), "reference"))  # a sibling checkout

CHILD = r'''
import contextlib, json, os, sys
ref, root = sys.argv[1], sys.argv[2]
sys.path.insert(0, ref); sys.path.insert(0, root)
os.environ.setdefault("TORCHDYNAMO_DISABLE", "1")
os.environ.setdefault("MASTER_ADDR", "127.0.0.1"); os.environ.setdefault("MASTER_PORT", "29541")
import torch
torch.cuda.current_device = lambda: torch.device("cpu")
import torch.distributed as dist
dist.init_process_group("gloo", rank=0, world_size=1)
from megatron.core import parallel_state as ps
ps.initialize_model_parallel(1, 1)
from megatron.core.tensor_parallel import random as _r
_r.CudaRNGStatesTracker.fork = lambda self, name=None: contextlib.nullcontext()
from megatron.core.models.gpt import gpt_layer_specs as S
from megatron.core.models.gpt.gpt_model import GPTModel
from megatron.core.transformer.transformer_config import TransformerConfig
from megatron_mixtera_b200.spec_provider import B200SpecProvider
from megatron_mixtera_b200.tensor_parallel.layers import ColumnParallelLinear, RowParallelLinear
from megatron_mixtera_b200.transformer.attention import PagedFlashDecodeAttention
from megatron_mixtera_b200.transformer.norm import B200Norm

def build(spec):
    cfg = TransformerConfig(num_layers=2, hidden_size=256, num_attention_heads=4, num_query_groups=2, kv_channels=64,
                            ffn_hidden_size=512, use_cpu_initialization=True, params_dtype=torch.bfloat16, bf16=True,
                            hidden_dropout=0.0, attention_dropout=0.0, normalization="RMSNorm", gated_linear_unit=True,
                            activation_func=torch.nn.functional.silu, add_bias_linear=False)
    return GPTModel(config=cfg, transformer_layer_spec=spec, vocab_size=512, max_sequence_length=128, parallel_output=True,
                    position_embedding_type="rope", rotary_base=500000, share_embeddings_and_output_weights=False)

plain = build(S.get_gpt_layer_local_spec(normalization="RMSNorm"))
S.LocalSpecProvider = B200SpecProvider            # the provider the assembly function instantiates
ours = build(S.get_gpt_layer_local_spec(normalization="RMSNorm"))

def shapes(m):
    return {k: tuple(v.shape) for k, v in m.state_dict().items() if v is not None and not k.endswith("_extra_state")}
def tree(m):  # (the reference's local core attention has softmax / dropout children; the paged kernel module has none)
    return sorted(n for n, _ in m.named_modules() if ".core_attention." not in n)
layer = ours.decoder.layers[0]
report = {
    "same_state_dict": shapes(plain) == shapes(ours),
    "keys": len(shapes(ours)),
    "same_tree": tree(plain) == tree(ours),
    "classes": {
        "linear_qkv": isinstance(layer.self_attention.linear_qkv, ColumnParallelLinear),
        "linear_proj": isinstance(layer.self_attention.linear_proj, RowParallelLinear),
        "core_attention": isinstance(layer.self_attention.core_attention, PagedFlashDecodeAttention),
        "linear_fc1": isinstance(layer.mlp.linear_fc1, ColumnParallelLinear),
        "linear_fc2": isinstance(layer.mlp.linear_fc2, RowParallelLinear),
        "input_layernorm": isinstance(layer.input_layernorm, B200Norm),
        "pre_mlp_layernorm": isinstance(layer.pre_mlp_layernorm, B200Norm),
    },
    "diff": sorted(set(shapes(plain).items()) ^ set(shapes(ours).items()))[:6],
}
# a state dict of the reference's model loads into the model built from our operator classes
missing = ours.load_state_dict({k: v for k, v in plain.state_dict().items() if v is not None and not k.endswith("_extra_state")}, strict=False)
report["missing_after_load"] = [k for k in missing.missing_keys if not k.endswith("_extra_state")]
report["unexpected_after_load"] = list(missing.unexpected_keys)
print("REPORT " + json.dumps(report))
'''


@pytest.mark.skipif(not os.path.isdir(os.path.join(REFERENCE, "megatron", "core")), reason="the reference checkout is not on this machine")
def test_reference_layer_spec_assembles_with_b200_operator_classes(tmp_path):
    script = tmp_path / "child.py"
    script.write_text(CHILD)
    proc = subprocess.run([sys.executable, str(script), REFERENCE, ROOT], capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stdout[-2000:] + proc.stderr[-4000:]
    import json

    line = next(l for l in proc.stdout.splitlines() if l.startswith("REPORT "))
    rep = json.loads(line[len("REPORT "):])
    assert all(rep["classes"].values()), rep["classes"]
    assert rep["same_tree"], rep
    assert rep["same_state_dict"] and rep["keys"] > 10, rep
    assert not rep["missing_after_load"] and not rep["unexpected_after_load"], rep
