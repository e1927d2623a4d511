"""Model-level parity at the benchmark's real widths: 2-layer cuts of the Llama-3-8B shape (hidden 4096, FFN 14336,
32 / 8 heads, vocabulary 128256) and of the Llama-3-70B shape (hidden 8192, FFN 28672, 64 / 8 heads) run through
context -> controller -> model -> kernels, teacher-forced against the CPU oracle on the same canonical weights.

Bars: the stated tolerances themselves (5e-3 relative L2 for bf16 logits, 2e-2 for every FP8 recipe).  Where the
oracle's own noise floor at that width (the oracle against itself with every dot product accumulated in the opposite
order, `width_parity.oracle_floor`) is above the bar, no implementation can meet the bar against this oracle; the
assertion is then `<= 1.1 x floor`, and the test prints bar, floor and measurement so that the record shows which one
applied.  Greedy flips are accepted only on near-ties of the oracle's own logits; block tables / KV slots are
compared bit-exactly by the tiny-model tests, which use the same context code.
"""
import pytest
import torch

import width_parity as WP

pytestmark = pytest.mark.gpu

W8B = dict(hidden_size=4096, ffn_hidden_size=14336, num_attention_heads=32, num_query_groups=8, vocab_size=128256)
W70B = dict(hidden_size=8192, ffn_hidden_size=28672, num_attention_heads=64, num_query_groups=8, vocab_size=32064)

CASES = [
    ("8b-bf16", W8B, dict()),
    ("8b-mxfp8", W8B, dict(fp8="mxfp8")),
    ("8b-blockwise", W8B, dict(fp8="blockwise")),
    ("8b-mxfp8-e4m3kv", W8B, dict(fp8="mxfp8", kv_fp8_scale=2.0**-6)),
    ("70b-bf16", W70B, dict()),
    ("70b-blockwise", W70B, dict(fp8="blockwise")),
]


@pytest.mark.parametrize("name,width,extra", CASES, ids=[c[0] for c in CASES])
def test_cut_matches_oracle_within_the_stated_bar(name, width, extra):
    meta = WP.cut_meta(**width, **extra)
    trace = WP.oracle_trace_for(meta)
    floor = WP.oracle_floor(meta, trace)
    res = WP.run_cuda_cut(meta, trace)
    bar = WP.bar_for(meta)
    worst, worst_floor = max(res["rel"]), max(floor)
    limit = bar if worst_floor <= bar / 1.1 else 1.1 * worst_floor
    print(f"\n[width parity] {name}: rel-L2 per step {['%.2e' % r for r in res['rel']]}, oracle-vs-oracle floor "
          f"{['%.2e' % r for r in floor]}, stated bar {bar:.0e}, limit applied {limit:.2e}, flips {len(res['flips'])}/"
          f"{res['decisions']}")
    assert res["graph_replays"] >= 1
    assert worst <= limit, (name, res["rel"], floor, bar)
    assert res["flips_ok"], res["flips"]
    # the mean must not hide behind the worst step either
    assert sum(res["rel"]) / len(res["rel"]) <= max(bar, 1.1 * sum(floor) / len(floor))
