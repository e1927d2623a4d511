"""The reference engine's view of this package's context and controller.

The reference's `DynamicInferenceEngine` (megatron/core/inference/engines/dynamic_engine.py) asserts the classes of
the controller and context it is given (:107-108) and then uses a fixed set of their attributes and methods.  In a
child process that imports the reference (it cannot travel, so the test is skipped where the checkout is absent):
  * `reference_subclasses()` yields classes that pass those isinstance checks and resolve every method to this
    package's implementation;
  * every `context.<name>` / `controller.<name>` the reference engine's source uses exists here, and where it is a
    method the parameter lists agree (names, order, defaults);
  * the dict the controller returns per step has the keys the engine reads (:576-582).
"""
import os
import subprocess
import sys

import pytest

from conftest import ROOT

REFERENCE = os.environ.get("MEGATRON_REFERENCE", os.path.join(os.path.dirname(ROOT), "reference"))  # a sibling checkout

CHILD = r'''
import inspect, json, os, re, sys
ref, root = sys.argv[1], sys.argv[2]
sys.path.insert(0, ref); sys.path.insert(0, root)
os.environ.setdefault("TORCHDYNAMO_DISABLE", "1")
import torch
torch.cuda.current_device = lambda: torch.device("cpu")
from megatron.core.inference.contexts.dynamic_context import DynamicInferenceContext as RefCtx
from megatron.core.inference.text_generation_controllers.simple_text_generation_controller import SimpleTextGenerationController as RefCtl
from megatron_mixtera_b200.inference.contexts.dynamic_context import DynamicInferenceContext as Ctx
from megatron_mixtera_b200.inference.text_generation_controllers.text_generation_controller import TextGenerationController as Ctl
from megatron_mixtera_b200.reference_seam import reference_subclasses

C, T = reference_subclasses()
out = {"sub": [issubclass(C, RefCtx), issubclass(C, Ctx), issubclass(T, RefCtl), issubclass(T, Ctl)],
       "same": reference_subclasses()[0] is C, "shadowed": [], "missing": [], "signature": []}
# every attribute the reference classes define resolves to this package's implementation when this package has one
for cls, ours in ((C, Ctx), (T, Ctl)):
    for name in dir(ours):
        if not name.startswith("__") and inspect.getattr_static(cls, name) is not inspect.getattr_static(ours, name):
            out["shadowed"].append(name)
src = open(os.path.join(ref, "megatron/core/inference/engines/dynamic_engine.py")).read()
def sig(f):
    return [(p.name, p.kind.name, repr(p.default)) for p in inspect.signature(f).parameters.values()]
for pattern, ours, theirs in ((r"(?<![\w.])(?:self\.)?context\.([a-z_]\w*)", Ctx, RefCtx), (r"controller\.([a-z_]\w*)", Ctl, RefCtl)):
    ours_src = inspect.getsource(ours)
    for name in sorted(set(re.findall(pattern, src))):
        if not (hasattr(ours, name) or re.search(r"self\.%s\b\s*(?::[^=\n]+)?=" % name, ours_src)):
            out["missing"].append(name)
        elif inspect.isfunction(getattr(theirs, name, None)) and sig(getattr(theirs, name)) != sig(getattr(ours, name)):
            out["signature"].append(name)
step = src[src.index("controller.async_generate_output_tokens_dynamic_batch("):]
keys = set(re.findall(r'= result\["(\w+)"\]', step[:step.index("schedule_waiting_requests")]))
out["result_keys_missing"] = sorted(k for k in keys if ('"%s":' % k) not in inspect.getsource(Ctl))
out["n_result_keys"] = len(keys)
print("RESULT " + json.dumps(out))
'''


@pytest.mark.skipif(not os.path.isdir(os.path.join(REFERENCE, "megatron", "core")), reason="reference checkout absent")
def test_reference_engine_accepts_our_classes():
    import json

    proc = subprocess.run([sys.executable, "-c", CHILD, REFERENCE, ROOT], capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-3000:]
    line = [l for l in proc.stdout.splitlines() if l.startswith("RESULT ")][-1]
    out = json.loads(line[len("RESULT "):])
    assert out["sub"] == [True, True, True, True] and out["same"]
    assert out["shadowed"] == ["add_request"]  # the wrapper that re-raises overflow errors as both families' (see the seam)
    assert out["missing"] == []
    assert out["signature"] == []
    assert out["n_result_keys"] >= 6 and out["result_keys_missing"] == []


def test_seam_needs_the_reference():
    """Without the reference on the path the helper fails with ImportError: nothing is stubbed."""
    code = ("import sys; sys.path.insert(0, %r)\n"
            "from megatron_mixtera_b200.reference_seam import reference_subclasses\n"
            "try:\n    reference_subclasses()\nexcept ImportError:\n    print('IMPORTERROR')\n" % ROOT)
    env = {k: v for k, v in os.environ.items() if k != "PYTHONPATH"}
    proc = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=300, env=env, cwd="/tmp")
    assert "IMPORTERROR" in proc.stdout, proc.stdout + proc.stderr[-2000:]


API_CHILD = r'''
import dataclasses, importlib, inspect, json, os, sys
ref, root = sys.argv[1], sys.argv[2]
sys.path.insert(0, ref); sys.path.insert(0, root)
os.environ.setdefault("TORCHDYNAMO_DISABLE", "1")
import torch
torch.cuda.current_device = lambda: torch.device("cpu")
R, O = "megatron.core.inference.", "megatron_mixtera_b200.inference."
CLASSES = [  # (module path below the inference package - the same in both trees -, class)
    ("engines.dynamic_engine", "DynamicInferenceEngine"),
    ("inference_client", "InferenceClient"),
    ("data_parallel_inference_coordinator", "DataParallelInferenceCoordinator"),
    ("contexts.dynamic_context", "DynamicInferenceContext"),
    ("contexts.dynamic_chunk_allocator", "ChunkAllocator"),
    ("text_generation_controllers.text_generation_controller", "TextGenerationController"),
    ("text_generation_controllers.simple_text_generation_controller", "SimpleTextGenerationController"),
    ("model_inference_wrappers.gpt.gpt_inference_wrapper", "GPTInferenceWrapper"),
]
RECORDS = [("sampling_params", "SamplingParams"), ("common_inference_params", "CommonInferenceParams"),
           ("inference_request", "DynamicInferenceRequest"),
           ("model_inference_wrappers.inference_wrapper_config", "InferenceWrapperConfig")]
def sig(f):
    return [(p.name, p.kind.name, repr(p.default)) for p in inspect.signature(f).parameters.values()]
out = {"missing": {}, "incompatible": {}, "fields": {}}
for module, name in CLASSES:
    theirs, ours = getattr(importlib.import_module(R + module), name), getattr(importlib.import_module(O + module), name)
    if name != theirs.__name__:  # a second name of a class compared above: it only has to resolve to the same class
        assert ours.__name__ == theirs.__name__, (name, ours, theirs)
        continue
    for n, f in inspect.getmembers(theirs, predicate=inspect.isfunction):
        if n.startswith("_") and n != "__init__":
            continue
        g = getattr(ours, n, None)
        if g is None:
            if n not in out["missing"].setdefault(name, []):
                out["missing"][name].append(n)
            continue
        a, b = sig(f), sig(g)
        extras = b[len(a):]
        # a call written for the reference must mean the same here: same leading parameters, additions optional
        if b[:len(a)] != a or any(d == repr(inspect.Parameter.empty) and k not in ("VAR_POSITIONAL", "VAR_KEYWORD") for _, k, d in extras):
            out["incompatible"].setdefault(name, []).append(n)
for module, name in RECORDS:
    theirs, ours = getattr(importlib.import_module(R + module), name), getattr(importlib.import_module(O + module), name)
    a = {f.name for f in dataclasses.fields(theirs)}
    b = {f.name for f in dataclasses.fields(ours)}
    out["fields"][name] = [sorted(a - b), sorted(b - a)]
# parallel_state functions the reference's dynamic-inference modules call
import re
import megatron_mixtera_b200.parallel_state as ours_ps
used = set()
for rel in ("engines/dynamic_engine.py", "contexts/dynamic_context.py", "text_generation_controllers/text_generation_controller.py",
            "model_inference_wrappers/abstract_model_inference_wrapper.py", "model_inference_wrappers/gpt/gpt_inference_wrapper.py"):
    used |= set(re.findall(r"parallel_state\.([a-z_]+)", open(os.path.join(ref, "megatron/core/inference", rel)).read()))
out["parallel_state_missing"] = sorted(n for n in used if not hasattr(ours_ps, n))
print("RESULT " + json.dumps(out))
'''


@pytest.mark.skipif(not os.path.isdir(os.path.join(REFERENCE, "megatron", "core")), reason="reference checkout absent")
def test_public_methods_and_records_cover_the_reference_api():
    """Every public method of the reference's classes on the dynamic-inference path exists here under the same name, and
    a call written against the reference binds the same way (same leading parameters; what this package adds is optional).
    What is absent is listed: static batching and pipeline parallelism, which are outside this path."""
    import json

    proc = subprocess.run([sys.executable, "-c", API_CHILD, REFERENCE, ROOT], capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-3000:]
    out = json.loads([l for l in proc.stdout.splitlines() if l.startswith("RESULT ")][-1][len("RESULT "):])
    assert out["incompatible"] == {}, out["incompatible"]
    assert out["parallel_state_missing"] == [], out["parallel_state_missing"]
    assert out["missing"] == {
        "TextGenerationController": [  # the static-batching generation loop and its helpers
            "detokenize_generations", "generate_all_output_tokens_static_batch", "pad_input_prompt_tokens",
            "prep_inference_input", "stream_tokens", "unpad_input_prompt_tokens", "update_generation_status"],
        "GPTInferenceWrapper": [  # static batching and pipeline-parallel forward passes
            "forward_pass_with_pipeline_parallel_large_input_batch", "forward_pass_with_pipeline_parallel_small_input_batch",
            "forward_pass_without_pipeline_parallel", "get_batch_for_context_window", "prep_inference_input"],
    }, out["missing"]
    assert out["fields"] == {name: [[], []] for name in ("SamplingParams", "CommonInferenceParams", "DynamicInferenceRequest",
                                                        "InferenceWrapperConfig")}, out["fields"]


ENGINE_CHILD = r'''
import json, os, sys, time
ref, root = sys.argv[1], sys.argv[2]
sys.path.insert(0, ref); sys.path.insert(0, root); sys.path.insert(0, os.path.join(root, "tests"))
os.environ.setdefault("TORCHDYNAMO_DISABLE", "1")
import torch
torch.cuda.current_device = lambda: torch.device("cpu")


class HostEvent:  # the reference engine times a step with CUDA events
    def __init__(self, *a, **k):
        self.t = 0.0
    def record(self):
        self.t = time.perf_counter()
    def synchronize(self):
        pass
    def elapsed_time(self, other):
        return (other.t - self.t) * 1e3


torch.cuda.Event = HostEvent
import megatron.core.inference.engines.dynamic_engine as ref_engine
ref_engine.range_push = lambda *a, **k: None
ref_engine.range_pop = lambda *a, **k: None
from megatron.core.inference.sampling_params import SamplingParams as RefSamplingParams
from megatron_mixtera_b200.reference_seam import reference_subclasses
import test_engine_host as H

Context, Controller = reference_subclasses()


class HostController(Controller):
    def sample_from_logits(self, last_token_logits, sampling_params=None, vocab_size=None, **kwargs):
        return torch.argmax(last_token_logits, dim=-1)


def run(buffer_size_gb):
    Context.TOKEN_ROUNDER, Context.REQUEST_ROUNDER = 4, 4
    ctx = Context(params_dtype=torch.float32, num_layers=2, kv_channels=8, num_attention_heads=2, max_sequence_length=96,
                  buffer_size_gb=buffer_size_gb, buffer_guaranteed_fraction=0.1, chunk_size_tokens=16,
                  tensor_model_parallel_size=1, max_requests_override=8, max_tokens_override=128, device="cpu",
                  allocate_memory_buffer=False)
    model = H.StandInModel(ctx)
    engine = ref_engine.DynamicInferenceEngine(HostController(model, tokenizer=__import__("serving_helpers").CharTokenizer(H.VOCAB)), ctx, termination_id=H.EOD, random_seed=0)
    prompts = H.prompts_of(0, 14)
    finished = engine.generate(list(prompts), RefSamplingParams(top_k=1, num_tokens_to_generate=24))
    got = {r.request_id: [int(t) for t in r.generated_tokens] for r in finished}
    want = {i: H.expected_completion(p, 24) for i, p in enumerate(prompts)}
    return {"equal": got == want, "n": len(got), "steps": len(model.steps), "paused_seen": any(p for _, _, p in model.steps),
            "engine": type(engine).__module__}


print("RESULT " + json.dumps({"roomy": run(0.01), "starved": run(0.0001)}))
'''


@pytest.mark.skipif(not os.path.isdir(os.path.join(REFERENCE, "megatron", "core")), reason="reference checkout absent")
def test_reference_engine_drives_our_context_and_controller():
    """The REFERENCE's `DynamicInferenceEngine` (its queueing, stepping and post-processing, unmodified) around this
    package's context and controller step, on the CPU: the model is the stand-in of `test_engine_host` (next token from
    the request's own last token and position), CUDA events and NVTX ranges are replaced by host stand-ins.  Every request
    must complete with its own tokens through a roomy pool and through one so small that requests wait and are paused -
    which needs the overflow errors of `add_request` to be the ones the reference engine catches."""
    import json

    proc = subprocess.run([sys.executable, "-c", ENGINE_CHILD, REFERENCE, ROOT], capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-3000:]
    out = json.loads([l for l in proc.stdout.splitlines() if l.startswith("RESULT ")][-1][len("RESULT "):])
    for case in ("roomy", "starved"):
        assert out[case]["engine"] == "megatron.core.inference.engines.dynamic_engine"
        assert out[case]["equal"] and out[case]["n"] == 14, out
    assert out["starved"]["paused_seen"] and not out["roomy"]["paused_seen"]
