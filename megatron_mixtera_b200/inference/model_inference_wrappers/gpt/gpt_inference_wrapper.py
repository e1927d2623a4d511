"""`GPTInferenceWrapper` under the reference's module path
(``megatron/core/inference/model_inference_wrappers/gpt/gpt_inference_wrapper.py``)."""
from ..gpt_inference_wrapper import GPTInferenceWrapper

__all__ = ["GPTInferenceWrapper"]
