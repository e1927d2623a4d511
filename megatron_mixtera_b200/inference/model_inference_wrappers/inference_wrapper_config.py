"""`InferenceWrapperConfig` under the reference's module path
(``megatron/core/inference/model_inference_wrappers/inference_wrapper_config.py``)."""
from .gpt_inference_wrapper import InferenceWrapperConfig

__all__ = ["InferenceWrapperConfig"]
