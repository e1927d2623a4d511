"""`CommonInferenceParams`, the reference's earlier name of `SamplingParams`
(``megatron/core/inference/common_inference_params.py``)."""
from .sampling_params import SamplingParams as CommonInferenceParams

__all__ = ["CommonInferenceParams"]
