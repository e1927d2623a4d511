"""Request-level sampling parameters (same fields and defaults as the reference's
``megatron/core/inference/sampling_params.py:6-25``; ``top_k=0`` means a full multinomial draw and
greedy decoding needs ``top_k=1``)."""
from dataclasses import dataclass


@dataclass
class SamplingParams:
    temperature: float = 1.0
    top_k: int = 0
    top_p: float = 0.0
    return_log_probs: bool = False
    return_segments: bool = False
    num_tokens_to_generate: int = 30
    top_n_logprobs: int = 0
    return_prompt_top_n_logprobs: bool = False

    def add_attributes(self, attribute_value_pair: dict):
        """Attach extra attributes, e.g. ``{'min_length': 4}``."""
        for key, value in attribute_value_pair.items():
            setattr(self, key, value)

    def serializable(self) -> dict:
        return self.__dict__.copy()

    @classmethod
    def deserialize(cls, data: dict) -> "SamplingParams":
        obj = cls()
        obj.add_attributes(data)
        return obj
