"""`SimpleTextGenerationController`, the reference's second name of the controller
(``megatron/core/inference/text_generation_controllers/simple_text_generation_controller.py``; its dynamic engine asserts
against this name)."""
from .text_generation_controller import TextGenerationController as SimpleTextGenerationController

__all__ = ["SimpleTextGenerationController"]
