"""Classes that the reference's own engine accepts.

`DynamicInferenceEngine.__init__` of the reference asserts ``isinstance(controller, SimpleTextGenerationController)``
and ``isinstance(context, DynamicInferenceContext)`` (megatron/core/inference/engines/dynamic_engine.py:107-108)
against ITS classes.  This package's context and controller mirror those classes method for method but do not import
the reference (it is not a dependency).  Where the reference is installed next to this package,
`reference_subclasses()` derives, once, a context and a controller class from BOTH families - this package's class
first in the method resolution order, so every method and attribute resolves to the CUDA-backed implementation, the
reference's class second, so the engine's assertions hold.  Construct them with this package's constructor arguments.

Nothing here touches the decode path; without the reference installed the function raises ImportError.
"""
from __future__ import annotations

from typing import Tuple

_classes = None


def reference_subclasses() -> Tuple[type, type]:
    """(context class, controller class) that are subclasses of both this package's and the reference's classes."""
    global _classes
    if _classes is not None:
        return _classes
    from megatron.core.inference.contexts.dynamic_context import DynamicInferenceContext as RefContext
    from megatron.core.inference.text_generation_controllers.simple_text_generation_controller import (
        SimpleTextGenerationController as RefController,
    )

    from .inference.contexts.dynamic_context import DynamicInferenceContext
    from .inference.text_generation_controllers.text_generation_controller import TextGenerationController

    context_cls = type("B200DynamicInferenceContext", (DynamicInferenceContext, RefContext), {
        "__doc__": "This package's dynamic context, also an instance of the reference's DynamicInferenceContext.",
        "__module__": __name__,
    })
    controller_cls = type("B200TextGenerationController", (TextGenerationController, RefController), {
        "__doc__": "This package's controller, also an instance of the reference's SimpleTextGenerationController.",
        "__module__": __name__,
    })
    _classes = (context_cls, controller_cls)
    return _classes
