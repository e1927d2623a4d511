"""Classes that the reference's own engine accepts.

`DynamicInferenceEngine.__init__` of the reference asserts ``isinstance(controller, SimpleTextGenerationController)``
and ``isinstance(context, DynamicInferenceContext)`` (megatron/core/inference/engines/dynamic_engine.py:107-108)
against ITS classes.  This package's context and controller mirror those classes method for method but do not import
the reference (it is not a dependency).  Where the reference is installed next to this package,
`reference_subclasses()` derives, once, a context and a controller class from BOTH families - this package's class
first in the method resolution order, so every method and attribute resolves to the CUDA-backed implementation, the
reference's class second, so the engine's assertions hold.  Construct them with this package's constructor arguments.

The reference engine also catches ITS `ContextOverflowError` around ``context.add_request`` (:383-400) to queue or fail
a request that does not fit.  The derived context therefore re-raises this package's overflow errors as instances of a
class derived from both families' error of the same name (same message, ``request_id`` and ``is_transient``); that
wrapper around ``add_request`` is the one method of the derived classes that is not this package's own function object.

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

    import megatron.core.inference.contexts.dynamic_context as ref_module

    from .inference.contexts.dynamic_context import ContextOverflowError, DynamicInferenceContext
    from .inference.text_generation_controllers.text_generation_controller import TextGenerationController

    dual_errors = {}

    def as_both(error: ContextOverflowError) -> ContextOverflowError:
        ours = type(error)
        if ours not in dual_errors:
            theirs = getattr(ref_module, ours.__name__, ref_module.ContextOverflowError)
            dual_errors[ours] = type(ours.__name__, (ours, theirs), {"__module__": __name__})
        both = dual_errors[ours].__new__(dual_errors[ours])
        both.__dict__.update(error.__dict__)
        both.args = error.args
        return both

    def add_request(self, *args, **kwargs):
        try:
            return DynamicInferenceContext.add_request(self, *args, **kwargs)
        except ContextOverflowError as error:
            raise as_both(error).with_traceback(error.__traceback__) from None

    add_request.__doc__ = DynamicInferenceContext.add_request.__doc__
    context_cls = type("B200DynamicInferenceContext", (DynamicInferenceContext, RefContext), {
        "__doc__": "This package's dynamic context, also an instance of the reference's DynamicInferenceContext.",
        "__module__": __name__,
        "add_request": add_request,
    })
    controller_cls = type("B200TextGenerationController", (TextGenerationController, RefController), {
        "__doc__": "This package's controller, also an instance of the reference's SimpleTextGenerationController.",
        "__module__": __name__,
    })
    _classes = (context_cls, controller_cls)
    return _classes
