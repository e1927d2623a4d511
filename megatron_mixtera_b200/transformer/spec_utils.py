"""Module specs: a class plus constructor params plus submodule specs, built on demand
(the mechanism of the reference's ``megatron/core/transformer/spec_utils.py``)."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Optional, Union


@dataclass
class ModuleSpec:
    module: type
    params: dict = field(default_factory=dict)
    submodules: Any = None


def build_module(spec_or_module: Union[ModuleSpec, type, None], *args, **kwargs):
    """Instantiate ``spec.module(*args, **spec.params, **kwargs, submodules=spec.submodules)``."""
    if spec_or_module is None:
        return None
    if isinstance(spec_or_module, ModuleSpec):
        kw = dict(spec_or_module.params)
        kw.update(kwargs)
        if spec_or_module.submodules is not None:
            kw["submodules"] = spec_or_module.submodules
        return spec_or_module.module(*args, **kw)
    return spec_or_module(*args, **kwargs)
