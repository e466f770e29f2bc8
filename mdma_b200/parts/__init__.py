"""Parts a layer is put together from; importing this package registers them."""
from . import attention, block, embedding, mlp, norm, rotary  # noqa: F401
from .base import Part, Runtime
from .linear import Linear

__all__ = ["Part", "Runtime", "Linear"]
