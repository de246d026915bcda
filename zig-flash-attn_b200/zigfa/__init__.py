"""zigfa API served by the B200-native library (libb200fa.so): same callables, arguments and autograd behaviour as
the reference package (reference src/zigfa/__init__.py:1-23). Importing this package imports neither torch nor CUDA."""
from . import torch as _functions
from .torch import *  # noqa: F401,F403  the nine public callables and InterSequenceMetadata

__all__ = list(_functions.__all__)
