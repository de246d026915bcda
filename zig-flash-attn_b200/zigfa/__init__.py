"""zigfa API served by the B200-native library (libb200fa.so): same callables, arguments and autograd behaviour as
the reference package (reference src/zigfa/__init__.py:1-23). Importing this package imports neither torch nor CUDA."""
from . import torch as _functions
from .torch import *  # noqa: F401,F403  the nine public callables and InterSequenceMetadata

__all__ = [*_functions.__all__, "set_pivot_gradients"]


def set_pivot_gradients(enabled: bool) -> bool:
    """Turns the pivot path of the backward pass on or off for this process and returns the previous setting.

    With it on, a key that holds more than 3/4 of the probability of a query row (the pivot) gets its score gradient as
    minus the sum of the rounded score gradients of the other keys of the row instead of P (dP - D), which cancels for
    P near 1: dq, dk of peaked rows then keep the accuracy the reference's backward has (its "softmax fix",
    reference tests/test_softmax_fix.py). The reference always works this way; here it is a setting because it costs the
    backward kernel about 16 %, and it starts off unless the environment has B200FA_PIVOT_DS=1. The forward pass needs no
    setting: its log-sum-exp of peaked rows is always formed accurately."""
    from ._impl import lib

    return bool(lib.library().b200fa_set_pivot_ds(1 if enabled else 0))
