"""zigfa API served by the B200-native library (libb200fa.so): same callables, arguments and autograd behaviour as
the reference package (reference src/zigfa/__init__.py:1-23). Importing this package imports neither torch nor CUDA."""
from .torch import (
    InterSequenceMetadata,
    flash_attn_func,
    flash_attn_inter_sequence_func,
    flash_attn_inter_sequence_kvpacked_func,
    flash_attn_kvpacked_func,
    flash_attn_qkvpacked_func,
    flash_attn_varlen_func,
    flash_attn_varlen_kvpacked_func,
    prepare_inter_sequence_metadata,
)

__all__ = [
    "InterSequenceMetadata",
    "flash_attn_func",
    "flash_attn_inter_sequence_func",
    "flash_attn_inter_sequence_kvpacked_func",
    "flash_attn_kvpacked_func",
    "flash_attn_qkvpacked_func",
    "flash_attn_varlen_func",
    "flash_attn_varlen_kvpacked_func",
    "prepare_inter_sequence_metadata",
]
