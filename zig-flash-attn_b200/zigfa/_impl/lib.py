"""ctypes binding of libb200fa.so (declared in include/b200fa.h).

Takes the place of the reference's runtime module (reference src/zigfa/_impl/runtime.py:168-259): instead of
loading one cubin per kernel instance and launching it through cuda.core, the host layer calls a handful of C
entry points that validate, plan and enqueue the sm_100a kernels. There is no fallback: if the shared library is
missing, loading raises.
"""
from __future__ import annotations

import ctypes
import functools
from pathlib import Path

import os

# B200FA_LIBRARY points at another build of the library (tuning builds); the default is the one next to the package.
LIBRARY_PATH = Path(os.environ.get("B200FA_LIBRARY") or Path(__file__).resolve().parent.parent / "libb200fa.so")

EXPORTS = (
    "b200fa_fwd_workspace_bytes",
    "b200fa_fwd",
    "b200fa_fwd_noalloc",
    "b200fa_bwd_workspace_bytes",
    "b200fa_bwd",
    "b200fa_bwd_timing_events",
    "b200fa_set_pivot_ds",
    "b200fa_set_trace",
    "b200fa_interseq_metadata",
    "b200fa_work_list",
    "b200fa_work_list_entries",
    "b200fa_work_list_host",
    "b200fa_interseq_metadata_host",
    "b200fa_key_blocks_host",
    "b200fa_query_blocks_host",
    "b200fa_device_status",
    "b200fa_last_error",
    "b200fa_version",
    "b200fa_supports_head_dim",
)

int32_p = ctypes.POINTER(ctypes.c_int32)


class Problem(ctypes.Structure):
    _fields_ = [
        ("batch", ctypes.c_int32),
        ("seqlen_q", ctypes.c_int32),
        ("seqlen_k", ctypes.c_int32),
        ("heads_q", ctypes.c_int32),
        ("heads_kv", ctypes.c_int32),
        ("head_dim", ctypes.c_int32),
        ("window_left", ctypes.c_int32),
        ("window_right", ctypes.c_int32),
        ("softmax_scale", ctypes.c_float),
        ("cu_seqlens_q", ctypes.c_void_p),
        ("cu_seqlens_k", ctypes.c_void_p),
        ("visibility_bits", ctypes.c_void_p),
        ("visibility_bits_t", ctypes.c_void_p),
        ("cu_visible_k", ctypes.c_void_p),
        ("cu_visible_q", ctypes.c_void_p),
        ("window_sizes", ctypes.c_void_p),
    ]


Stride3 = ctypes.c_int64 * 3
Stride2 = ctypes.c_int64 * 2


class FwdArgs(ctypes.Structure):
    _fields_ = [
        ("problem", Problem),
        ("q", ctypes.c_void_p),
        ("k", ctypes.c_void_p),
        ("v", ctypes.c_void_p),
        ("out", ctypes.c_void_p),
        ("softmax_lse", ctypes.c_void_p),
        ("q_stride", Stride3),
        ("k_stride", Stride3),
        ("v_stride", Stride3),
        ("out_stride", Stride3),
        ("lse_stride", Stride2),
        ("workspace", ctypes.c_void_p),
        ("workspace_bytes", ctypes.c_size_t),
    ]


class BwdArgs(ctypes.Structure):
    _fields_ = [
        ("problem", Problem),
        ("q", ctypes.c_void_p),
        ("k", ctypes.c_void_p),
        ("v", ctypes.c_void_p),
        ("out", ctypes.c_void_p),
        ("dout", ctypes.c_void_p),
        ("softmax_lse", ctypes.c_void_p),
        ("dq", ctypes.c_void_p),
        ("dk", ctypes.c_void_p),
        ("dv", ctypes.c_void_p),
        ("q_stride", Stride3),
        ("k_stride", Stride3),
        ("v_stride", Stride3),
        ("out_stride", Stride3),
        ("dout_stride", Stride3),
        ("dq_stride", Stride3),
        ("dk_stride", Stride3),
        ("dv_stride", Stride3),
        ("lse_stride", Stride2),
        ("workspace", ctypes.c_void_p),
        ("workspace_bytes", ctypes.c_size_t),
    ]


class LibraryError(RuntimeError):
    pass


@functools.cache
def library() -> ctypes.CDLL:
    if not LIBRARY_PATH.exists():
        raise LibraryError(
            f"{LIBRARY_PATH} is missing: build it with `python zig-flash-attn_b200/build.py`; there is no fallback path"
        )
    lib = ctypes.CDLL(str(LIBRARY_PATH))
    lib.b200fa_fwd_workspace_bytes.restype = ctypes.c_size_t
    lib.b200fa_fwd_workspace_bytes.argtypes = [ctypes.POINTER(Problem)]
    lib.b200fa_fwd.restype = ctypes.c_int
    lib.b200fa_fwd.argtypes = [ctypes.POINTER(FwdArgs), ctypes.c_void_p]
    lib.b200fa_fwd_noalloc.restype = ctypes.c_int
    lib.b200fa_fwd_noalloc.argtypes = [ctypes.POINTER(FwdArgs), ctypes.c_void_p]
    lib.b200fa_bwd_workspace_bytes.restype = ctypes.c_size_t
    lib.b200fa_bwd_workspace_bytes.argtypes = [ctypes.POINTER(Problem)]
    lib.b200fa_bwd.restype = ctypes.c_int
    lib.b200fa_bwd.argtypes = [ctypes.POINTER(BwdArgs), ctypes.c_void_p]
    lib.b200fa_bwd_timing_events.restype = ctypes.c_int
    lib.b200fa_bwd_timing_events.argtypes = [ctypes.POINTER(ctypes.c_void_p)]
    lib.b200fa_set_pivot_ds.restype = ctypes.c_int
    lib.b200fa_set_pivot_ds.argtypes = [ctypes.c_int]
    lib.b200fa_set_trace.restype = ctypes.c_int
    lib.b200fa_set_trace.argtypes = [ctypes.c_void_p]
    lib.b200fa_interseq_metadata.restype = ctypes.c_int
    lib.b200fa_interseq_metadata.argtypes = [ctypes.c_void_p] * 3 + [ctypes.c_int32] + [ctypes.c_void_p] * 4
    lib.b200fa_work_list.restype = ctypes.c_int
    lib.b200fa_work_list.argtypes = [ctypes.c_void_p, ctypes.c_void_p] + [ctypes.c_int32] * 4 + [ctypes.c_void_p] * 2
    lib.b200fa_work_list_entries.restype = ctypes.c_int64
    lib.b200fa_work_list_entries.argtypes = [ctypes.c_int64] * 3
    lib.b200fa_work_list_host.restype = ctypes.c_int
    lib.b200fa_work_list_host.argtypes = [ctypes.c_void_p, ctypes.c_void_p] + [ctypes.c_int32] * 4 + [ctypes.c_void_p]
    lib.b200fa_interseq_metadata_host.restype = ctypes.c_int
    lib.b200fa_interseq_metadata_host.argtypes = [ctypes.c_void_p] * 3 + [ctypes.c_int32] + [ctypes.c_void_p] * 3
    lib.b200fa_key_blocks_host.restype = ctypes.c_int
    lib.b200fa_key_blocks_host.argtypes = [ctypes.POINTER(Problem)] + [ctypes.c_int32] * 3 + [ctypes.c_void_p, ctypes.c_int32]
    lib.b200fa_query_blocks_host.restype = ctypes.c_int
    lib.b200fa_query_blocks_host.argtypes = [ctypes.POINTER(Problem)] + [ctypes.c_int32] * 3 + [ctypes.c_void_p, ctypes.c_int32]
    lib.b200fa_device_status.restype = ctypes.c_int
    lib.b200fa_device_status.argtypes = []
    lib.b200fa_last_error.restype = ctypes.c_char_p
    lib.b200fa_last_error.argtypes = []
    lib.b200fa_version.restype = ctypes.c_int
    lib.b200fa_supports_head_dim.restype = ctypes.c_int
    lib.b200fa_supports_head_dim.argtypes = [ctypes.c_int32, ctypes.c_int32]
    return lib


def last_error() -> str:
    return library().b200fa_last_error().decode()


def check(status: int) -> None:
    """Maps a C return code to the exception the reference's host layer raises for the same condition."""
    if status == 0:
        return
    message = last_error()
    if status == -3:
        raise NotImplementedError(message)
    if status == -1:
        raise ValueError(message)
    raise RuntimeError(message)


def pointer(tensor) -> int | None:
    return None if tensor is None else tensor.data_ptr()


def strides3(tensor, packed: bool) -> Stride3:
    """(batch, row, head) strides in elements of a (batch, row, head, dim) or packed (row, head, dim) tensor."""
    stride = tensor.stride()
    if packed:
        return Stride3(0, stride[0], stride[1])
    return Stride3(stride[0], stride[1], stride[2])


def make_problem(
    q,
    k,
    cu_seqlens_q,
    cu_seqlens_k,
    softmax_scale,
    window_left,
    window_right,
    visibility_bits=None,
    visibility_bits_t=None,
    cu_visible_k=None,
    cu_visible_q=None,
    window_sizes=None,
) -> Problem:
    packed = cu_seqlens_q is not None
    if packed:
        batch, seqlen_q, seqlen_k = cu_seqlens_q.shape[0] - 1, q.shape[0], k.shape[0]
    else:
        batch, seqlen_q, seqlen_k = q.shape[0], q.shape[1], k.shape[1]
    return Problem(
        batch=batch,
        seqlen_q=seqlen_q,
        seqlen_k=seqlen_k,
        heads_q=q.shape[-2],
        heads_kv=k.shape[-2],
        head_dim=q.shape[-1],
        window_left=window_left,
        window_right=window_right,
        softmax_scale=softmax_scale,
        cu_seqlens_q=pointer(cu_seqlens_q),
        cu_seqlens_k=pointer(cu_seqlens_k),
        visibility_bits=pointer(visibility_bits),
        visibility_bits_t=pointer(visibility_bits_t),
        cu_visible_k=pointer(cu_visible_k),
        cu_visible_q=pointer(cu_visible_q),
        window_sizes=pointer(window_sizes),
    )
