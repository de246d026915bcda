"""Host layer between the public API and the C-ABI library: validation, allocation, torch custom ops with fake
implementations, and the autograd Functions.

Mirrors the behaviour of the reference's op layer (reference src/zigfa/_impl/ops.py): the same custom-op argument
order (ops.py:161-173, 219-234, 274-293, 665-668, 701-716, 807-825, 854-876), the same errors for bad inputs
(ValueError), unsupported options (NotImplementedError naming the option, ops.py:334-371), the same handling of
tensors the kernels cannot read directly (copied to a contiguous buffer, ops.py:38-51), and gradients written
straight into packed buffers (ops.py:418-439). Work is enqueued on the current stream of the tensors' device and
never synchronises. The kernels themselves live in libb200fa.so; if it cannot be loaded every op raises.
"""
from __future__ import annotations

import ctypes
import numbers

import torch

from ..torch import InterSequenceMetadata
from . import lib as _lib

ALIGNMENT_BYTES = 16
ALIGNMENT_ELEMENTS = 8
FORWARD, BACKWARD = 0, 1
CANDIDATE_HEAD_DIMS = (64, 72, 96, 128, 256, 512)


def head_dims(direction: int = FORWARD) -> tuple[int, ...]:
    """Head dimensions the loaded library has kernels for."""
    library = _lib.library()
    return tuple(d for d in CANDIDATE_HEAD_DIMS if library.b200fa_supports_head_dim(d, direction))


# ------------------------------------------------------------------------------------------------ validation
def default_softmax_scale(softmax_scale, head_dim):
    return head_dim**-0.5 if softmax_scale is None else softmax_scale


def require_window(left, right):
    if not (isinstance(left, numbers.Integral) and isinstance(right, numbers.Integral)):
        raise TypeError(
            f"window bounds must be integers, got left={type(left).__name__}, right={type(right).__name__}"
        )
    if left < -1 or right < -1:
        raise ValueError(f"window bounds must each be -1 or non-negative, got left={left}, right={right}")


def kernel_ready(tensor) -> bool:
    """True when the kernels can address the tensor in place: 16-byte aligned base, unit last stride, other strides
    multiples of 8 elements (reference src/zigfa/_impl/tensors.py:114-127)."""
    strides = tensor.stride()
    return (
        tensor.data_ptr() % ALIGNMENT_BYTES == 0
        and strides[-1] == 1
        and all(stride % ALIGNMENT_ELEMENTS == 0 for stride in strides[:-1])
    )


def readable(tensor):
    return tensor if kernel_ready(tensor) else tensor.clone(memory_format=torch.contiguous_format)


def writable(tensor):
    return tensor if kernel_ready(tensor) else tensor.new_empty(tensor.shape)


def lse_shape(q, packed):
    return (q.shape[1], q.shape[0]) if packed else (q.shape[0], q.shape[2], q.shape[1])


def check_cu_seqlens(cu_seqlens_q, cu_seqlens_k):
    for name, value in (("cu_seqlens_q", cu_seqlens_q), ("cu_seqlens_k", cu_seqlens_k)):
        if value.dtype != torch.int32 or value.dim() != 1:
            raise ValueError(f"{name} must be a one-dimensional int32 tensor")
    if cu_seqlens_q.shape != cu_seqlens_k.shape:
        raise ValueError("cu_seqlens_q and cu_seqlens_k must have the same length")


def check_inputs(q, k, v, cu_seqlens_q, cu_seqlens_k, direction=FORWARD):
    packed = cu_seqlens_q is not None
    if packed != (cu_seqlens_k is not None):
        raise ValueError("cu_seqlens_q and cu_seqlens_k must be given together")
    for name, tensor in (("q", q), ("k", k), ("v", v)):
        if tensor.dtype != torch.bfloat16:
            raise ValueError(f"{name} must be bfloat16, got {tensor.dtype}")
    rank = 3 if packed else 4
    for name, tensor in (("q", q), ("k", k), ("v", v)):
        if tensor.dim() != rank:
            raise ValueError(f"{name} must have {rank} dimensions, got {tensor.dim()}")
    if k.shape != v.shape:
        raise ValueError("k and v must have the same shape")
    supported = head_dims(direction)
    if q.shape[-1] != k.shape[-1] or q.shape[-1] not in supported:
        raise ValueError(f"head_dim must be one of {list(supported)} and equal for q and k")
    if q.shape[-2] % k.shape[-2]:
        raise ValueError("the query head count must be a multiple of the key head count (num_heads_q % num_heads_k)")
    if packed:
        check_cu_seqlens(cu_seqlens_q, cu_seqlens_k)
    elif q.shape[0] != k.shape[0]:
        raise ValueError("q and k must have the same batch size")


def check_backward_operands(dout, q, k, v, out, softmax_lse, dq, dk, dv, packed):
    for name, tensor in (("dout", dout), ("out", out), ("dq", dq), ("dk", dk), ("dv", dv)):
        if tensor.dtype != torch.bfloat16:
            raise ValueError(f"{name} must be bfloat16, got {tensor.dtype}")
    if dout.shape != q.shape or out.shape != q.shape or dq.shape != q.shape:
        raise ValueError("dout, out and dq must have the shape of q")
    if dk.shape != k.shape or dv.shape != v.shape:
        raise ValueError("dk and dv must have the shape of k")
    if softmax_lse.dtype != torch.float32 or tuple(softmax_lse.shape) != tuple(lse_shape(q, packed)):
        raise ValueError(
            "softmax_lse must be a float32 tensor shaped (batch, num_heads_q, seqlen_q) or (num_heads_q, total_q)"
        )


def reject_unsupported(**options):
    """Raises NotImplementedError naming the first option this library does not implement."""
    for name in ("qv", "q_descale", "k_descale", "v_descale", "seqused_q", "seqused_k", "alibi_slopes"):
        if options.get(name) is not None:
            raise NotImplementedError(f"{name} is not supported")
    for name, only in (("dropout_p", 0.0), ("attention_chunk", 0), ("softcap", 0.0)):
        value = options.get(name, only)
        if value != only:
            raise NotImplementedError(f"{name}={value} is not supported; only {only} is")
    num_splits = options.get("num_splits", 1)
    if num_splits not in (0, 1):
        raise NotImplementedError(f"num_splits={num_splits} is not supported; only 0 and 1 are")
    if options.get("deterministic", False):
        raise NotImplementedError(
            "deterministic=True is not supported: the backward pass accumulates dQ with floating-point atomics"
        )


# ------------------------------------------------------------------------------------------------ launches
def _stream(device):
    return torch.cuda.current_stream(device).cuda_stream


def _workspace(nbytes, device):
    return torch.empty(max(int(nbytes), 1), dtype=torch.uint8, device=device)


def _contiguous_int(tensor):
    return tensor if tensor is None or tensor.is_contiguous() else tensor.contiguous()


def launch_forward(q, k, v, out, softmax_lse, cu_seqlens_q, cu_seqlens_k, softmax_scale, left, right, interseq=None):
    """out, softmax_lse <- attention(q, k, v). `interseq` = (bits, bits_t, cu_visible_k, cu_visible_q, window_sizes)."""
    packed = cu_seqlens_q is not None
    library = _lib.library()
    problem = _lib.make_problem(q, k, cu_seqlens_q, cu_seqlens_k, softmax_scale, left, right, *(interseq or ()))
    with torch.cuda.device(q.device):
        workspace = _workspace(library.b200fa_fwd_workspace_bytes(ctypes.byref(problem)), q.device)
        args = _lib.FwdArgs(
            problem=problem,
            q=q.data_ptr(),
            k=k.data_ptr(),
            v=v.data_ptr(),
            out=out.data_ptr(),
            softmax_lse=softmax_lse.data_ptr(),
            q_stride=_lib.strides3(q, packed),
            k_stride=_lib.strides3(k, packed),
            v_stride=_lib.strides3(v, packed),
            out_stride=_lib.strides3(out, packed),
            lse_stride=_lib.Stride2(0, softmax_lse.stride(0)) if packed else _lib.Stride2(*softmax_lse.stride()[:2]),
            workspace=workspace.data_ptr(),
            workspace_bytes=workspace.numel(),
        )
        _lib.check(library.b200fa_fwd(ctypes.byref(args), _stream(q.device)))


def launch_backward(
    dout, q, k, v, out, softmax_lse, dq, dk, dv, cu_seqlens_q, cu_seqlens_k, softmax_scale, left, right, interseq=None
):
    packed = cu_seqlens_q is not None
    library = _lib.library()
    problem = _lib.make_problem(q, k, cu_seqlens_q, cu_seqlens_k, softmax_scale, left, right, *(interseq or ()))
    with torch.cuda.device(q.device):
        workspace = _workspace(library.b200fa_bwd_workspace_bytes(ctypes.byref(problem)), q.device)
        strides = {
            name + "_stride": _lib.strides3(tensor, packed)
            for name, tensor in dict(q=q, k=k, v=v, out=out, dout=dout, dq=dq, dk=dk, dv=dv).items()
        }
        args = _lib.BwdArgs(
            problem=problem,
            q=q.data_ptr(),
            k=k.data_ptr(),
            v=v.data_ptr(),
            out=out.data_ptr(),
            dout=dout.data_ptr(),
            softmax_lse=softmax_lse.data_ptr(),
            dq=dq.data_ptr(),
            dk=dk.data_ptr(),
            dv=dv.data_ptr(),
            lse_stride=_lib.Stride2(0, softmax_lse.stride(0)) if packed else _lib.Stride2(*softmax_lse.stride()[:2]),
            workspace=workspace.data_ptr(),
            workspace_bytes=workspace.numel(),
            **strides,
        )
        _lib.check(library.b200fa_bwd(ctypes.byref(args), _stream(q.device)))


def forward_impl(q, k, v, cu_seqlens_q, cu_seqlens_k, softmax_scale, left, right, interseq=None, direction=FORWARD):
    check_inputs(q, k, v, cu_seqlens_q, cu_seqlens_k, direction)
    require_window(left, right)
    q, k, v = (readable(tensor) for tensor in (q, k, v))
    packed = cu_seqlens_q is not None
    out = q.new_empty(q.shape)
    softmax_lse = q.new_empty(lse_shape(q, packed), dtype=torch.float32)
    launch_forward(
        q, k, v, out, softmax_lse, _contiguous_int(cu_seqlens_q), _contiguous_int(cu_seqlens_k), softmax_scale, left,
        right, interseq,
    )
    return out, softmax_lse


def backward_into(
    dout, q, k, v, out, softmax_lse, cu_seqlens_q, cu_seqlens_k, softmax_scale, left, right, dq, dk, dv, interseq=None
):
    packed = cu_seqlens_q is not None
    check_inputs(q, k, v, cu_seqlens_q, cu_seqlens_k, BACKWARD)
    check_backward_operands(dout, q, k, v, out, softmax_lse, dq, dk, dv, packed)
    require_window(left, right)
    dout, q, k, v, out = (readable(tensor) for tensor in (dout, q, k, v, out))
    softmax_lse = softmax_lse.contiguous()
    targets = (dq, dk, dv)
    buffers = tuple(writable(tensor) for tensor in targets)
    launch_backward(
        dout, q, k, v, out, softmax_lse, *buffers, _contiguous_int(cu_seqlens_q), _contiguous_int(cu_seqlens_k),
        softmax_scale, left, right, interseq,
    )
    for target, buffer in zip(targets, buffers):
        if buffer is not target:
            target.copy_(buffer)


# ------------------------------------------------------------------------------------------------ custom ops
@torch.library.custom_op("zigfa::flash_attn_forward", mutates_args=(), device_types="cuda")
def flash_attn_forward(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    cu_seqlens_q: torch.Tensor | None,
    cu_seqlens_k: torch.Tensor | None,
    max_seqlen_q: int | None,
    max_seqlen_k: int | None,
    softmax_scale: float,
    window_size_left: int,
    window_size_right: int,
) -> tuple[torch.Tensor, torch.Tensor]:
    return forward_impl(q, k, v, cu_seqlens_q, cu_seqlens_k, softmax_scale, window_size_left, window_size_right)


@flash_attn_forward.register_fake
def _(q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, softmax_scale, window_size_left, window_size_right):
    return q.new_empty(q.shape), q.new_empty(lse_shape(q, cu_seqlens_q is not None), dtype=torch.float32)


@torch.library.custom_op("zigfa::flash_attn_backward", mutates_args=(), device_types="cuda")
def flash_attn_backward(
    dout: torch.Tensor,
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    out: torch.Tensor,
    softmax_lse: torch.Tensor,
    cu_seqlens_q: torch.Tensor | None,
    cu_seqlens_k: torch.Tensor | None,
    max_seqlen_q: int | None,
    max_seqlen_k: int | None,
    softmax_scale: float,
    window_size_left: int,
    window_size_right: int,
) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    dq, dk, dv = q.new_empty(q.shape), k.new_empty(k.shape), v.new_empty(v.shape)
    backward_into(
        dout, q, k, v, out, softmax_lse, cu_seqlens_q, cu_seqlens_k, softmax_scale, window_size_left,
        window_size_right, dq, dk, dv,
    )
    return dq, dk, dv


@flash_attn_backward.register_fake
def _(dout, q, k, v, *unused):
    return q.new_empty(q.shape), k.new_empty(k.shape), v.new_empty(v.shape)


def split_qkv(qkv, num_heads_q):
    if qkv.dim() == 5:
        if qkv.shape[-3] != 3:
            raise ValueError(f"a five-dimensional qkv must have size 3 in dimension -3, got {qkv.shape[-3]}")
        return qkv.unbind(dim=-3)
    if qkv.dim() != 4 or num_heads_q is None:
        raise ValueError("qkv must have five dimensions, or four dimensions together with num_heads_q")
    num_heads_k, remainder = divmod(qkv.shape[2] - num_heads_q, 2)
    if remainder or num_heads_k < 0:
        raise ValueError("qkv head dimension must equal num_heads_q plus twice the key head count")
    return qkv.split([num_heads_q, num_heads_k, num_heads_k], dim=-2)


def gradient_views(q, dq, dpacked):
    """(dq, dk, dv) views into the packed gradient buffer: dqkv when dq is None, else (dq, dkv)."""
    if dq is None:
        return split_qkv(dpacked, q.shape[-2])
    dk, dv = dpacked.unbind(dim=-3)
    return dq, dk, dv


@torch.library.custom_op("zigfa::flash_attn_backward_packed", mutates_args=("dq", "dpacked"), device_types="cuda")
def flash_attn_backward_packed(
    dout: torch.Tensor,
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    out: torch.Tensor,
    softmax_lse: torch.Tensor,
    cu_seqlens_q: torch.Tensor | None,
    cu_seqlens_k: torch.Tensor | None,
    max_seqlen_q: int | None,
    max_seqlen_k: int | None,
    softmax_scale: float,
    window_size_left: int,
    window_size_right: int,
    dq: torch.Tensor | None,
    dpacked: torch.Tensor,
) -> None:
    backward_into(
        dout, q, k, v, out, softmax_lse, cu_seqlens_q, cu_seqlens_k, softmax_scale, window_size_left,
        window_size_right, *gradient_views(q, dq, dpacked),
    )


@flash_attn_backward_packed.register_fake
def _(*unused):
    return None


# ---- inter-sequence
def words_per_row(num_sequences):
    return (num_sequences + 31) // 32


def check_int32(name, tensor, shape):
    if tensor.dtype != torch.int32 or tuple(tensor.shape) != tuple(shape) or not tensor.is_contiguous():
        raise ValueError(
            f"{name} must be a contiguous int32 tensor of shape {tuple(shape)}, got {tensor.dtype} {tuple(tensor.shape)}"
        )


def check_inter_sequence_layout(cu_seqlens_q, cu_seqlens_k, visibility_bits, window_sizes=None):
    check_cu_seqlens(cu_seqlens_q, cu_seqlens_k)
    count = cu_seqlens_q.shape[0] - 1
    if count < 1:
        raise ValueError("cu_seqlens_q must describe at least one sequence")
    check_int32("visibility_bits", visibility_bits, (count, words_per_row(count)))
    if window_sizes is not None:
        check_int32("window_sizes", window_sizes, (2, count))
    return count


def metadata_buffers(cu_seqlens_q):
    count = cu_seqlens_q.shape[0] - 1
    return (
        cu_seqlens_q.new_empty((count, words_per_row(count))),
        cu_seqlens_q.new_empty((count + 1,)),
        cu_seqlens_q.new_empty((count + 1,)),
    )


@torch.library.custom_op("zigfa::inter_sequence_metadata", mutates_args=(), device_types="cuda")
def inter_sequence_metadata(
    cu_seqlens_q: torch.Tensor, cu_seqlens_k: torch.Tensor, visibility_bits: torch.Tensor
) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    count = check_inter_sequence_layout(cu_seqlens_q, cu_seqlens_k, visibility_bits)
    bits_t, cu_visible_k, cu_visible_q = metadata_buffers(cu_seqlens_q)
    cu_seqlens_q, cu_seqlens_k = _contiguous_int(cu_seqlens_q), _contiguous_int(cu_seqlens_k)
    with torch.cuda.device(visibility_bits.device):
        _lib.check(
            _lib.library().b200fa_interseq_metadata(
                cu_seqlens_q.data_ptr(), cu_seqlens_k.data_ptr(), visibility_bits.data_ptr(), count, bits_t.data_ptr(),
                cu_visible_k.data_ptr(), cu_visible_q.data_ptr(), _stream(visibility_bits.device),
            )
        )
    return bits_t, cu_visible_k, cu_visible_q


@inter_sequence_metadata.register_fake
def _(cu_seqlens_q, cu_seqlens_k, visibility_bits):
    return metadata_buffers(cu_seqlens_q)


def prepare_inter_sequence_metadata(cu_seqlens_q, cu_seqlens_k, visibility_bits):
    return InterSequenceMetadata(inter_sequence_metadata(cu_seqlens_q, cu_seqlens_k, visibility_bits))


def inter_sequence_head_dims(direction=FORWARD):
    return head_dims(direction)


def check_inter_sequence_head_dim(q, direction):
    supported = inter_sequence_head_dims(direction)
    if q.shape[-1] not in supported and q.shape[-1] in CANDIDATE_HEAD_DIMS:
        raise NotImplementedError(
            f"inter-sequence attention supports head_dim {list(supported)} on this device, got {q.shape[-1]}"
        )


@torch.library.custom_op("zigfa::inter_sequence_forward", mutates_args=(), device_types="cuda")
def inter_sequence_forward(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    cu_seqlens_q: torch.Tensor,
    cu_seqlens_k: torch.Tensor,
    visibility_bits: torch.Tensor,
    visibility_bits_t: torch.Tensor,
    cu_visible_k: torch.Tensor,
    cu_visible_q: torch.Tensor,
    window_sizes: torch.Tensor | None,
    softmax_scale: float,
    window_size_left: int,
    window_size_right: int,
) -> tuple[torch.Tensor, torch.Tensor]:
    check_inter_sequence_head_dim(q, FORWARD)
    check_inputs(q, k, v, cu_seqlens_q, cu_seqlens_k, FORWARD)
    check_inter_sequence_layout(cu_seqlens_q, cu_seqlens_k, visibility_bits, window_sizes)
    interseq = (visibility_bits, visibility_bits_t, cu_visible_k, cu_visible_q, window_sizes)
    return forward_impl(q, k, v, cu_seqlens_q, cu_seqlens_k, softmax_scale, window_size_left, window_size_right, interseq)


@inter_sequence_forward.register_fake
def _(q, k, v, *unused):
    return q.new_empty(q.shape), q.new_empty(lse_shape(q, True), dtype=torch.float32)


def inter_sequence_backward_into(
    dout, q, k, v, out, softmax_lse, cu_seqlens_q, cu_seqlens_k, visibility_bits, visibility_bits_t, cu_visible_k,
    cu_visible_q, window_sizes, softmax_scale, left, right, dq, dk, dv,
):
    check_inter_sequence_head_dim(q, BACKWARD)
    check_inter_sequence_layout(cu_seqlens_q, cu_seqlens_k, visibility_bits, window_sizes)
    interseq = (visibility_bits, visibility_bits_t, cu_visible_k, cu_visible_q, window_sizes)
    backward_into(
        dout, q, k, v, out, softmax_lse, cu_seqlens_q, cu_seqlens_k, softmax_scale, left, right, dq, dk, dv, interseq
    )


@torch.library.custom_op("zigfa::inter_sequence_backward", mutates_args=(), device_types="cuda")
def inter_sequence_backward(
    dout: torch.Tensor,
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    out: torch.Tensor,
    softmax_lse: torch.Tensor,
    cu_seqlens_q: torch.Tensor,
    cu_seqlens_k: torch.Tensor,
    visibility_bits: torch.Tensor,
    visibility_bits_t: torch.Tensor,
    cu_visible_k: torch.Tensor,
    cu_visible_q: torch.Tensor,
    window_sizes: torch.Tensor | None,
    softmax_scale: float,
    window_size_left: int,
    window_size_right: int,
) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    dq, dk, dv = q.new_empty(q.shape), k.new_empty(k.shape), v.new_empty(v.shape)
    inter_sequence_backward_into(
        dout, q, k, v, out, softmax_lse, cu_seqlens_q, cu_seqlens_k, visibility_bits, visibility_bits_t, cu_visible_k,
        cu_visible_q, window_sizes, softmax_scale, window_size_left, window_size_right, dq, dk, dv,
    )
    return dq, dk, dv


@inter_sequence_backward.register_fake
def _(dout, q, k, v, *unused):
    return q.new_empty(q.shape), k.new_empty(k.shape), v.new_empty(v.shape)


@torch.library.custom_op(
    "zigfa::inter_sequence_backward_packed", mutates_args=("dq", "dpacked"), device_types="cuda"
)
def inter_sequence_backward_packed(
    dout: torch.Tensor,
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    out: torch.Tensor,
    softmax_lse: torch.Tensor,
    cu_seqlens_q: torch.Tensor,
    cu_seqlens_k: torch.Tensor,
    visibility_bits: torch.Tensor,
    visibility_bits_t: torch.Tensor,
    cu_visible_k: torch.Tensor,
    cu_visible_q: torch.Tensor,
    window_sizes: torch.Tensor | None,
    softmax_scale: float,
    window_size_left: int,
    window_size_right: int,
    dq: torch.Tensor,
    dpacked: torch.Tensor,
) -> None:
    inter_sequence_backward_into(
        dout, q, k, v, out, softmax_lse, cu_seqlens_q, cu_seqlens_k, visibility_bits, visibility_bits_t, cu_visible_k,
        cu_visible_q, window_sizes, softmax_scale, window_size_left, window_size_right,
        *gradient_views(q, dq, dpacked),
    )


@inter_sequence_backward_packed.register_fake
def _(*unused):
    return None


# ------------------------------------------------------------------------------------------------ autograd
def _pad(ctx, *gradients):
    return (*gradients, *(None,) * (len(ctx.needs_input_grad) - len(gradients)))


def _run_forward(ctx, q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, softmax_scale, causal, window_size,
                 return_softmax):
    softmax_scale = default_softmax_scale(softmax_scale, q.shape[-1])
    left, right = window_size
    require_window(left, right)
    window = (left, 0 if causal else right)
    if cu_seqlens_q is None:
        max_seqlen_q, max_seqlen_k = q.shape[1], k.shape[1]
    out, softmax_lse = flash_attn_forward(
        q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, softmax_scale, *window
    )
    ctx.save_for_backward(q, k, v, out, softmax_lse, cu_seqlens_q, cu_seqlens_k)
    ctx.hints = (max_seqlen_q, max_seqlen_k)
    ctx.softmax_scale = softmax_scale
    ctx.window = window
    if not return_softmax:
        return out
    ctx.mark_non_differentiable(softmax_lse)
    return out, softmax_lse


def _backward_arguments(ctx, dout):
    return (dout, *ctx.saved_tensors, *ctx.hints, ctx.softmax_scale, *ctx.window)


def _stacked(tensor, count):
    return (*tensor.shape[:-2], count, *tensor.shape[-2:])


def _kvpacked_backward(ctx, dout):
    arguments = _backward_arguments(ctx, dout)
    q, k = arguments[1], arguments[2]
    dq, dkv = q.new_empty(q.shape), k.new_empty(_stacked(k, 2))
    flash_attn_backward_packed(*arguments, dq, dkv)
    return _pad(ctx, dq, dkv)


class FlashAttnFunc(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, softmax_scale, causal, qv=None, q_descale=None, k_descale=None, v_descale=None,
                window_size=(-1, -1), attention_chunk=0, softcap=0.0, num_splits=1, pack_gqa=None, deterministic=False,
                sm_margin=0, return_attn_probs=False):
        reject_unsupported(qv=qv, q_descale=q_descale, k_descale=k_descale, v_descale=v_descale,
                           attention_chunk=attention_chunk, softcap=softcap, num_splits=num_splits,
                           deterministic=deterministic)
        return _run_forward(ctx, q, k, v, None, None, None, None, softmax_scale, causal, window_size, return_attn_probs)

    @staticmethod
    def backward(ctx, dout, *unused):
        return _pad(ctx, *flash_attn_backward(*_backward_arguments(ctx, dout)))


class FlashAttnVarlenFunc(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, seqused_q=None, seqused_k=None,
                softmax_scale=None, causal=False, qv=None, q_descale=None, k_descale=None, v_descale=None,
                window_size=(-1, -1), attention_chunk=0, softcap=0.0, num_splits=1, pack_gqa=None, deterministic=False,
                sm_margin=0, return_attn_probs=False):
        reject_unsupported(qv=qv, q_descale=q_descale, k_descale=k_descale, v_descale=v_descale, seqused_q=seqused_q,
                           seqused_k=seqused_k, attention_chunk=attention_chunk, softcap=softcap, num_splits=num_splits,
                           deterministic=deterministic)
        return _run_forward(ctx, q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, softmax_scale, causal,
                            window_size, return_attn_probs)

    @staticmethod
    def backward(ctx, dout, *unused):
        return _pad(ctx, *flash_attn_backward(*_backward_arguments(ctx, dout)))


class FlashAttnQKVPackedFunc(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv, softmax_scale, causal, q_descale=None, k_descale=None, v_descale=None, window_size=(-1, -1),
                attention_chunk=0, softcap=0.0, deterministic=False, num_heads_q=None, sm_margin=0,
                return_attn_probs=False):
        reject_unsupported(q_descale=q_descale, k_descale=k_descale, v_descale=v_descale,
                           attention_chunk=attention_chunk, softcap=softcap, deterministic=deterministic)
        q, k, v = split_qkv(qkv, num_heads_q)
        ctx.qkv_rank = qkv.dim()
        return _run_forward(ctx, q, k, v, None, None, None, None, softmax_scale, causal, window_size, return_attn_probs)

    @staticmethod
    def backward(ctx, dout, *unused):
        arguments = _backward_arguments(ctx, dout)
        q, k = arguments[1], arguments[2]
        if ctx.qkv_rank == 5:
            dqkv = q.new_empty(_stacked(q, 3))
        else:
            dqkv = q.new_empty((*q.shape[:-2], q.shape[-2] + 2 * k.shape[-2], q.shape[-1]))
        flash_attn_backward_packed(*arguments, None, dqkv)
        return _pad(ctx, dqkv)


class FlashAttnKVPackedFunc(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, kv, dropout_p, softmax_scale, causal, window_size=(-1, -1), softcap=0.0, alibi_slopes=None,
                deterministic=False, return_attn_probs=False):
        reject_unsupported(dropout_p=dropout_p, alibi_slopes=alibi_slopes, softcap=softcap, deterministic=deterministic)
        k, v = kv.unbind(dim=-3)
        return _run_forward(ctx, q, k, v, None, None, None, None, softmax_scale, causal, window_size, return_attn_probs)

    @staticmethod
    def backward(ctx, dout, *unused):
        return _kvpacked_backward(ctx, dout)


class FlashAttnVarlenKVPackedFunc(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, kv, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, dropout_p, softmax_scale, causal,
                window_size=(-1, -1), softcap=0.0, alibi_slopes=None, deterministic=False, return_attn_probs=False):
        reject_unsupported(dropout_p=dropout_p, alibi_slopes=alibi_slopes, softcap=softcap, deterministic=deterministic)
        k, v = kv.unbind(dim=-3)
        return _run_forward(ctx, q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, softmax_scale, causal,
                            window_size, return_attn_probs)

    @staticmethod
    def backward(ctx, dout, *unused):
        return _kvpacked_backward(ctx, dout)


def _inter_sequence_window(causal, window_size, window_sizes):
    left, right = window_size
    if window_sizes is not None and (causal or (left, right) != (-1, -1)):
        raise ValueError("window_sizes cannot be combined with causal=True or a window_size")
    return left, 0 if causal else right


def _run_inter_sequence_forward(ctx, q, k, v, cu_seqlens_q, cu_seqlens_k, visibility_bits, softmax_scale, causal,
                                window_size, window_sizes, metadata, deterministic, return_softmax):
    reject_unsupported(deterministic=deterministic)
    softmax_scale = default_softmax_scale(softmax_scale, q.shape[-1])
    window = _inter_sequence_window(causal, window_size, window_sizes)
    require_window(*window_size)
    if metadata is None:
        metadata = prepare_inter_sequence_metadata(cu_seqlens_q, cu_seqlens_k, visibility_bits)
    layout = (cu_seqlens_q, cu_seqlens_k, visibility_bits, *metadata._tensors, window_sizes)
    out, softmax_lse = inter_sequence_forward(q, k, v, *layout, softmax_scale, *window)
    ctx.save_for_backward(q, k, v, out, softmax_lse, *layout)
    ctx.softmax_scale = softmax_scale
    ctx.window = window
    if not return_softmax:
        return out
    ctx.mark_non_differentiable(softmax_lse)
    return out, softmax_lse


class FlashAttnInterSequenceFunc(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, visibility_bits, softmax_scale,
                causal, window_size=(-1, -1), window_sizes=None, metadata=None, deterministic=False,
                return_attn_probs=False):
        return _run_inter_sequence_forward(ctx, q, k, v, cu_seqlens_q, cu_seqlens_k, visibility_bits, softmax_scale,
                                           causal, window_size, window_sizes, metadata, deterministic, return_attn_probs)

    @staticmethod
    def backward(ctx, dout, *unused):
        gradients = inter_sequence_backward(dout, *ctx.saved_tensors, ctx.softmax_scale, *ctx.window)
        return _pad(ctx, *gradients)


class FlashAttnInterSequenceKVPackedFunc(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, kv, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, visibility_bits, softmax_scale,
                causal, window_size=(-1, -1), window_sizes=None, metadata=None, deterministic=False,
                return_attn_probs=False):
        k, v = kv.unbind(dim=-3)
        return _run_inter_sequence_forward(ctx, q, k, v, cu_seqlens_q, cu_seqlens_k, visibility_bits, softmax_scale,
                                           causal, window_size, window_sizes, metadata, deterministic, return_attn_probs)

    @staticmethod
    def backward(ctx, dout, *unused):
        arguments = (dout, *ctx.saved_tensors, ctx.softmax_scale, *ctx.window)
        q, k = arguments[1], arguments[2]
        dq, dkv = q.new_empty(q.shape), k.new_empty(_stacked(k, 2))
        inter_sequence_backward_packed(*arguments, dq, dkv)
        return _pad(ctx, dq, dkv)
