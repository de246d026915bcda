"""GPU tests of inter-sequence attention (visibility bits) and of the integer kernels: metadata and work lists are
bit-exact against their definitions; outputs and gradients match the oracle on dense masks. The layout families
follow the ones the reference tests (reference tests/test_inter_sequence.py:96-151,197-301)."""
import itertools

import numpy as np
import pytest
import torch

import attention_oracle as oracle
import parity
import zigfa
from zigfa._impl import lib, ops

pytestmark = pytest.mark.gpu

DENSE, CAUSAL = (-1, -1), (-1, 0)
WINDOWS = [(-1, -1), (-1, 0), (-1, 7), (5, -1), (9, 3), (0, 0)]
HEAD_LAYOUTS = {"mha": (6, 6), "mqa": (6, 1), "gqa": (6, 3)}


class Layout:
    def __init__(self, lengths_q, lengths_k, visible, windows):
        self.lengths_q, self.lengths_k = list(lengths_q), list(lengths_k)
        self.visible = torch.as_tensor(np.asarray(visible), dtype=torch.bool)
        self.windows = [tuple(w) for w in windows]

    @property
    def count(self):
        return len(self.lengths_q)

    def tensors(self):
        cu_q = torch.tensor([0, *itertools.accumulate(self.lengths_q)], dtype=torch.int32, device="cuda")
        cu_k = torch.tensor([0, *itertools.accumulate(self.lengths_k)], dtype=torch.int32, device="cuda")
        bits = torch.from_numpy(oracle.visibility_bits_of(self.visible.numpy())).cuda()
        window_sizes = torch.tensor(self.windows, dtype=torch.int32).t().contiguous().cuda()
        return cu_q, cu_k, bits, window_sizes


def samples_layout(samples, windows_of_parts, parts_seen=None):
    """Each sample is a list of parts; part p of a sample sees parts `parts_seen[p]` (default: all earlier parts and
    itself) of the same sample."""
    lengths_q, lengths_k, windows, seen = [], [], [], []
    for sample in samples:
        first = len(lengths_q)
        for part, length in enumerate(sample):
            length_q, length_k = length if isinstance(length, tuple) else (length, length)
            lengths_q.append(length_q)
            lengths_k.append(length_k)
            windows.append(windows_of_parts[part])
            seen.append([first + p for p in (range(part + 1) if parts_seen is None else parts_seen[part])])
    visible = torch.zeros(len(lengths_q), len(lengths_q), dtype=torch.bool)
    for query, keys in enumerate(seen):
        visible[query, keys] = True
    return Layout(lengths_q, lengths_k, visible, windows)


def random_layout(count, generator, gaps=False, separate_keys=False):
    lengths_q = torch.randint(1, 160, (count,), generator=generator).tolist()
    lengths_k = list(lengths_q)
    if separate_keys:
        lengths_k = [length + int(torch.randint(0, 40, (), generator=generator)) for length in lengths_q]
        for index in range(0, count, max(1, count // 3)):
            lengths_q[index] = 0
    visible = torch.rand(count, count, generator=generator) < 0.4
    if gaps:
        visible = torch.zeros(count, count, dtype=torch.bool)
        visible[:, ::2] = True
        visible.fill_diagonal_(True)
    windows = [WINDOWS[int(i)] for i in torch.randint(0, len(WINDOWS), (count,), generator=generator)]
    return Layout(lengths_q, lengths_k, visible, windows)


def build_layout(name, seed):
    generator = torch.Generator().manual_seed(seed)
    if name == "image_then_text":
        samples = [tuple(int(x) for x in row) for row in torch.randint(16, 300, (5, 2), generator=generator)]
        return samples_layout(samples, [DENSE, CAUSAL])
    if name == "text_then_images":
        samples = [tuple(int(x) for x in torch.randint(8, 260, (3,), generator=generator)) for _ in range(3)]
        return samples_layout(samples, [CAUSAL, DENSE, DENSE])
    if name == "interleaved":
        samples = [tuple(row) for row in torch.randint(8, 260, (3, 4), generator=generator).tolist()]
        return samples_layout(samples, [CAUSAL, DENSE, CAUSAL, DENSE], ((0,), (0, 1), (0, 1, 2), (0, 1, 2, 3)))
    if name == "extend":  # cached keys with few new query tokens (query length != key length)
        images, texts = torch.randint(16, 300, (2, 5), generator=generator).tolist()
        new = [1, 0, *torch.randint(2, 200, (3,), generator=generator).tolist()]
        samples = [((0, image), (n, text + n)) for image, text, n in zip(images, texts, new)]
        return samples_layout(samples, [DENSE, CAUSAL])
    if name == "shared_prefix":  # one prefix, continuations that see the prefix and themselves
        samples = [(200, 64, 64, 64), (130, 50, 70)]
        return samples_layout(samples, [CAUSAL] * 4, ((0,), (0, 1), (0, 2), (0, 3)))
    return random_layout(11 if name != "gapped" else 9, generator, gaps=name == "gapped",
                         separate_keys=name == "separate_keys")


LAYOUTS = ["image_then_text", "text_then_images", "interleaved", "extend", "shared_prefix", "random", "gapped", "separate_keys"]


def leaves(layout, heads_q, heads_kv, head_dim):
    rows_q, rows_k = sum(layout.lengths_q), sum(layout.lengths_k)
    make = lambda rows, heads: torch.randn(rows, heads, head_dim, device="cuda", dtype=torch.bfloat16).requires_grad_()
    return make(rows_q, heads_q), make(rows_k, heads_kv), make(rows_k, heads_kv)


def check_layout(layout, heads_q, heads_kv, head_dim, backward=True, **options):
    q, k, v = leaves(layout, heads_q, heads_kv, head_dim)
    cu_q, cu_k, bits, window_sizes = layout.tensors()
    windows = layout.windows
    if "causal" in options or "window_size" in options:
        left, right = options.get("window_size", (-1, -1))
        windows = [(left, 0 if options.get("causal") else right)] * layout.count
    else:
        options["window_sizes"] = window_sizes
    out, lse = zigfa.flash_attn_inter_sequence_func(
        q, k, v, cu_q, cu_k, max(layout.lengths_q), max(layout.lengths_k), bits, return_attn_probs=True, **options
    )
    mask = oracle.inter_sequence_mask(cu_q.tolist(), cu_k.tolist(), layout.visible, windows)
    dout = torch.randn_like(out)
    grads = torch.autograd.grad(out, (q, k, v), dout) if backward and q.numel() else None
    parity.check_masked((out.detach(), lse, grads), q.detach(), k.detach(), v.detach(), dout, mask)
    return out.detach(), lse, grads, mask


@pytest.mark.parametrize("head_dim", [64, 128, 256])
@pytest.mark.parametrize("name", LAYOUTS)
def test_layouts_match_oracle(head_dim, name):
    for heads_name, seed in itertools.product(HEAD_LAYOUTS, range(2)):
        torch.manual_seed(seed)
        check_layout(build_layout(name, seed), *HEAD_LAYOUTS[heads_name], head_dim)


@pytest.mark.parametrize("name", LAYOUTS)
def test_layouts_forward_head_dim_512(name):
    # head_dim 512 has a forward kernel only
    for heads_name in HEAD_LAYOUTS:
        torch.manual_seed(1)
        check_layout(build_layout(name, 1), *HEAD_LAYOUTS[heads_name], 512, backward=False)


@pytest.mark.parametrize("options", [dict(causal=True), dict(window_size=(6, 2)), dict(window_size=(-1, -1))])
def test_scalar_windows(options):
    torch.manual_seed(3)
    check_layout(build_layout("random", 3), 6, 2, 128, **dict(options))


def test_rows_that_see_no_keys_return_zeros():
    layout = build_layout("image_then_text", 4)
    layout.visible[2] = False
    layout.visible[5, 5] = False
    layout.windows[3] = (0, -1)
    torch.manual_seed(4)
    out, lse, grads, mask = check_layout(layout, 4, 4, 128)
    blind = ~mask.any(dim=-1).cuda()
    assert blind.any()
    assert (out[blind] == 0).all() and (lse[:, blind] == float("-inf")).all()
    assert (grads[0][blind] == 0).all()


@pytest.mark.parametrize("lengths_q, lengths_k", [([0, 0], [300, 256]), ([10, 30], [0, 0])])
def test_batches_without_queries_or_keys(lengths_q, lengths_k):
    layout = Layout(lengths_q, lengths_k, [[True, False], [True, True]], [CAUSAL, DENSE])
    cu_q, cu_k, bits, window_sizes = layout.tensors()
    torch.manual_seed(12)
    q, k, v = leaves(layout, 4, 2, 128)
    out, lse = zigfa.flash_attn_inter_sequence_func(
        q, k, v, cu_q, cu_k, max(lengths_q), max(lengths_k), bits, window_sizes=window_sizes, return_attn_probs=True
    )
    assert (out == 0).all() and (lse == float("-inf")).all()
    gradients = torch.autograd.grad(out, (q, k, v), torch.randn_like(out), allow_unused=True)
    for gradient in gradients:
        assert gradient is None or (gradient == 0).all()


def test_many_sequences_span_several_words():
    generator = torch.Generator().manual_seed(5)
    layout = random_layout(70, generator)
    lengths = [length // 4 + 1 for length in layout.lengths_q]
    torch.manual_seed(5)
    check_layout(Layout(lengths, lengths, layout.visible, layout.windows), 4, 2, 128)


def test_long_shared_prefix_groups():
    # the shape family of the shared-prefix benchmark configuration, shrunk: prefix + continuations per group
    samples = [(1024, 256, 256, 256)] * 2
    layout = samples_layout(samples, [CAUSAL] * 4, ((0,), (0, 1), (0, 2), (0, 3)))
    torch.manual_seed(6)
    check_layout(layout, 8, 2, 128, causal=True)


def test_kvpacked_matches_unpacked_and_metadata_is_reusable():
    layout = build_layout("gapped", 6)
    torch.manual_seed(6)
    q, k, v = leaves(layout, 6, 2, 128)
    cu_q, cu_k, bits, window_sizes = layout.tensors()
    arguments = (cu_q, cu_k, max(layout.lengths_q), max(layout.lengths_k), bits)
    out = zigfa.flash_attn_inter_sequence_func(q, k, v, *arguments, window_sizes=window_sizes)
    kv = torch.stack([k.detach(), v.detach()], dim=1).requires_grad_()
    packed = zigfa.flash_attn_inter_sequence_kvpacked_func(q, kv, *arguments, window_sizes=window_sizes)
    dout = torch.randn_like(out)
    dq, dk, dv = torch.autograd.grad(out, (q, k, v), dout)
    packed_dq, dkv = torch.autograd.grad(packed, (q, kv), dout)
    assert torch.equal(packed, out)
    assert (packed_dq.float() - dq.float()).abs().max() < 1e-2
    assert torch.equal(dkv, torch.stack([dk, dv], dim=1))
    metadata = zigfa.prepare_inter_sequence_metadata(cu_q, cu_k, bits)
    reused = zigfa.flash_attn_inter_sequence_func(q, k, v, *arguments, window_sizes=window_sizes, metadata=metadata)
    assert torch.equal(reused, out)


def test_invalid_arguments_raise():
    layout = build_layout("image_then_text", 8)
    q, k, v = (t.detach() for t in leaves(layout, 4, 2, 128))
    cu_q, cu_k, bits, window_sizes = layout.tensors()
    arguments = (q, k, v, cu_q, cu_k, 1, 1)
    with pytest.raises(ValueError, match="window_sizes"):
        zigfa.flash_attn_inter_sequence_func(*arguments, bits, causal=True, window_sizes=window_sizes)
    with pytest.raises(NotImplementedError, match="deterministic"):
        zigfa.flash_attn_inter_sequence_func(*arguments, bits, deterministic=True)
    with pytest.raises(ValueError, match="visibility_bits"):
        zigfa.flash_attn_inter_sequence_func(*arguments, bits[:-1])
    with pytest.raises(ValueError, match="window_sizes"):
        zigfa.flash_attn_inter_sequence_func(*arguments, bits, window_sizes=window_sizes[:, :-1])


# ------------------------------------------------------------------------------------------------ integer kernels
@pytest.mark.parametrize("count", [1, 31, 32, 33, 100, 1100])
def test_metadata_kernels_match_their_definition(count):
    generator = torch.Generator().manual_seed(count)
    layout = random_layout(count, generator, separate_keys=True)
    cu_q, cu_k, bits, _ = layout.tensors()
    bits_t, cu_visible_k, cu_visible_q = ops.inter_sequence_metadata(cu_q, cu_k, bits)
    expected = oracle.metadata_definition(layout.lengths_q, layout.lengths_k, layout.visible.numpy())
    assert np.array_equal(bits_t.cpu().numpy(), expected[0])
    assert np.array_equal(cu_visible_k.cpu().numpy(), expected[1])
    assert np.array_equal(cu_visible_q.cpu().numpy(), expected[2])


@pytest.mark.parametrize("batch", [1, 4, 31, 33, 1023, 1025, 3000])
@pytest.mark.parametrize("kind", ["heavy_tail", "zero", "tile_multiples"])
@pytest.mark.parametrize("block,descending", [(256, 1), (128, 0)])
def test_work_list_kernel_matches_its_definition(batch, kind, block, descending):
    rng = np.random.default_rng(batch * 7 + len(kind))
    if kind == "zero":
        lengths = rng.integers(0, 3, batch) * rng.integers(1, 300, batch)
        lengths[: batch // 2] = 0
    elif kind == "tile_multiples":
        lengths = rng.integers(0, 4, batch) * block
    else:
        lengths = (rng.random(batch) ** 6 * 4000).astype(np.int64) + 1
    other = rng.integers(0, 5000, batch)
    cu = torch.from_numpy((np.concatenate([[0], np.cumsum(lengths)]) + 17).astype(np.int32)).cuda()
    cu_other = torch.from_numpy((np.concatenate([[0], np.cumsum(other)]) + 17).astype(np.int32)).cuda()
    entries = oracle.work_list_entries(int(lengths.sum()), batch, block)
    table = torch.full((max(entries, 1), 2), -1, dtype=torch.int32, device="cuda")
    status = lib.library().b200fa_work_list(
        cu.data_ptr(), cu_other.data_ptr(), batch, block, descending, entries, table.data_ptr(),
        torch.cuda.current_stream().cuda_stream,
    )
    assert status == 0, lib.last_error()
    listed = table[:entries].cpu().numpy()
    assert sorted(map(tuple, listed.tolist())) == oracle.every_block(lengths.tolist(), block, entries)
    assert np.array_equal(listed, oracle.work_list_definition(lengths, other, block, bool(descending), entries))
