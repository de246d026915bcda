"""Regenerates the performance table of the library on the current GPU.

    python zig-flash-attn_b200/perf_report.py --out profiles/perf_report.md [--no-cudnn] [--seconds 0.15]

The grid is the one the reference's report is built on (reference reports/update_perf_report.py,
benchmarks/benchmark_attn.py:399-400 and reports/perf_report.html:417): 16 384 tokens in total, model dimension 2048
(so head_dim 64 / 128 / 256 means 32 / 16 / 8 query heads), "mha" (as many key heads) and "gqa" (a quarter as many),
dense and causal masks, sequence lengths 512 ... 8192 with batch = 16384 / seqlen; plus one sliding-window case (one
16 384-token sequence, window 4096) and one packed case (sequences of 4096 ... 12 288 tokens) at head_dim 128. Every cell
is forward / backward TFLOP/s (4 * heads * head_dim * visible pairs forward, 2.5 x that backward), device-timed with
CUDA events, median of three timings; the cuDNN column is PyTorch's scaled_dot_product_attention under
SDPBackend.CUDNN_ATTENTION on the same tensors, a comparison point only.
"""
import argparse
import itertools
import json
import math
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

TOKENS, MODEL_DIM = 16384, 2048
SEQLENS = (512, 1024, 2048, 4096, 8192)


def timed(function, seconds):
    import torch

    def once(count):
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        for _ in range(count):
            function()
        stop.record()
        torch.cuda.synchronize()
        return start.elapsed_time(stop) / count

    function()
    count = int(min(200, max(3, math.ceil(seconds * 1e3 / max(once(1), 1e-3)))))
    return sorted(once(count) for _ in range(3))[1]


def visible_pairs(seqlen, window):
    left, right = window
    total = 0
    for row in range(seqlen):
        hi = seqlen if right < 0 else min(seqlen, row + right + 1)
        lo = 0 if left < 0 else max(0, row - left)
        total += max(hi - lo, 0)
    return total


def fixed_case(batch, seqlen, heads_q, heads_kv, d, window, seconds, with_cudnn):
    import torch
    from torch.nn import functional
    from torch.nn.attention import SDPBackend, sdpa_kernel

    from zigfa._impl import ops

    make = lambda heads: torch.randn(batch, seqlen, heads, d, device="cuda", dtype=torch.bfloat16)
    q, k, v, dout = make(heads_q), make(heads_kv), make(heads_kv), make(heads_q)
    out, lse = torch.empty_like(q), torch.empty(batch, heads_q, seqlen, dtype=torch.float32, device="cuda")
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    scale = d**-0.5
    forward = lambda: ops.launch_forward(q, k, v, out, lse, None, None, scale, *window)
    backward = lambda: ops.launch_backward(dout, q, k, v, out, lse, dq, dk, dv, None, None, scale, *window)
    flops = 4.0 * heads_q * d * batch * visible_pairs(seqlen, window)
    forward()
    cell = {"fwd": flops / timed(forward, seconds) / 1e9, "bwd": 2.5 * flops / timed(backward, seconds) / 1e9}
    if with_cudnn and window in ((-1, -1), (-1, 0)):
        try:
            qt, kt, vt = (x.transpose(1, 2).detach().requires_grad_() for x in (q, k, v))
            options = {"enable_gqa": True} if heads_q != heads_kv else {}

            def reference_forward():
                with sdpa_kernel(SDPBackend.CUDNN_ATTENTION):
                    return functional.scaled_dot_product_attention(qt, kt, vt, is_causal=window[1] == 0, **options)

            result = reference_forward()
            grad = dout.transpose(1, 2)
            reference_backward = lambda: torch.autograd.grad(result, (qt, kt, vt), grad, retain_graph=True)
            reference_backward()
            cell["cudnn_fwd"] = flops / timed(reference_forward, seconds) / 1e9
            cell["cudnn_bwd"] = 2.5 * flops / timed(reference_backward, seconds) / 1e9
        except Exception as error:
            cell["cudnn_error"] = f"{type(error).__name__}: {error}"[:120]
    return cell


def packed_case(lengths, heads_q, heads_kv, d, window, seconds):
    import torch

    import zigfa

    total = sum(lengths)
    q = torch.randn(total, heads_q, d, device="cuda", dtype=torch.bfloat16).requires_grad_()
    k, v = (torch.randn(total, heads_kv, d, device="cuda", dtype=torch.bfloat16).requires_grad_() for _ in range(2))
    dout = torch.randn_like(q)
    cu = torch.tensor([0, *itertools.accumulate(lengths)], dtype=torch.int32, device="cuda")
    forward = lambda: zigfa.flash_attn_varlen_func(q, k, v, cu, cu, max(lengths), max(lengths), window_size=window)
    out = forward()
    backward = lambda: torch.autograd.grad(out, (q, k, v), dout, retain_graph=True)
    flops = 4.0 * heads_q * d * sum(visible_pairs(n, window) for n in lengths)
    return {"fwd": flops / timed(forward, seconds) / 1e9, "bwd": 2.5 * flops / timed(backward, seconds) / 1e9}


def main():
    parser = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    parser.add_argument("--out", default="perf_report.md")
    parser.add_argument("--seconds", type=float, default=0.15, help="length of one timing")
    parser.add_argument("--no-cudnn", action="store_true")
    options = parser.parse_args()
    import torch

    torch.manual_seed(0)
    rows, data = [], {}
    for d in (64, 128, 256):
        heads = MODEL_DIM // d
        for layout, heads_kv in (("mha", heads), ("gqa", heads // 4)):
            for mask, window in (("dense", (-1, -1)), ("causal", (-1, 0))):
                cells = [fixed_case(TOKENS // s, s, heads, heads_kv, d, window, options.seconds, not options.no_cudnn)
                         for s in SEQLENS]
                data[f"{layout}/{mask}/{d}"] = cells
                for direction in ("fwd", "bwd"):
                    ours = " | ".join(f"{cell[direction]:.0f}" for cell in cells)
                    rows.append(f"| {layout} {mask} hd{d} {direction} | {ours} |")
                    if "cudnn_fwd" in cells[-1]:
                        theirs = " | ".join(f"{cell.get('cudnn_' + direction, float('nan')):.0f}" for cell in cells)
                        rows.append(f"| &nbsp;&nbsp;cuDNN (torch SDPA), same tensors | {theirs} |")
    heads = MODEL_DIM // 128
    sliding = fixed_case(1, TOKENS, heads, heads // 4, 128, (4096, 0), options.seconds, False)
    varlen = packed_case([4096, 12288], heads, heads // 4, 128, (-1, 0), options.seconds)
    data["sliding/4096/128"], data["varlen/causal/128"] = sliding, varlen
    name = torch.cuda.get_device_name(0)
    text = [f"# Performance table of the library ({name}, torch {torch.__version__}, {time.strftime('%Y-%m-%d')})", "",
            "Command: `python zig-flash-attn_b200/perf_report.py --out profiles/perf_report.md` (plain run, CUDA events, no profiler).",
            "TFLOP/s; 16 384 tokens, model dimension 2048; columns are sequence lengths (batch = 16384 / seqlen).", "",
            "| case | " + " | ".join(map(str, SEQLENS)) + " |", "|---|" + "---|" * len(SEQLENS), *rows, "",
            f"Sliding window (one 16 384-token sequence, gqa hd128, window 4096, causal): forward {sliding['fwd']:.0f}, backward {sliding['bwd']:.0f}.",
            f"Packed (sequences of 4096 and 12 288 tokens, gqa hd128, causal): forward {varlen['fwd']:.0f}, backward {varlen['bwd']:.0f}.", ""]
    Path(options.out).write_text("\n".join(text))
    Path(options.out).with_suffix(".json").write_text(json.dumps(data))
    print("\n".join(text))


if __name__ == "__main__":
    main()
