"""Benchmark of the attention hot path on N GPUs of one node.

    python bench.py --gpus N --steps K --warmup W [--workload c1|c1s|d256s|c2|c3|c4] [--impl reference]

One step = one forward + one backward pass of the workload on every rank. Default workload "c1" is the configuration
the headline metric is quoted on: fixed-length causal GQA, batch 4, seqlen 8192, 32 query / 8 key heads, head_dim
128, BF16 N(0,1) inputs from a seed. With N > 1 every rank runs its own copy of that batch (independent shards, no
collective on the data path; scaling "weak").

The timed region is `--rounds` rounds (default 7) of exactly K steps each, more than a second in total, so that the
figures are taken at the clocks the GPU settles to under its power cap and not at those of a cold start; `value` and
`ms_per_step` are those of the median round, every round is listed in `rounds_ms_per_step`, and `cycles` gives
time x median SM MHz so that two builds can be compared across clock states.

Besides the headline the JSON line carries
  workloads   (N = 1) forward / backward time, TFLOP/s and fraction of the measured BF16 peak of the other
              configurations: c2 packed + window, c3 inter-sequence at head_dim 256 and 512 (forward), one shard of c4, head_dim 64 and 256 fixed length, and the shape the reference's own report is quoted on;
  c4          the long-context configuration (batch 16, seqlen 32768, 32/4 heads, window (4096, 0)) split evenly by
              batch over the N ranks (the whole of it at N = 1): strong scaling, whole-job TFLOP/s and tokens/s from the max-over-ranks time;
  anchors     (N = 1) PyTorch's cuDNN attention on the same GPU and shapes, for comparison only;
  e2e         the headline workload through the public API with pinned host buffers, copies inside the timed region;
  roofline    the backward main kernel timed by itself (the library's timing hook) against the measured BF16 peak;
  cpu_baseline the CPU restatement of the reference's oracle on the host cores (a bounded sample of c1, and config 0).

`--workload c4` makes the long-context configuration the headline (strong scaling); "c2" and "c3" run the packed
workloads alone on one GPU; "c1s" and "d256s" are the small profiling cases.

`--impl reference` times the CPU restatement of the reference's oracle (oracle/attention_oracle.py; the reference's
own kernels are Zig -> PTX and cannot be built here) on a bounded sample of the same workload, K steps after W warm-ups.
"""
import argparse
import ctypes
import itertools
import json
import math
import os
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT / "zig-flash-attn_b200"))

WORKLOADS = {
    "c1": dict(batch=4, seqlen=8192, heads_q=32, heads_kv=8, head_dim=128, window=(-1, 0), seed=1,
               name="fixed-length causal GQA fwd+bwd: batch 4, seqlen 8192, heads 32/8, head_dim 128"),
    "c1s": dict(batch=1, seqlen=8192, heads_q=32, heads_kv=8, head_dim=128, window=(-1, 0), seed=1,
                name="one batch entry of c1 (profiling case): batch 1, seqlen 8192, heads 32/8, head_dim 128, causal"),
    "d256s": dict(batch=1, seqlen=8192, heads_q=16, heads_kv=4, head_dim=256, window=(-1, 0), seed=3,
                  name="head_dim 256 profiling case: batch 1, seqlen 8192, heads 16/4, head_dim 256, causal"),
    "c2": dict(kind="varlen", total=65536, min_len=256, max_len=8192, heads_q=64, heads_kv=8, head_dim=128,
               window=(4096, 0), seed=2,
               name="packed (varlen) fwd+bwd: 65536 tokens in sequences of 256..8192, heads 64/8, head_dim 128, window (4096, 0)"),
    "c3": dict(kind="interseq", groups=8, prefix=2048, continuations=7, continuation_len=512, heads_q=32, heads_kv=8,
               head_dim=256, seed=3,
               name="inter-sequence fwd+bwd: 8 groups of a 2048-token prefix and 7 continuations of 512 that see it, "
                    "heads 32/8, head_dim 256, causal"),
    "c4": dict(batch=16, seqlen=32768, heads_q=32, heads_kv=4, head_dim=128, window=(4096, 0), seed=4,
               name="long-context sharded fwd+bwd: batch 16, seqlen 32768, heads 32/4, head_dim 128, window (4096, 0)"),
}
# Fixed-length shapes of the `workloads` record (N = 1): name -> (batch, seqlen, heads_q, heads_kv, head_dim, window).
EXTRA_FIXED = {
    "reference_report_shape_b2_s8192_h16_4_d128_causal": (2, 8192, 16, 4, 128, (-1, 0)),
    "d64_b4_s8192_h32_8_causal": (4, 8192, 32, 8, 64, (-1, 0)),
    "d256_b4_s8192_h16_4_causal": (4, 8192, 16, 4, 256, (-1, 0)),
    "c1_dense_b4_s8192_h32_8_d128": (4, 8192, 32, 8, 128, (-1, -1)),
    "c4_one_shard_of_8_b2_s32768_h32_4_d128_window4096": (2, 32768, 32, 4, 128, (4096, 0)),
}


def visible_pairs(seqlen, window):
    """Visible (query, key) pairs of one sequence under a bottom-right aligned band (-1 = unbounded)."""
    import numpy as np

    left, right = window
    rows = np.arange(seqlen, dtype=np.int64)
    hi = np.full(seqlen, seqlen, dtype=np.int64) if right < 0 else np.minimum(seqlen, rows + right + 1)
    lo = np.zeros(seqlen, dtype=np.int64) if left < 0 else np.maximum(0, rows - left)
    return int(np.maximum(hi - lo, 0).sum())


def measured_peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        data = json.loads(path.read_text())
        return dict(source="measured", burst=data["bf16_tflops"], sustained=data["bf16_tflops_sustained"],
                    hbm=data["hbm_gbs"])
    return dict(source="fallback", burst=1590.0, sustained=1400.0, hbm=6650.0)


def config_of(workload, world, strong):
    """The `config` object of the JSON line; both arms print the same one for the same command line."""
    batch = workload["batch"] // world if strong else workload["batch"]
    return {"workload": workload["name"], "per_gpu_batch": batch, "global_batch": batch * world,
            "seq_len": workload["seqlen"], "parallelism": f"batch shards x{world}, no collective on the data path",
            "l2": "inputs (675 MB+) exceed the 126 MB L2", "flop_convention": "4*Hq*D*visible_pairs fwd, 2.5x bwd"}


class ClockSampler:
    """Samples SM clocks, power and throttle reasons through NVML (read-only) while the timed region runs."""

    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}

    def __init__(self, index):
        self.index, self.samples, self.running, self.thread, self.error = index, [], False, None, None
        self.max_mhz = None

    def start(self):
        try:
            import pynvml

            pynvml.nvmlInit()
            self.nvml = pynvml
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(self.index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM)
        except Exception as error:  # NVML missing: report that instead of clocks
            self.error = f"nvml unavailable: {error}"
            return
        self.running = True
        self.thread = threading.Thread(target=self._poll, daemon=True)
        self.thread.start()

    def _poll(self):
        while self.running:
            try:
                clock = self.nvml.nvmlDeviceGetClockInfo(self.handle, self.nvml.NVML_CLOCK_SM)
                reasons = self.nvml.nvmlDeviceGetCurrentClocksThrottleReasons(self.handle)
                power = self.nvml.nvmlDeviceGetPowerUsage(self.handle) / 1000.0
                self.samples.append((time.perf_counter(), clock, reasons, power))
            except Exception as error:
                self.error = str(error)
                return
            time.sleep(0.02)

    def median_since(self, start_time):
        """Median SM MHz of the samples taken since `start_time` (perf_counter), None without samples."""
        clocks = sorted(clock for when, clock, _, _ in self.samples if when >= start_time)
        return clocks[len(clocks) // 2] if clocks else None

    def stop(self):
        self.running = False
        if self.thread is not None:
            self.thread.join(timeout=1)
        if not self.samples:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=[self.error or "no samples"])
        clocks = sorted(clock for _, clock, _, _ in self.samples)
        seen = 0
        for _, _, reasons, _ in self.samples:
            seen |= reasons
        reasons = [name for bit, name in self.REASONS.items() if seen & bit]
        return dict(sm_mhz=clocks[len(clocks) // 2], sm_max_mhz=self.max_mhz, reasons=reasons, samples=len(clocks),
                    sm_mhz_min=clocks[0], power_w_max=max(power for _, _, _, power in self.samples))


# ------------------------------------------------------------------------------------------------ CPU arm
def cpu_sample(workload, steps, warmup):
    """Times the oracle (CPU restatement of the reference's attention oracle) on a bounded sample of the workload:
    one batch entry and one key head with its query heads, at most the first 8192 rows of the sequence. Returns TFLOP/s."""
    sys.path.insert(0, str(ROOT / "oracle"))
    import torch

    import attention_oracle as oracle

    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    group = workload["heads_q"] // workload["heads_kv"]
    seqlen = min(workload["seqlen"], 8192)
    d = workload["head_dim"]
    torch.manual_seed(workload["seed"])
    q = torch.randn(1, seqlen, group, d, dtype=torch.bfloat16)
    k, v = (torch.randn(1, seqlen, 1, d, dtype=torch.bfloat16) for _ in range(2))
    dout = torch.randn(1, seqlen, group, d, dtype=torch.bfloat16)
    flops = 3.5 * 4 * group * d * visible_pairs(seqlen, workload["window"])
    times = []
    for step in range(warmup + steps):
        start = time.perf_counter()
        oracle.gradients(oracle.attention, q, k, v, dout, window_size=workload["window"])
        if step >= warmup:
            times.append(time.perf_counter() - start)
    seconds = sum(times) / len(times)
    sample = f"batch 1, {group} query heads / 1 key head, first {seqlen} rows of the sequence, fp32 math, fwd+bwd"
    return dict(value=flops / seconds / 1e12, unit="TFLOP/s", cores=threads, kind="port", sample=sample,
                seconds_per_step=seconds)


def cpu_config0():
    """The CPU-runnable configuration in full (batch 2, seqlen 512, heads 8/2, head_dim 128, causal, seed 0): median of
    five forward + backward passes of the oracle on all host threads, after one warm-up."""
    sys.path.insert(0, str(ROOT / "oracle"))
    import torch

    import attention_oracle as oracle

    torch.set_num_threads(os.cpu_count() or 1)
    torch.manual_seed(0)
    q = torch.randn(2, 512, 8, 128, dtype=torch.bfloat16)
    k, v = (torch.randn(2, 512, 2, 128, dtype=torch.bfloat16) for _ in range(2))
    dout = torch.randn(2, 512, 8, 128, dtype=torch.bfloat16)
    times = []
    for step in range(6):
        start = time.perf_counter()
        oracle.gradients(oracle.attention, q, k, v, dout, causal=True)
        if step:
            times.append(time.perf_counter() - start)
    seconds = sorted(times)[len(times) // 2]
    flops = 3.5 * 4 * 8 * 128 * 2 * visible_pairs(512, (-1, 0))
    return dict(workload="config 0: batch 2, seqlen 512, heads 8/2, head_dim 128, causal, fp32 math, fwd+bwd",
                ms=seconds * 1e3, gflops=flops / seconds / 1e9, cores=os.cpu_count() or 1)


def reference_arm(options, workload):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    world = int(os.environ.get("WORLD_SIZE", str(options.gpus)))
    steps, warmup = options.steps, options.warmup
    result = cpu_sample(workload, steps, warmup)
    line = {
        "impl": "reference", "metric": "attn_fwd_bwd_tflops", "value": result["value"], "unit": "TFLOP/s",
        "n_gpus": options.gpus, "steps": steps, "warmup": warmup, "ms_per_step": result["seconds_per_step"] * 1e3,
        "higher_is_better": True, "scaling": "strong" if options.workload == "c4" else "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic", "config": config_of(workload, world, options.workload == "c4"),
        "cpu_baseline": {k: result[k] for k in ("value", "unit", "cores", "kind", "sample")},
        "e2e": {"value": result["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "reference's own kernels are Zig->PTX (zig-nvptx fork + cuda-core absent): CPU port of its oracle timed "
                "instead; each step is the bounded sample named in cpu_baseline.sample, ms_per_step is that of the sample",
    }
    print(json.dumps(line))


# ------------------------------------------------------------------------------------------------ timing helpers
def device_time(function, count, barrier=None, reduce_max=None):
    """Milliseconds per call over `count` back-to-back calls, CUDA events on the current stream."""
    import torch

    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    (barrier or torch.cuda.synchronize)()
    start.record()
    for _ in range(count):
        function()
    stop.record()
    (barrier or torch.cuda.synchronize)()
    elapsed = start.elapsed_time(stop) / count
    return reduce_max(elapsed) if reduce_max else elapsed


def budgeted_time(function, seconds=0.25, least=2, most=40, barrier=None, reduce_max=None):
    """Median of three timings of about `seconds` each (the call count comes from one calibrating call)."""
    function()
    one = device_time(function, 1, barrier, reduce_max)
    count = int(min(most, max(least, math.ceil(seconds * 1e3 / max(one, 1e-3)))))
    samples = sorted(device_time(function, count, barrier, reduce_max) for _ in range(3))
    return samples[1]


def rates(flops_fwd, ms_fwd, ms_bwd, peaks, tokens):
    record = {"ms_fwd": ms_fwd, "fwd_tflops": flops_fwd / (ms_fwd * 1e-3) / 1e12,
              "fwd_frac_of_peak": flops_fwd / (ms_fwd * 1e-3) / 1e12 / peaks["burst"]}
    if ms_bwd is not None:
        record.update({"ms_bwd": ms_bwd, "bwd_tflops": 2.5 * flops_fwd / (ms_bwd * 1e-3) / 1e12,
                       "bwd_frac_of_peak": 2.5 * flops_fwd / (ms_bwd * 1e-3) / 1e12 / peaks["burst"],
                       "tokens_per_s": tokens / ((ms_fwd + ms_bwd) * 1e-3)})
    return record


def fixed_problem(batch, seqlen, heads_q, heads_kv, d, window, seed, device):
    """Device-resident BF16 N(0,1) tensors of a fixed-length problem and its forward / backward launchers."""
    import torch

    from zigfa._impl import ops

    generator = torch.Generator(device=device).manual_seed(seed)
    make = lambda heads: torch.randn(batch, seqlen, heads, d, device=device, dtype=torch.bfloat16, generator=generator)
    q, k, v, dout = make(heads_q), make(heads_kv), make(heads_kv), make(heads_q)
    out = torch.empty_like(q)
    lse = torch.empty(batch, heads_q, seqlen, dtype=torch.float32, device=device)
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    scale, (left, right) = d**-0.5, window

    def forward():
        ops.launch_forward(q, k, v, out, lse, None, None, scale, left, right)

    def backward():
        ops.launch_backward(dout, q, k, v, out, lse, dq, dk, dv, None, None, scale, left, right)

    flops_fwd = 4.0 * heads_q * d * batch * visible_pairs(seqlen, window)
    return forward, backward, flops_fwd


def packed_problem(workload, device, head_dim=None):
    """Tensors, forward and backward closures and FLOPs of the packed workloads c2 (varlen) and c3 (inter-sequence)."""
    import torch

    import zigfa

    heads_q, heads_kv = workload["heads_q"], workload["heads_kv"]
    d = head_dim or workload["head_dim"]
    torch.manual_seed(workload["seed"])
    bits = None
    if workload["kind"] == "varlen":
        generator = torch.Generator().manual_seed(workload["seed"])
        lengths = []
        while sum(lengths) < workload["total"]:
            lengths.append(int(torch.randint(workload["min_len"], workload["max_len"] + 1, (1,), generator=generator)))
        lengths[-1] -= sum(lengths) - workload["total"]
        left = workload["window"][0]
        pairs = sum(sum(min(i + 1, left + 1) for i in range(n)) for n in lengths)
    else:
        lengths = ([workload["prefix"]] + [workload["continuation_len"]] * workload["continuations"]) * workload["groups"]
        per_group = 1 + workload["continuations"]
        # visibility bits: bit j of row i (32 per int32 word) = sequence i sees the keys of sequence j
        words = (len(lengths) + 31) // 32
        rows = [[0] * words for _ in lengths]
        for i in range(len(lengths)):
            for j in {i, i - i % per_group}:  # itself and the prefix of its group
                rows[i][j // 32] |= 1 << (j % 32)
        bits = torch.tensor(rows, dtype=torch.int64).to(torch.int32).to(device)
        p, c = workload["prefix"], workload["continuation_len"]
        pairs = workload["groups"] * (p * (p + 1) // 2 + workload["continuations"] * (c * (c + 1) // 2 + c * p))
    total = sum(lengths)
    cu = torch.tensor([0, *itertools.accumulate(lengths)], dtype=torch.int32, device=device)
    q = torch.randn(total, heads_q, d, device=device, dtype=torch.bfloat16).requires_grad_()
    k, v = (torch.randn(total, heads_kv, d, device=device, dtype=torch.bfloat16).requires_grad_() for _ in range(2))
    dout = torch.randn(total, heads_q, d, device=device, dtype=torch.bfloat16)
    longest = max(lengths)

    def forward():
        if workload["kind"] == "varlen":
            return zigfa.flash_attn_varlen_func(q, k, v, cu, cu, longest, longest, window_size=workload["window"])
        return zigfa.flash_attn_inter_sequence_func(q, k, v, cu, cu, longest, longest, bits, causal=True)

    state = {}

    def backward():
        if "out" not in state:
            state["out"] = forward()
        return torch.autograd.grad(state["out"], (q, k, v), dout, retain_graph=True)

    return forward, backward, 4.0 * heads_q * d * pairs, total, len(lengths)


def packed_arm(options, workload):
    """Workloads c2 (varlen) and c3 (inter-sequence) alone on one GPU through the public API, device-timed with the
    inputs resident in HBM."""
    import torch

    from zigfa._impl import lib

    if int(os.environ.get("WORLD_SIZE", "1")) != 1:
        raise SystemExit("the packed workloads run on one GPU; shard them with zig-flash-attn_b200/sharding.py")
    torch.cuda.set_device(0)
    warmup, steps = max(options.warmup, 3), options.steps
    forward, backward, flops_fwd, total, sequences = packed_problem(workload, "cuda")
    for _ in range(warmup):
        forward()
        backward()
    sampler = ClockSampler(0)
    sampler.start()
    ms_fwd, ms_bwd = device_time(forward, steps), device_time(backward, steps)
    clocks = sampler.stop()
    flops_bwd = 2.5 * flops_fwd
    peaks = measured_peaks()
    line = {
        "metric": "attn_fwd_bwd_tflops", "value": (flops_fwd + flops_bwd) / ((ms_fwd + ms_bwd) * 1e-3) / 1e12,
        "unit": "TFLOP/s", "n_gpus": 1, "steps": steps, "warmup": warmup, "ms_per_step": ms_fwd + ms_bwd,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": workload["name"], "sequences": sequences, "tokens": total,
                   "l2": "inputs exceed the 126 MB L2", "flop_convention": "4*Hq*D*visible_pairs fwd, 2.5x bwd"},
        "fwd_tflops_per_gpu": flops_fwd / (ms_fwd * 1e-3) / 1e12, "bwd_tflops_per_gpu": flops_bwd / (ms_bwd * 1e-3) / 1e12,
        "tokens_per_s": total / ((ms_fwd + ms_bwd) * 1e-3), "ms_fwd": ms_fwd, "ms_bwd": ms_bwd,
        "gpu_launches": steps * 6, "e2e": None,
        # the whole backward op (work list, preprocess, main kernel, postprocess): autograd runs it on its own thread, out
        # of reach of the per-thread timing hook that isolates the main kernel in the fixed-length workloads
        "roofline": {"kernel": "backward op (work list + preprocess + dK/dV/dQ main + postprocess)", "bound": "tensor",
                     "achieved": flops_bwd / (ms_bwd * 1e-3) / 1e12, "peak": peaks["burst"], "unit": "TFLOP/s",
                     "frac": flops_bwd / (ms_bwd * 1e-3) / 1e12 / peaks["burst"], "traffic": None,
                     "peak_source": f"{peaks['source']} cuBLAS BF16 burst"},
        "clocks": clocks, "device_status": lib.library().b200fa_device_status(),
    }
    print(json.dumps(line))


def other_workloads(device, peaks):
    """The `workloads` record: the configurations the headline does not cover, about half a second of timing each."""
    import torch

    records = {}
    for name, (batch, seqlen, heads_q, heads_kv, d, window) in EXTRA_FIXED.items():
        forward, backward, flops_fwd = fixed_problem(batch, seqlen, heads_q, heads_kv, d, window, 17, device)
        forward()
        backward()
        records[name] = rates(flops_fwd, budgeted_time(forward), budgeted_time(backward), peaks, batch * seqlen)
        del forward, backward
        torch.cuda.empty_cache()
    # Config 1 with the pivot path of the backward on (zigfa.set_pivot_gradients): what the reference's stricter accuracy
    # guarantees for peaked rows cost; the headline runs with the default, off.
    import zigfa

    batch, seqlen, heads_q, heads_kv, d, window = 4, 8192, 32, 8, 128, (-1, 0)
    forward, backward, flops_fwd = fixed_problem(batch, seqlen, heads_q, heads_kv, d, window, 17, device)
    forward()
    before = zigfa.set_pivot_gradients(True)
    try:
        backward()
        records["c1_backward_with_pivot_gradients"] = rates(flops_fwd, budgeted_time(forward), budgeted_time(backward), peaks,
                                                            batch * seqlen)
    finally:
        zigfa.set_pivot_gradients(before)
    del forward, backward
    torch.cuda.empty_cache()
    for name, key, d, with_backward in (("c2_packed_window", "c2", None, True), ("c3_inter_sequence_d256", "c3", None, True),
                                        ("c3_inter_sequence_d512_forward", "c3", 512, False)):
        forward, backward, flops_fwd, total, sequences = packed_problem(WORKLOADS[key], device, d)
        forward()
        ms_bwd = None
        if with_backward:
            backward()
            ms_bwd = budgeted_time(backward)
        records[name] = dict(rates(flops_fwd, budgeted_time(forward), ms_bwd, peaks, total), tokens=total,
                             sequences=sequences, through="public API (custom ops + autograd)")
        del forward, backward
        torch.cuda.empty_cache()
    return records


def cudnn_anchors(device, peaks):
    """PyTorch's cuDNN attention (scaled_dot_product_attention under SDPBackend.CUDNN_ATTENTION, key heads shared with
    enable_gqa, as the reference's benchmarks/benchmark_attn.py:177-215 measures it) on this GPU: a comparison point
    only, never on the library's path. The reference's published B200 figures stand next to cuDNN's on its machine
    (forward / backward 1261 / 992 against 1271 / 1061 TFLOP/s at batch 2, seqlen 8192, heads 16/4), so library / cuDNN
    on one box carries those figures over to it."""
    import torch
    from torch.nn import functional
    from torch.nn.attention import SDPBackend, sdpa_kernel

    anchors = {}
    for name, (batch, seqlen, heads_q, heads_kv, d) in {"c1_b4_s8192_h32_8_d128_causal": (4, 8192, 32, 8, 128),
                                                       "reference_report_shape_b2_s8192_h16_4_d128_causal": (2, 8192, 16, 4, 128)}.items():
        try:
            generator = torch.Generator(device=device).manual_seed(23)
            make = lambda heads: torch.randn(batch, heads, seqlen, d, device=device, dtype=torch.bfloat16,
                                             generator=generator).requires_grad_()
            q, k, v = make(heads_q), make(heads_kv), make(heads_kv)
            dout = torch.randn(batch, heads_q, seqlen, d, device=device, dtype=torch.bfloat16, generator=generator)

            def forward():
                with sdpa_kernel(SDPBackend.CUDNN_ATTENTION):
                    return functional.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=True)

            out = forward()

            def backward():
                return torch.autograd.grad(out, (q, k, v), dout, retain_graph=True)

            backward()
            flops_fwd = 4.0 * heads_q * d * batch * visible_pairs(seqlen, (-1, 0))
            anchors[name] = dict(rates(flops_fwd, budgeted_time(forward), budgeted_time(backward), peaks, batch * seqlen),
                                 backend="torch SDPA, cuDNN attention", cudnn=torch.backends.cudnn.version())
            del q, k, v, dout, out
        except Exception as error:  # backend not available on this image or device
            anchors[name] = {"unavailable": f"{type(error).__name__}: {error}"[:300]}
        torch.cuda.empty_cache()
    return anchors


# ------------------------------------------------------------------------------------------------ GPU arm
def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=10)
    parser.add_argument("--warmup", type=int, default=3)
    parser.add_argument("--rounds", type=int, default=7, help="timed rounds of --steps steps each; the median is reported")
    parser.add_argument("--workload", choices=sorted(WORKLOADS), default="c1")
    parser.add_argument("--impl", choices=["b200", "reference"], default="b200")
    parser.add_argument("--skip-cpu", action="store_true", help="skip the CPU baseline leg")
    parser.add_argument("--skip-e2e", action="store_true", help="skip the host-buffer end-to-end leg (profiling runs)")
    parser.add_argument("--skip-extras", action="store_true", help="skip the workloads / c4 / anchors records (profiling runs)")
    options = parser.parse_args()
    workload = WORKLOADS[options.workload]
    if workload.get("kind"):
        if options.impl == "reference":
            raise SystemExit("the reference arm times the fixed-length workloads")
        return packed_arm(options, workload)
    if options.impl == "reference":
        return reference_arm(options, workload)

    import torch
    import torch.distributed as dist

    import zigfa
    from zigfa._impl import lib, ops

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    warmup = max(options.warmup, 3)
    steps = options.steps
    rounds = max(options.rounds, 3)
    peaks = measured_peaks()

    strong = options.workload == "c4"
    batch = workload["batch"] // world if strong else workload["batch"]
    seqlen, heads_q, heads_kv, d = workload["seqlen"], workload["heads_q"], workload["heads_kv"], workload["head_dim"]
    window = workload["window"]
    causal = window == (-1, 0)
    generator = torch.Generator(device="cpu").manual_seed(workload["seed"] * 1000 + rank)
    shapes = dict(q=(batch, seqlen, heads_q, d), k=(batch, seqlen, heads_kv, d), v=(batch, seqlen, heads_kv, d),
                  dout=(batch, seqlen, heads_q, d))
    # host buffers are pinned; the resident copies are made once, before the timed region
    host = {}
    for name, shape in shapes.items():
        buffer = torch.empty(shape, dtype=torch.bfloat16).pin_memory()
        for b in range(batch):  # fill per batch entry to bound the float32 temporary
            buffer[b] = torch.randn(shape[1:], generator=generator, dtype=torch.float32).to(torch.bfloat16)
        host[name] = buffer
    resident = {name: tensor.to(device) for name, tensor in host.items()}
    pairs = batch * visible_pairs(seqlen, window)
    flops_fwd = 4.0 * heads_q * d * pairs
    flops_bwd = 2.5 * flops_fwd
    tokens = batch * seqlen
    scale = d**-0.5
    left, right = window

    q, k, v, dout = (resident[name] for name in ("q", "k", "v", "dout"))
    out = torch.empty_like(q)
    lse = torch.empty(batch, heads_q, seqlen, dtype=torch.float32, device=device)
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)

    def forward():
        ops.launch_forward(q, k, v, out, lse, None, None, scale, left, right)

    def backward():
        ops.launch_backward(dout, q, k, v, out, lse, dq, dk, dv, None, None, scale, left, right)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def reduce_max(value):
        if world == 1:
            return value
        tensor = torch.tensor([value], device=device)
        dist.all_reduce(tensor, op=dist.ReduceOp.MAX)
        return tensor.item()

    def step():
        forward()
        backward()

    def median(values):
        return sorted(values)[len(values) // 2]

    for _ in range(warmup):
        step()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    # `rounds` rounds of exactly `steps` steps each, every one bracketed by a barrier and a synchronize, device-timed,
    # max over ranks; the headline is the median round.
    mark = time.perf_counter()
    round_ms = [device_time(step, steps, barrier, reduce_max) for _ in range(rounds)]
    mhz_step = sampler.median_since(mark)
    ms_step = median(round_ms)
    mark = time.perf_counter()
    ms_fwd = median([device_time(forward, steps, barrier, reduce_max) for _ in range(3)])
    mhz_fwd = sampler.median_since(mark)
    mark = time.perf_counter()
    ms_bwd = median([device_time(backward, steps, barrier, reduce_max) for _ in range(3)])
    mhz_bwd = sampler.median_since(mark)

    # dominant kernel by itself: the backward main kernel between the library's timing events
    events = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
    for event in events:
        event.record()
    torch.cuda.synchronize()
    handles = (ctypes.c_void_p * 4)(*[event.cuda_event for event in events])
    main_ms, pre_ms, post_ms = [], [], []
    for _ in range(max(3, min(steps, 10))):
        lib.library().b200fa_bwd_timing_events(handles)
        backward()
        torch.cuda.synchronize()
        pre_ms.append(events[0].elapsed_time(events[1]))
        main_ms.append(events[1].elapsed_time(events[2]))
        post_ms.append(events[2].elapsed_time(events[3]))
    ms_main = sum(main_ms) / len(main_ms)
    clocks = sampler.stop() if rank == 0 else None

    # End to end through the public API with host buffers. Every step copies its q, k, v, dout from pinned host memory
    # and its out, dq, dk, dv back; the three legs run on three streams with two sets of device buffers, so the
    # copies of neighbouring steps overlap the kernels (the way a training input pipeline would feed the op).
    host_out = {name: torch.empty(shapes[key], dtype=torch.bfloat16).pin_memory()
                for name, key in (("out", "q"), ("dq", "q"), ("dk", "k"), ("dv", "v"))}
    h2d_stream, d2h_stream = torch.cuda.Stream(device), torch.cuda.Stream(device)
    staged = [{name: torch.empty_like(tensor) for name, tensor in resident.items()} for _ in range(2)]

    def e2e_steps(count):
        main = torch.cuda.current_stream(device)
        h2d_stream.wait_stream(main)
        d2h_stream.wait_stream(main)
        in_ready = [torch.cuda.Event() for _ in range(count)]
        computed = [torch.cuda.Event() for _ in range(count)]
        copied_out = [torch.cuda.Event() for _ in range(count)]
        keep = [None, None]
        for i in range(count):
            buffers = staged[i & 1]
            with torch.cuda.stream(h2d_stream):
                if i >= 2:
                    h2d_stream.wait_event(computed[i - 2])  # the kernels of step i - 2 have read this buffer set
                for name in ("q", "k", "v", "dout"):
                    buffers[name].copy_(host[name], non_blocking=True)
                in_ready[i].record(h2d_stream)
            main.wait_event(in_ready[i])
            qd, kd, vd = (buffers[name].detach().requires_grad_() for name in ("q", "k", "v"))
            result = zigfa.flash_attn_func(qd, kd, vd, causal=causal, window_size=(left, -1 if causal else right))
            grads = torch.autograd.grad(result, (qd, kd, vd), buffers["dout"])
            computed[i].record(main)
            with torch.cuda.stream(d2h_stream):
                d2h_stream.wait_event(computed[i])
                if i >= 1:
                    d2h_stream.wait_event(copied_out[i - 1])  # one set of pinned result buffers
                for name, tensor in (("out", result.detach()), ("dq", grads[0]), ("dk", grads[1]), ("dv", grads[2])):
                    host_out[name].copy_(tensor, non_blocking=True)
                    tensor.record_stream(d2h_stream)
                copied_out[i].record(d2h_stream)
            keep[i & 1] = (result, grads)
        main.wait_stream(d2h_stream)
        main.wait_stream(h2d_stream)

    if options.skip_e2e:
        ms_e2e = float("nan")
    else:
        e2e_steps(2)
        count = max(4, min(steps, 32))  # as many steps as the device-timed legs: filling and draining the copy pipeline
        # costs one input and one result copy, which eight steps still show as 15 % per step
        ms_e2e = device_time(lambda: e2e_steps(count), 1, barrier, reduce_max) / count
    h2d = sum(t.numel() * 2 for t in host.values())
    d2h = sum(t.numel() * 2 for t in host_out.values())
    torch.cuda.empty_cache()

    # The long-context configuration split by batch over the ranks (strong scaling), every rank generating its own
    # batch entries on the device. With the c4 workload as the headline it is already measured above.
    c4 = None
    if not options.skip_extras and not strong and 16 % world == 0:
        long_context = WORKLOADS["c4"]
        shard = long_context["batch"] // world
        c4_forward, c4_backward, c4_flops_fwd = fixed_problem(shard, long_context["seqlen"], long_context["heads_q"],
                                                              long_context["heads_kv"], long_context["head_dim"],
                                                              long_context["window"], 4000 + rank, device)
        c4_forward()
        c4_backward()
        c4_ms_fwd = budgeted_time(c4_forward, 0.25, 2, 20, barrier, reduce_max)
        c4_ms_bwd = budgeted_time(c4_backward, 0.25, 2, 20, barrier, reduce_max)
        c4_tokens = long_context["batch"] * long_context["seqlen"]
        c4 = {"workload": long_context["name"], "scaling": "strong", "n_gpus": world, "per_gpu_batch": shard,
              "ms_fwd": c4_ms_fwd, "ms_bwd": c4_ms_bwd, "ms_per_step": c4_ms_fwd + c4_ms_bwd,
              "value": 3.5 * c4_flops_fwd * world / ((c4_ms_fwd + c4_ms_bwd) * 1e-3) / 1e12, "unit": "TFLOP/s",
              "fwd_tflops_per_gpu": c4_flops_fwd / (c4_ms_fwd * 1e-3) / 1e12,
              "bwd_tflops_per_gpu": 2.5 * c4_flops_fwd / (c4_ms_bwd * 1e-3) / 1e12,
              "tokens_per_s": c4_tokens / ((c4_ms_fwd + c4_ms_bwd) * 1e-3),
              "timing": "device time, max over ranks, median of 3 timings of >= 0.25 s"}
        del c4_forward, c4_backward
        torch.cuda.empty_cache()
    status = lib.library().b200fa_device_status()

    if rank == 0:
        total_flops = (flops_fwd + flops_bwd) * world
        value = total_flops / (ms_step * 1e-3) / 1e12
        cycles = lambda ms, mhz: None if mhz is None else ms * mhz * 1e-3
        line = {
            "metric": "attn_fwd_bwd_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": steps,
            "warmup": warmup, "ms_per_step": ms_step, "higher_is_better": True,
            "scaling": "strong" if strong else "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": config_of(workload, world, strong),
            "rounds": rounds, "rounds_ms_per_step": round_ms, "timed_region_s": sum(round_ms) * steps * 1e-3,
            "fwd_tflops_per_gpu": flops_fwd / (ms_fwd * 1e-3) / 1e12,
            "bwd_tflops_per_gpu": flops_bwd / (ms_bwd * 1e-3) / 1e12,
            "fwd_frac_of_peak": flops_fwd / (ms_fwd * 1e-3) / 1e12 / peaks["burst"],
            "bwd_frac_of_peak": flops_bwd / (ms_bwd * 1e-3) / 1e12 / peaks["burst"],
            "fwd_frac_of_nominal_2250": flops_fwd / (ms_fwd * 1e-3) / 1e12 / 2250.0,
            "bwd_frac_of_nominal_2250": flops_bwd / (ms_bwd * 1e-3) / 1e12 / 2250.0,
            "tokens_per_s": tokens * world / (ms_step * 1e-3),
            "ms_fwd": ms_fwd, "ms_bwd": ms_bwd,
            # time x median SM clock of the same leg: million SM cycles per step, comparable across clock states
            "cycles": {"unit": "million SM cycles", "step": cycles(ms_step, mhz_step), "fwd": cycles(ms_fwd, mhz_fwd),
                       "bwd": cycles(ms_bwd, mhz_bwd), "sm_mhz": {"step": mhz_step, "fwd": mhz_fwd, "bwd": mhz_bwd}},
            "bwd_kernel_ms": {"preprocess": sum(pre_ms) / len(pre_ms), "main": ms_main, "postprocess": sum(post_ms) / len(post_ms)},
            "gpu_launches": steps * rounds * 4,
            "e2e": {"value": total_flops / (ms_e2e * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": ms_e2e,
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "pipeline": "copies of neighbouring steps overlap the kernels (3 streams, 2 device buffer sets)"},
            "roofline": {"kernel": ("bwd_d256_kernel" if d > 128 else f"bwd_kernel<{64 if d <= 64 else 128}>") + " (dK/dV/dQ main)",
                         "bound": "tensor",
                         "achieved": flops_bwd / (ms_main * 1e-3) / 1e12, "peak": peaks["burst"], "unit": "TFLOP/s",
                         "frac": flops_bwd / (ms_main * 1e-3) / 1e12 / peaks["burst"],
                         # dram__bytes_read.sum + dram__bytes_write.sum of one ncu capture of this kernel on one batch
                         # entry of this workload (workload c1s), scaled by the batch entries per launch: batch entries
                         # are independent CTAs, so the traffic grows in proportion
                         "traffic": BWD_MAIN_DRAM_BYTES_PER_BATCH_ENTRY * batch if options.workload in ("c1", "c1s") else None,
                         "peak_source": f"{peaks['source']} cuBLAS BF16 burst", "sustained_peak": peaks["sustained"]},
            "roofline_fwd": {"kernel": "fwd_d256_kernel" if d > 128 else f"fwd_kernel<{64 if d <= 64 else 128}>", "bound": "tensor", "achieved": flops_fwd / (ms_fwd * 1e-3) / 1e12,
                             "peak": peaks["burst"], "unit": "TFLOP/s",
                             "frac": flops_fwd / (ms_fwd * 1e-3) / 1e12 / peaks["burst"]},
            "clocks": clocks, "device_status": status,
        }
        if c4 is not None:
            line["c4"] = c4
        if not options.skip_extras and world == 1:
            line["workloads"] = other_workloads(device, peaks)
            line["anchors"] = cudnn_anchors(device, peaks)
            line["device_status"] = lib.library().b200fa_device_status() or status
        if not options.skip_cpu and world == 1:  # the CPU baseline belongs to the one-GPU line (the other ranks of a
            # multi-GPU launch spin in the closing barrier on the same host cores, which distorts it)
            line["cpu_baseline"] = {k: v for k, v in cpu_sample(workload, 3, 1).items() if k != "seconds_per_step"}
            line["cpu_baseline"]["config0"] = cpu_config0()
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


# DRAM bytes (read + written) of one launch of the backward main kernel on one batch entry of c1 (seqlen 8192, heads
# 32/8, head_dim 128, causal), from an ncu capture of the kernel as committed.
BWD_MAIN_DRAM_BYTES_PER_BATCH_ENTRY = 501.3e6


if __name__ == "__main__":
    main()
