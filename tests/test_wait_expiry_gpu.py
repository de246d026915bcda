"""A device-side wait that really runs out.

Every wait in the kernels is a bounded `mbarrier.try_wait` loop (csrc/ptx.cuh): when its budget is spent the CTA
records `code << 16 | CTA` in a status word, raises its abort flag, frees its TMEM and returns. The budget is two
seconds in the library, so a healthy run never sees this path. Here a small kernel built from the same header with a
budget of one millisecond waits on a barrier that nobody arrives at. The test checks that the launch comes back by
itself with the expected status, that the CUDA context is still usable, and that an ordinary attention call afterwards
is still correct. The wait gives up and returns; nothing traps, faults or spins without a limit.
"""
import ctypes
import shutil
import subprocess
from pathlib import Path

import pytest
import torch

import attention_oracle as oracle
import zigfa
from zigfa._impl import lib

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parent.parent
WAIT_S_FULL = 5  # WaitCode kWaitSFull in csrc/ptx.cuh


def build_test_kernel(directory):
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    target = directory / "libexpiring_wait.so"
    command = [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-O2", "-std=c++17", "-shared", "-Xcompiler", "-fPIC",
               "-I", str(ROOT / "zig-flash-attn_b200" / "csrc"), str(ROOT / "tests" / "expiring_wait.cu"), "-o", str(target)]
    result = subprocess.run(command, capture_output=True, text=True)
    assert result.returncode == 0, result.stdout + result.stderr
    return ctypes.CDLL(str(target))


def test_a_wait_that_runs_out_returns_with_its_status_and_leaves_the_gpu_usable(tmp_path):
    torch.cuda.init()
    torch.zeros(1, device="cuda")
    kernel = build_test_kernel(tmp_path)
    kernel.run_expiring_wait.restype = ctypes.c_int
    kernel.run_expiring_wait.argtypes = [ctypes.c_int] + [ctypes.c_void_p] * 3
    blocks = 3
    status, passed, milliseconds = ctypes.c_int(-1), ctypes.c_int(-1), ctypes.c_float(-1)
    error = kernel.run_expiring_wait(blocks, ctypes.byref(status), ctypes.byref(passed), ctypes.byref(milliseconds))
    assert error == 0, f"CUDA error {error}: the launch did not come back cleanly"
    assert passed.value == 0, "a warp saw a barrier complete that nobody arrived at"
    assert status.value >> 16 == WAIT_S_FULL and 0 <= (status.value & 0xFFFF) < blocks, hex(status.value)
    assert 1.0 <= milliseconds.value < 1000.0, f"the wait took {milliseconds.value} ms for a 1 ms budget"

    # the context is intact: an ordinary forward + backward afterwards is right, and the library saw no timeout
    torch.manual_seed(5)
    q = torch.randn(1, 384, 4, 128, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    k, v = (torch.randn(1, 384, 2, 128, device="cuda", dtype=torch.bfloat16, requires_grad=True) for _ in range(2))
    dout = torch.randn_like(q)
    out = zigfa.flash_attn_func(q, k, v, causal=True)
    dq, dk, dv = torch.autograd.grad(out, (q, k, v), dout)
    ref_out, _, ref_dq, ref_dk, ref_dv = oracle.gradients(
        oracle.attention, q.detach(), k.detach(), v.detach(), dout, window_size=(-1, 0), softmax_scale=128**-0.5)
    for ours, reference in ((out, ref_out), (dq, ref_dq), (dk, ref_dk), (dv, ref_dv)):
        bound = 3 * 2**-7 * reference.abs().max().item() + 1e-4  # the reference's own BF16 rule (tests/checks.py:11-13)
        assert (ours.float() - reference.float()).abs().max().item() <= bound
    assert lib.library().b200fa_device_status() == 0
