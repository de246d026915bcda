"""The device-zone profiler (zigfa/profile.py; reference src/zigfa/profile.py:98-391): decoding of the trace buffer and
the three writers on the CPU with a synthetic buffer, and one real capture of each kernel on the GPU with the tuning
build of the library."""
import json
import os
import subprocess
import sys
from pathlib import Path

import pytest

from zigfa import profile

ROOT = Path(__file__).resolve().parent.parent
PACKAGE = ROOT / "zig-flash-attn_b200"


def synthetic_buffer():
    words = [0] * (profile.HEADER_WORDS + profile.ROLES * profile.EVENTS_PER_ROLE)
    words[3] = 12345  # a wait-cycle counter of the header
    clock = 1_000_000
    log = {0: [(50 + 5, 40), (100 + 5, 700), (200 + 5, 1500), (250 + 5, 1900)],  # MMA role, iteration 5
           1: [(500 + 5, 10), (600 + 5, 900), (700 + 5, 1000), (800 + 5, 2600)],
           2: [(9100 + 5, 2700), (900 + 5, 3300)]}
    for role, events in log.items():
        for n, (ident, offset) in enumerate(events):
            words[profile.HEADER_WORDS + profile.EVENTS_PER_ROLE * role + n] = (ident << 48) | (clock + offset)
    return words


def test_decode_names_events_and_orders_them_by_cycle():
    capture = profile.decode(synthetic_buffer(), "bwd")
    assert capture.wait_cycles[3] == 12345
    assert [event.cycle for event in capture.events] == sorted(event.cycle for event in capture.events)
    assert capture.events[0].cycle == 0 and capture.events[0].name == "scores ready" and capture.events[0].index == 5
    names = {(event.role, event.name) for event in capture.events}
    assert (0, "dV issued") in names and (2, "dQ drained") in names and (1, "dS stored") in names
    zones = capture.zones()
    assert (0, 30, 690, "dV issued", 5) in zones  # from "P complete" at 40 - 10 to "dV issued" at 700 - 10
    assert capture.roles() == [0, 1, 2]
    with pytest.raises(ValueError):
        profile.decode([], "sideways")


def test_writers_produce_a_chrome_trace_an_html_timeline_and_a_listing():
    capture = profile.decode(synthetic_buffer(), "bwd")
    trace = json.loads(profile.to_chrome_trace(capture))
    slices = [record for record in trace["traceEvents"] if record["ph"] == "X"]
    assert len(slices) == len(capture.zones()) and all(record["dur"] > 0 for record in slices)
    assert {record["args"]["name"] for record in trace["traceEvents"] if record["ph"] == "M"} == {"MMA issue", "compute (first warp)", "dQ drain"}
    html = profile.to_html(capture)
    assert html.count("<rect") == len(capture.zones()) and "dQ drained [5]" in html
    text = profile.to_text(capture)
    assert text.count("\n") == len(capture.events) + 1 and "dS stored" in text


@pytest.mark.gpu
@pytest.mark.parametrize("kernel", ["fwd", "bwd"])
def test_capture_of_a_real_launch_with_the_tuning_build(kernel, tmp_path):
    library = PACKAGE / "zigfa" / "libb200fa_trace.so"
    if not library.exists():
        subprocess.run([sys.executable, str(PACKAGE / "build.py"), "--trace"], check=True, capture_output=True)
    environment = dict(os.environ, B200FA_LIBRARY=str(library), PYTHONPATH=str(PACKAGE))
    prefix = tmp_path / "trace"
    result = subprocess.run([sys.executable, "-m", "zigfa.profile", "--kernel", kernel, "--seqlen", "4096", "--out", str(prefix)],
                            env=environment, capture_output=True, text=True)
    assert result.returncode == 0, result.stdout + result.stderr
    trace = json.loads(prefix.with_suffix(".json").read_text())
    lanes = {record["tid"] for record in trace["traceEvents"] if record["ph"] == "X"}
    assert len(lanes) >= 3, "the MMA, softmax / compute and drain or second softmax roles must all have logged"
    assert "<svg" in prefix.with_suffix(".html").read_text()
    assert ("P stored" if kernel == "bwd" else "all of P0 stored") in prefix.with_suffix(".txt").read_text()
