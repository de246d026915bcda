"""Device-zone profiler of the attention kernels: capture, decode, view.

Takes the place of the reference's device-zone profiler (reference zig/profile.zig:13-207 records begin / end ticks of
named zones per warp; src/zigfa/profile.py:98-391 decodes them; reports/profile_viewer.html shows them). Here a tuning
build of the library (`python zig-flash-attn_b200/build.py --trace`, which compiles with -DB200FA_TRACE into
zigfa/libb200fa_trace.so) makes one CTA of a launch log `event id << 48 | SM cycle counter` per warp role into a
buffer handed over with b200fa_set_trace; the regular build compiles the logging out. A zone is the span between two
consecutive events of one role, named after the event that ends it.

    B200FA_LIBRARY=zig-flash-attn_b200/zigfa/libb200fa_trace.so \
        python -m zigfa.profile --kernel bwd --head-dim 128 --out trace    # writes trace.json, trace.html, trace.txt

trace.json is in the Chrome trace-event format (chrome://tracing, ui.perfetto.dev); trace.html is a self-contained
timeline of the roles; trace.txt lists the events with their cycle offsets. `decode` and the writers are plain Python
and run without a GPU.
"""
from __future__ import annotations

import argparse
import ctypes
import json
from dataclasses import dataclass
from pathlib import Path

HEADER_WORDS = 64        # int64 words ahead of the events: the per-wait cycle sums of the kernels (slots 0-31)
EVENTS_PER_ROLE = 720
ROLES = 5

# (first id, ids in the family, role name, what has happened when the event fires); the index within the family is the
# key block (forward, modulo 100) or the iteration (backward, first ten iterations).
FORWARD_EVENTS = (
    (100, 100, "S of stage 0 issued"), (300, 100, "upper half of P0 present"), (500, 100, "all of P0 present"),
    (600, 100, "PV of stage 0 issued"), (1100, 100, "S of stage 1 issued"), (1300, 100, "upper half of P1 present"),
    (1500, 100, "all of P1 present"), (1600, 100, "PV of stage 1 issued"), (2000, 100, "scores of stage 0 present"),
    (3000, 100, "scores of stage 1 present"), (4000, 100, "row maximum of stage 0 known"),
    (5000, 100, "row maximum of stage 1 known"), (6000, 100, "upper half of P0 stored"),
    (7000, 100, "upper half of P1 stored"), (8000, 100, "all of P0 stored"), (9000, 100, "all of P1 stored"),
)
BACKWARD_EVENTS = (
    (50, 10, "P complete"), (100, 10, "dV issued"), (200, 10, "S of the next iteration issued"), (250, 10, "dS complete"),
    (300, 10, "dK and dQ issued"), (350, 10, "dO of the next iteration and the dQ drain ready"),
    (400, 10, "dP of the next iteration issued"), (500, 10, "scores ready"), (600, 10, "P stored"), (700, 10, "dP ready"),
    (800, 10, "dS stored"), (900, 10, "dQ drained"), (1000, 10, "dO load issued"), (1500, 10, "scores ready (last warp)"),
    (1600, 10, "P stored (last warp)"), (1700, 10, "dP ready (last warp)"), (1800, 10, "dS stored (last warp)"),
    (9100, 10, "dQ ready"), (9300, 10, "first chunk handed to the reduce-add"), (9400, 10, "staging buffer free"),
    (9500, 10, "staging stores issued"),
)
ROLE_NAMES = {
    "fwd": ("MMA issue", "softmax stage 0", "softmax stage 1", "load", "-"),
    "bwd": ("MMA issue", "compute (first warp)", "dQ drain", "load", "compute (last warp)"),
}
FAMILIES = {"fwd": FORWARD_EVENTS, "bwd": BACKWARD_EVENTS}


@dataclass(frozen=True)
class Event:
    role: int
    cycle: int      # SM cycles since the first event of the capture
    ident: int
    name: str
    index: int      # key block (forward) or iteration (backward)


@dataclass
class Capture:
    kernel: str
    events: list
    wait_cycles: list   # the 32 header counters of the tuning build (cycles spent in each wait, summed over warps)

    def roles(self):
        return sorted({event.role for event in self.events})

    def zones(self):
        """(role, begin, end, name, index) for consecutive events of each role."""
        result = []
        for role in self.roles():
            track = [event for event in self.events if event.role == role]
            for before, after in zip(track, track[1:]):
                result.append((role, before.cycle, after.cycle, after.name, after.index))
        return result


def name_of(kernel, ident):
    best = None
    for first, count, name in FAMILIES[kernel]:
        if first <= ident < first + count and (best is None or first > best[0]):
            best = (first, name)
    if best is None:
        return f"event {ident}", 0
    return best[1], ident - best[0]


def decode(words, kernel):
    """`words`: the int64 trace buffer as a sequence of Python ints (HEADER_WORDS + ROLES * EVENTS_PER_ROLE long)."""
    if kernel not in FAMILIES:
        raise ValueError(f"kernel must be one of {sorted(FAMILIES)}")
    raw = []
    for role in range(ROLES):
        start = HEADER_WORDS + EVENTS_PER_ROLE * role
        for word in words[start : start + EVENTS_PER_ROLE]:
            if word:
                raw.append((word & 0xFFFFFFFFFFFF, role, (word >> 48) & 0xFFFF))
    raw.sort()
    origin = raw[0][0] if raw else 0
    events = []
    for cycle, role, ident in raw:
        name, index = name_of(kernel, ident)
        events.append(Event(role, cycle - origin, ident, name, index))
    return Capture(kernel, events, [int(word) for word in words[:32]])


def to_text(capture):
    lines = [f"# {capture.kernel} kernel: one CTA, SM cycles since its first event"]
    names = ROLE_NAMES[capture.kernel]
    for event in capture.events:
        lines.append(f"{event.cycle:10d}  {names[event.role]:22s} [{event.index:3d}]  {event.name}")
    return "\n".join(lines) + "\n"


def to_chrome_trace(capture, cycles_per_microsecond=1000.0):
    """Chrome trace-event JSON: one thread per role, one complete ('X') slice per zone; 1000 cycles are shown as 1 us
    unless the SM clock is given."""
    names = ROLE_NAMES[capture.kernel]
    records = [{"name": "thread_name", "ph": "M", "pid": 0, "tid": role, "args": {"name": names[role]}}
               for role in capture.roles()]
    for role, begin, end, name, index in capture.zones():
        records.append({"name": f"{name} [{index}]", "ph": "X", "pid": 0, "tid": role,
                        "ts": begin / cycles_per_microsecond, "dur": max(end - begin, 1) / cycles_per_microsecond})
    return json.dumps({"traceEvents": records, "displayTimeUnit": "ns"})


def to_html(capture, width=1600):
    """A self-contained timeline: one lane per role, one rectangle per zone, the zone name as its tooltip."""
    zones = capture.zones()
    roles = capture.roles()
    names = ROLE_NAMES[capture.kernel]
    last = max((end for _, _, end, _, _ in zones), default=1)
    scale = (width - 220) / max(last, 1)
    palette = ("#4e79a7", "#f28e2b", "#59a14f", "#e15759", "#76b7b2", "#edc948", "#b07aa1", "#9c755f")
    colours = {}
    parts = [f'<svg xmlns="http://www.w3.org/2000/svg" width="{width}" height="{40 * len(roles) + 40}" font-family="monospace" font-size="11">']
    for lane, role in enumerate(roles):
        parts.append(f'<text x="4" y="{40 * lane + 34}">{names[role]}</text>')
    for role, begin, end, name, index in zones:
        colour = colours.setdefault(name, palette[len(colours) % len(palette)])
        lane = roles.index(role)
        parts.append(f'<rect x="{220 + begin * scale:.1f}" y="{40 * lane + 16}" width="{max((end - begin) * scale, 0.5):.1f}" height="26" '
                     f'fill="{colour}" stroke="#222" stroke-width="0.3"><title>{name} [{index}]: {begin}..{end} ({end - begin} cycles)</title></rect>')
    parts.append(f'<text x="220" y="12">0</text><text x="{width - 80}" y="12">{last} cycles</text></svg>')
    legend = "".join(f'<span style="background:{colour};padding:2px 6px;margin:2px;display:inline-block">{name}</span>'
                     for name, colour in colours.items())
    return f"<!doctype html><html><body><h3>{capture.kernel} kernel, one CTA</h3>{''.join(parts)}<p>{legend}</p></body></html>\n"


def capture(kernel, head_dim=128, seqlen=8192, batch=1, heads_q=32, heads_kv=8, causal=True):
    """Runs one forward (and, for kernel='bwd', one backward) launch of a fixed-length problem with tracing on and
    returns the decoded Capture. Needs a GPU and a library built with -DB200FA_TRACE (else the buffer stays empty)."""
    import torch

    from . import _impl  # noqa: F401
    from ._impl import lib, ops

    library = lib.library()
    torch.manual_seed(0)
    make = lambda heads: torch.randn(batch, seqlen, heads, head_dim, device="cuda", dtype=torch.bfloat16)
    q, k, v, dout = make(heads_q), make(heads_kv), make(heads_kv), make(heads_q)
    out = torch.empty_like(q)
    lse = torch.empty(batch, heads_q, seqlen, dtype=torch.float32, device="cuda")
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    scale, window = head_dim**-0.5, (-1, 0 if causal else -1)
    forward = lambda: ops.launch_forward(q, k, v, out, lse, None, None, scale, *window)
    backward = lambda: ops.launch_backward(dout, q, k, v, out, lse, dq, dk, dv, None, None, scale, *window)
    forward()
    if kernel == "bwd":
        backward()
    torch.cuda.synchronize()
    trace = torch.zeros(HEADER_WORDS + ROLES * EVENTS_PER_ROLE + 64, dtype=torch.int64, device="cuda")
    library.b200fa_set_trace(ctypes.c_void_p(trace.data_ptr()))
    try:
        (backward if kernel == "bwd" else forward)()
        torch.cuda.synchronize()
    finally:
        library.b200fa_set_trace(None)
    return decode(trace.tolist(), kernel)


def main(arguments=None):
    parser = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    parser.add_argument("--kernel", choices=sorted(FAMILIES), default="bwd")
    parser.add_argument("--head-dim", type=int, default=128)
    parser.add_argument("--seqlen", type=int, default=8192)
    parser.add_argument("--dense", action="store_true", help="no causal mask")
    parser.add_argument("--out", default="trace", help="path prefix of the .json, .html and .txt files")
    options = parser.parse_args(arguments)
    result = capture(options.kernel, options.head_dim, options.seqlen, causal=not options.dense)
    if not result.events:
        raise SystemExit("no events: the loaded library was not built with -DB200FA_TRACE (python build.py --trace, then "
                         "B200FA_LIBRARY=.../zigfa/libb200fa_trace.so)")
    prefix = Path(options.out)
    prefix.with_suffix(".json").write_text(to_chrome_trace(result))
    prefix.with_suffix(".html").write_text(to_html(result))
    prefix.with_suffix(".txt").write_text(to_text(result))
    print(f"{len(result.events)} events of {len(result.roles())} roles -> {prefix}.json / .html / .txt")


if __name__ == "__main__":
    main()
