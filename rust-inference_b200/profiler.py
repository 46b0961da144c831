"""Section timers: where a step's time goes, by part.

Off by default.  ``enable()`` (the runner's ``--profile``) makes ``section(name)`` bracket the
work inside it with a pair of CUDA events on the current stream; ``report()`` waits for the
device, adds up each section's event times and prints them largest first with share and number
of calls, as thanhauco/rust-inference's profiler does for its host timers
(src/profiler.rs:12-135; hooked into its model at src/models/qwen3.rs:82-99, 132-141, 274-286).
The times are device times of eager launches, one section after the other, so steps are not
replayed from CUDA graphs while the timers are on, and overlap between neighbouring kernels
(programmatic dependent launch) shows up in the earlier section.

The parts call ``section`` around their kernels; a part of another architecture names its own
sections, nothing here lists them.
"""
from __future__ import annotations

from typing import Dict, List, Tuple

import torch

_enabled = False
_open: List[Tuple[str, "torch.cuda.Event", "torch.cuda.Event"]] = []
_totals: Dict[str, List[float]] = {}           # name -> [milliseconds, calls]


class _Off:
    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False


_OFF = _Off()


class _Section:
    __slots__ = ("name", "start")

    def __init__(self, name: str):
        self.name = name

    def __enter__(self):
        self.start = torch.cuda.Event(enable_timing=True)
        self.start.record()
        return self

    def __exit__(self, *exc):
        end = torch.cuda.Event(enable_timing=True)
        end.record()
        _open.append((self.name, self.start, end))
        if len(_open) >= 4096:
            _drain()
        return False


def enable(on: bool = True) -> None:
    global _enabled
    _enabled = bool(on) and torch.cuda.is_available()


def enabled() -> bool:
    return _enabled


def section(name: str):
    """``with section("attention"): ...``; costs nothing while the timers are off."""
    return _Section(name) if _enabled else _OFF


def _drain() -> None:
    if not _open:
        return
    _open[-1][2].synchronize()
    for name, start, end in _open:
        t = _totals.setdefault(name, [0.0, 0])
        t[0] += start.elapsed_time(end)
        t[1] += 1
    _open.clear()


def reset() -> None:
    _open.clear()
    _totals.clear()


def snapshot() -> List[Tuple[str, float, int]]:
    """(section, seconds, calls) of every section that ran, largest first."""
    _drain()
    return sorted(((n, ms / 1e3, calls) for n, (ms, calls) in _totals.items()), key=lambda r: -r[1])


def report() -> str:
    rows = snapshot()
    total = sum(r[1] for r in rows)
    out = ["section                  total(s)   share    calls"]
    for name, secs, calls in rows:
        share = 100.0 * secs / total if total > 0 else 0.0
        out.append(f"{name:<22} {secs:>10.4f} {share:>6.1f}% {calls:>8}")
    return "\n".join(out) + "\n"
