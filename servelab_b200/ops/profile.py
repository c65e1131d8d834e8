"""Per-kernel times inside a real step, behind a switch.

    with StepProfile() as prof:
        runner.step(entries)              # eagerly: a replayed graph launches nothing from Python
    print(prof.render())

A CUDA event is recorded after every launch of this package's kernels (``library.after_launch``)
and after every library GEMM that ``ops.linear`` calls; the time between two consecutive events
is charged to the kernel that the second one follows.  The events serialise the stream, so
kernels do not overlap their predecessors as they do in a replayed graph: the shares are those
of the kernels one after the other with warm caches, the sum is a little above the step's time.
The reference only documents profiler command lines (docs/benchmark_guide.md:29-49).
"""

from __future__ import annotations

from collections import OrderedDict
from typing import Dict, List, Tuple

import torch

from . import library as L


class StepProfile:
    def __init__(self):
        self.events: List[Tuple[str, torch.cuda.Event]] = []
        self._saved = None

    def mark(self, name: str) -> None:
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        self.events.append((name, ev))

    def __enter__(self) -> "StepProfile":
        self._saved = L.after_launch
        self.mark("(start)")
        L.after_launch = self.mark
        return self

    def __exit__(self, *exc) -> None:
        L.after_launch = self._saved

    def totals(self) -> "OrderedDict[str, Tuple[int, float]]":
        """kernel name -> (launches, microseconds in total), in order of first launch."""
        torch.cuda.synchronize()
        out: "OrderedDict[str, Tuple[int, float]]" = OrderedDict()
        for (_, a), (name, b) in zip(self.events, self.events[1:]):
            n, us = out.get(name, (0, 0.0))
            out[name] = (n + 1, us + a.elapsed_time(b) * 1e3)
        return out

    def summary(self, steps: int = 1) -> Dict[str, float]:
        """kernel name -> microseconds per step."""
        return {name: round(us / steps, 2) for name, (_, us) in self.totals().items()}

    def render(self, steps: int = 1) -> str:
        totals = self.totals()
        whole = sum(us for _, us in totals.values()) or 1.0
        rows = [("kernel", "launches/step", "us/step", "us/launch", "share")]
        for name, (n, us) in sorted(totals.items(), key=lambda kv: -kv[1][1]):
            rows.append((name, f"{n / steps:.1f}", f"{us / steps:.1f}", f"{us / n:.2f}", f"{us / whole:.1%}"))
        rows.append(("total", "", f"{whole / steps:.1f}", "", ""))
        widths = [max(len(r[i]) for r in rows) for i in range(5)]
        return "\n".join("  ".join(c.ljust(w) for c, w in zip(r, widths)) for r in rows)


def mark(name: str) -> None:
    """Called by code that launches a library kernel (a vendor GEMM), so that its time is not
    charged to the kernel after it."""
    if L.after_launch is not None:
        L.after_launch(name)
