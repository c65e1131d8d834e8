"""A timeline of a step's kernels as the device saw them (measurements).

    with DeviceTimeline() as tl:          # before the graphs are captured: the buffer's address
        engine = ...                      # is an argument of the launches and is baked into them
        run a few steps
        tl.reset()
        run the step to look at
    print(tl.render())

One thread of every block of the decode-step kernels (the tcgen05 products, the decode
attention, the norms) records the device's nanosecond timer when the block starts, when its
wait for the preceding kernel returns, when its main loop is done and when it ends
(``csrc/common.cuh``).  ``launches()`` condenses that to one row per launch: first start,
first and last return of the wait, last main loop done (the norms: inputs loaded), an extra
mark (the cluster norm: sums of squares exchanged; the cluster products: the blocks' results
parked, from where a block sums its share of the tokens), last end, relative to the first event;
``render()`` prints them with the gaps between consecutive launches, which is what the time of
a decode step beyond its memory traffic consists of.  The reference has no counterpart (its
docs name profiler command lines, docs/benchmark_guide.md:29-49).
"""

from __future__ import annotations

from typing import Dict, List

import torch

from . import library as L

KERNELS = {1: "gemm_tc_decode", 2: "gemm_tc_cluster (store)", 3: "gemm_tc_cluster (q|k|v + rope)",
           4: "decode_attention_ws", 5: "add_rmsnorm", 6: "add_rmsnorm_parts_cluster",
           7: "gemm_tc_cluster (+ resid, norm)"}


LAUNCHES, BLOCKS, EVENTS = 2048, 512, 5     # the slot layout of csrc/common.cuh (512 launches a library)


class DeviceTimeline:
    def __init__(self, device: str = "cuda:0"):
        self.buf = torch.zeros(2 * LAUNCHES * BLOCKS * EVENTS, dtype=torch.int64, device=device)

    def _set(self, ptr) -> None:
        # every library numbers its launches itself: each gets a range of launch slots of its own
        for n, lib in enumerate(L.loaded_libraries()):
            lib.slb_set_trace.argtypes = [L.P, L.I]
            lib.slb_set_trace(ptr, n)

    def __enter__(self) -> "DeviceTimeline":
        L.trace_buffer = self.buf.data_ptr()       # libraries loaded later get it too
        self._set(self.buf.data_ptr())
        return self

    def __exit__(self, *exc) -> None:
        torch.cuda.synchronize()
        L.trace_buffer = None
        self._set(None)

    def reset(self) -> None:
        torch.cuda.synchronize()
        self.buf.zero_()

    def events(self) -> List[dict]:
        torch.cuda.synchronize()
        host = self.buf.cpu().view(LAUNCHES, BLOCKS, EVENTS, 2)
        used = (host[..., 0] != 0).nonzero().tolist()
        out = []
        for launch, block, event in used:
            now, meta = host[launch, block, event].tolist()
            meta &= (1 << 64) - 1
            out.append({"ns": now, "kernel": (meta >> 48) & 0xffff, "event": (meta >> 40) & 0xff,
                        "sm": (meta >> 24) & 0xffff, "block": meta & 0xffffff, "seq": launch})
        return out

    def launches(self) -> List[dict]:
        """One row per launch, in order of first start; times in microseconds from the first event."""
        ev = self.events()
        if not ev:
            return []
        t0 = min(e["ns"] for e in ev)
        by: Dict[tuple, dict] = {}
        for e in ev:
            row = by.setdefault((e["kernel"], e["seq"]), {"kernel": KERNELS.get(e["kernel"], str(e["kernel"])),
                                                          "seq": e["seq"], "blocks": set(), "sms": set(), "t": {}})
            row["blocks"].add(e["block"])
            row["sms"].add(e["sm"])
            row["t"].setdefault(e["event"], []).append((e["ns"] - t0) / 1e3)
        out = []
        for row in by.values():
            t = row["t"]
            out.append({"kernel": row["kernel"], "seq": row["seq"], "blocks": len(row["blocks"]),
                        "sms": len(row["sms"]),
                        "first_start": min(t.get(0, [0.0])), "last_start": max(t.get(0, [0.0])),
                        "first_waited": min(t.get(1, [float("nan")])), "last_waited": max(t.get(1, [float("nan")])),
                        "last_loop_done": max(t.get(2, [float("nan")])),
                        "last_extra": max(t.get(4, [float("nan")])),
                        "last_end": max(t.get(3, [0.0]) + (t.get(4, [0.0]) if row["kernel"] == KERNELS[4] else [0.0]))})
        out.sort(key=lambda r: r["first_waited"] if r["first_waited"] == r["first_waited"] else r["first_start"])
        return out

    def render(self, limit: int = 80) -> str:
        rows = self.launches()[:limit]
        head = ("kernel", "blocks", "SMs", "first start", "last start", "waited (first..last)",
                "loop done", "extra", "end", "ran", "after prev end")
        table = [head]
        prev_end = None
        for r in rows:
            ran = r["last_end"] - r["first_waited"]
            gap = "" if prev_end is None else f"{r['first_waited'] - prev_end:+.2f}"
            table.append((r["kernel"], str(r["blocks"]), str(r["sms"]), f"{r['first_start']:.2f}",
                          f"{r['last_start']:.2f}", f"{r['first_waited']:.2f}..{r['last_waited']:.2f}",
                          f"{r['last_loop_done']:.2f}", f"{r['last_extra']:.2f}", f"{r['last_end']:.2f}",
                          f"{ran:.2f}", gap))
            prev_end = r["last_end"]
        widths = [max(len(row[i]) for row in table) for i in range(len(head))]
        return "\n".join("  ".join(c.ljust(w) for c, w in zip(row, widths)) for row in table)
