"""Trace replay: feed given token ids through a model step by step, write logits.

It samples nothing and has no forward pass, cache or loader of its own: every
step goes through ``ModelRunner.step`` with the framework's cache manager, the
same objects generation uses.  The reference's nearest thing is a manual
cross-validation script that drives the scheduler by hand and prints logit
differences (scripts/debug/debug_spec_crossval.py:50-71).

Input (stdin), one JSON object per line:

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

For a step that wants logits, ``<out>/<step>.f32`` receives them as little-endian
float32 [wanted, vocab], in the order of the entries and of ``want``.  After each
step ``done <step>`` is printed and flushed.
"""

from __future__ import annotations

import argparse
import json
import os
import sys
from typing import Dict


class TraceSession:
    """The state of one replay: a ModelRunner, its cache manager, and how many
    tokens each live request holds.  ``run_step`` executes one trace step."""

    def __init__(self, model: str, dtype: str, max_tokens: int, page_size: int = 16,
                 max_live: int = 8, poison_cache: bool = False, cuda_graphs: bool = False,
                 runner=None):
        """``model``: a model folder; or hand in a ``runner`` built elsewhere (a typed config
        with weights made on the device).  ``poison_cache`` and ``cuda_graphs`` are what
        tests switch on: unwritten cache slots hold a huge value; steps of single tokens
        replay captured graphs, as in generation."""
        from .config.engine import CacheConfig
        from .engine.runner import ModelRunner

        self.max_tokens, self.max_live = max_tokens, max_live
        if runner is None:
            pages = max(1, -(-max_tokens // page_size))
            runner = ModelRunner.from_folder(
                model, dtype=dtype, max_num_seqs=max_live, cuda_graphs=cuda_graphs,
                cache_config=CacheConfig(block_size=page_size, num_blocks=pages,
                                         poison_cache=poison_cache))
        self.runner = runner
        self.cache = self.runner.cache
        self.held: Dict[str, int] = {}             # request -> tokens in the cache

    def run_step(self, step: dict):
        """Returns the step's logits [wanted, vocab] as a float32 numpy array, or
        None when nothing was wanted."""
        runner, cache, held = self.runner, self.cache, self.held
        entries, ids = [], []
        for e in step.get("entries", []):
            rid, tokens = str(e["id"]), [int(t) for t in e["tokens"]]
            runner.check_tokens(tokens)
            if rid not in held:
                if not cache.open(rid):
                    raise RuntimeError(f"no state slot left for request {rid} "
                                       f"(more than {self.max_live} live requests)")
                held[rid] = 0
            start = held[rid]
            if not cache.ensure(rid, start + len(tokens)):
                raise RuntimeError(f"step {step.get('step')}: out of cache pages for request "
                                   f"{rid}; --max-tokens {self.max_tokens} is too small")
            entries.append(runner.entry(rid, tokens, start, e.get("want", ())))
            ids.append(rid)
        logits = runner.step(entries)
        result = None
        if logits.shape[0] > 0:
            result = logits.to("cpu").contiguous().numpy().astype("<f4", copy=False)
        for rid, be in zip(ids, entries):
            held[rid] += len(be.tokens)
            cache.trim(rid, held[rid])
        for rid in step.get("end", []):
            cache.release(str(rid))
            held.pop(str(rid), None)
        return result


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder for <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens live requests hold at any time (each rounded up to 64)")
    ap.add_argument("--page-size", type=int, default=16, help="tokens per cache page")
    ap.add_argument("--max-live", type=int, default=8, help="state slots (live requests)")
    args = ap.parse_args(argv)

    print("[trace_run] loading (kernels are compiled at first use)", file=sys.stderr, flush=True)
    os.makedirs(args.out, exist_ok=True)
    try:
        session = TraceSession(args.model, args.dtype, args.max_tokens, args.page_size,
                               args.max_live)
        print("[trace_run] ready", file=sys.stderr, flush=True)
        for line in sys.stdin:
            line = line.strip()
            if not line:
                continue
            step = json.loads(line)
            logits = session.run_step(step)
            if logits is not None:
                logits.tofile(os.path.join(args.out, f"{step['step']}.f32"))
            print(f"done {step['step']}", flush=True)
    except RuntimeError as e:
        print(f"trace_run: {e}", file=sys.stderr, flush=True)
        return 1
    return 0


if __name__ == "__main__":
    sys.exit(main())
