"""Writes tests/golden/plain_tiny.npz: logits of the plain implementation
(tests/plain_model.py) on the tiny random models of tests/helpers.py, so that a change in the
plain implementation itself shows up.

The reference's own model code (servelab/models/decoder.py) is absent from its
tree -- its .gitignore excludes the whole package -- so it cannot be imported or
compiled here; these numbers rest on the reference's formulas as restated in
servelab/parallel/tp_model.py:121-157 and servelab/engine/speculative.py:53-87,
not on an execution of its model.

    python tests/golden/make_golden.py
"""
import os
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

import helpers as H  # noqa: E402


def compute():
    out = {}
    for name, (cfg, seed, _) in H.CONFIGS.items():
        with tempfile.TemporaryDirectory() as d:
            H.make_model(d, cfg, seed)
            ids = H.random_ids(40, cfg["vocab_size"], 4242 + seed)
            logits = H.plain_logits(d, ids)
        out[f"{name}_ids"] = np.asarray(ids, dtype=np.int32)
        out[f"{name}_logits_rows"] = logits[[0, 1, 17, 39]].astype(np.float32)
    return out


if __name__ == "__main__":
    np.savez(os.path.join(HERE, "plain_tiny.npz"), **compute())
    print("wrote", os.path.join(HERE, "plain_tiny.npz"))
