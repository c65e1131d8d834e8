"""Offline generation demo (same role as the reference's examples/run_engine.py):

    python examples/run_engine.py                              # tiny random model
    python examples/run_engine.py --model DIR --prompt-ids 1,2,3 --max-tokens 16
"""
import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))

from servelab_b200.cli import main  # noqa: E402

if __name__ == "__main__":
    sys.exit(main())
