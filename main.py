#!/usr/bin/env python
"""Command-line entry point, flag-compatible with the reference's ``main.py``::

    torchrun --nnodes=1 --nproc_per_node=8 main.py -s <scene> -m <model> --bvh_depth 3 \\
        --MAX_BATCH_SIZE 2 --MAX_LOAD 4 -r 1 [--eval] [--EVAL_ONLY]

Reads ``WORLD_SIZE/RANK/LOCAL_RANK/MASTER_ADDR/MASTER_PORT`` from the environment (single process when
they are absent).  Unlike the reference (``main.py:58-68``) a failure is not swallowed: the traceback is
logged to ``debugger/debug_<rank>_<time>.txt`` and the process exits non-zero so that peers and
launchers notice.
"""
import sys

from retinags_b200.cli import main

if __name__ == "__main__":
    sys.exit(main())
