#!/usr/bin/env python
"""Entry point with the name and place that command lines written for the reference use
(tracker/dmlc_mpi.py ...); the launcher itself is ps_lite_b200.launch.mpi."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from ps_lite_b200.launch.mpi import main  # noqa: E402

if __name__ == "__main__":
    sys.exit(main())
