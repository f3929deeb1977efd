#!/usr/bin/env python3
"""One-command demo, as the reference's ``run_demo.py``:  ``python run_demo.py --model tiny``.

Shows a cold request, a warm request whose shared prefix is served from cached pages,
and a batch.  All options of ``python -m hetero_serve_b200`` apply."""

import sys

from hetero_serve_b200.cli import main

if __name__ == "__main__":
    sys.exit(main())
