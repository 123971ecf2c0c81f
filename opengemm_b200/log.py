"""One-line progress messages on stderr, prefixed like the reference's (opengemm/python/log.py:3-4)."""

import sys


def log(message):
    print(f"[OpenGEMM] {message}", file=sys.stderr, flush=True)
