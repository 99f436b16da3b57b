"""``python -m fbamtrain_b200.tenscmp a.safetensors b.safetensors -t 0.3`` — compares two safetensors files tensor
by tensor with an absolute threshold; exit status 0 when everything matches (reference: ``src/tenscmp.cpp:12-79``).
The comparison itself is the native runtime's ``fbam_tenscmp``."""
from __future__ import annotations

import argparse
import sys

from . import runtime


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="tenscmp")
    ap.add_argument("first")
    ap.add_argument("second")
    ap.add_argument("-t", "--threshold", type=float, default=1e-3)
    a = ap.parse_args(argv)
    bad, report = runtime.tenscmp(a.first, a.second, a.threshold)
    if report:
        sys.stdout.write(report)
    print(f"{bad} tensor(s) differ beyond {a.threshold}" if bad else "all tensors match")
    return 1 if bad else 0


if __name__ == "__main__":
    sys.exit(main())
