"""``python -m fbamtrain_b200 ...`` is the command-line trainer (same as ``python -m fbamtrain_b200.cli``)."""
import sys

from .cli import main

if __name__ == "__main__":
    sys.exit(main())
