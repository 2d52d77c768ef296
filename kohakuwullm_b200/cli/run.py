"""``python -m kohakuwullm_b200.cli.run <script.py> --config <file.py> --set KEY=VALUE``."""

import sys

from kohakuwullm_b200.utils.config import run_script

if __name__ == "__main__":
    if len(sys.argv) < 2:
        raise SystemExit(__doc__)
    run_script(sys.argv[1], sys.argv[2:])
