"""Launcher: run one of the reference's entry scripts with the B200 backend selected.

    python -m lingbot_map_b200.run /path/to/lingbot-map/gct_profile.py --backend flashinfer --dtype bf16 ...

The script's own `--backend flashinfer` path (the default) is kept; the names it resolves for the global
block and the cache manager are rebound first (see select.install).  The reference package must be
importable (its repository root is put on sys.path when the script lives there).
"""
import os
import runpy
import sys


def main(argv=None):
    argv = list(sys.argv[1:] if argv is None else argv)
    if not argv:
        raise SystemExit(__doc__)
    script = os.path.abspath(argv[0])
    sys.path.insert(0, os.path.dirname(script))
    from . import select
    select.install()
    sys.argv = [script] + argv[1:]
    runpy.run_path(script, run_name="__main__")


if __name__ == "__main__":
    main()
