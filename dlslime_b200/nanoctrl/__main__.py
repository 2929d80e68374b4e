"""``python -m dlslime_b200.nanoctrl <server|start|status|stop|obs> ...`` runs the native nanoctrl program."""

import os
import sys


def main() -> int:
    from .. import _build

    exe = _build.nanoctrl_bin_path()
    if not exe.exists():
        _build.build_host()
    os.execv(str(exe), [str(exe), *sys.argv[1:]])
    return 127


if __name__ == "__main__":
    sys.exit(main())
