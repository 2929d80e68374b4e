"""``dlslime-cache`` command line: start / status / stop a cache service process.

    python -m dlslime_b200.cache.cli start --ctrl http://127.0.0.1:3000 --memory-size 1G [--slab-size 256K]
    python -m dlslime_b200.cache.cli status
    python -m dlslime_b200.cache.cli stop

``start`` re-executes this module detached (``__run``) and records pid / meta / log files under
``$DLSLIME_CACHE_RUNTIME_DIR``, else ``$XDG_RUNTIME_DIR/dlslime-cache``, else ``/tmp/dlslime-cache``, as the
reference's CLI does (``dlslime/cache/cli.py:36-70,404-424,494-627`` in the reference). Sizes accept the
suffixes K/M/G/T (optionally followed by ``iB`` or ``B``), powers of 1024. ``--config file.json`` supplies
defaults for any option. Built on argparse.
"""

from __future__ import annotations

import argparse
import json
import os
import re
import signal
import subprocess
import sys
import time
from pathlib import Path

from .types import DEFAULT_AGENT_ALIAS, DEFAULT_SLAB_SIZE

_SIZE = re.compile(r"^\s*(\d+(?:\.\d+)?)\s*([KMGT]?)(?:i?B)?\s*$", re.IGNORECASE)


def parse_size(text: str | int) -> int:
    if isinstance(text, int):
        return text
    m = _SIZE.match(str(text))
    if not m:
        raise argparse.ArgumentTypeError(f"invalid size {text!r} (examples: 262144, 256K, 1G, 2GiB)")
    value = float(m.group(1)) * 1024 ** " KMGT".index(m.group(2).upper() or " ")
    if value != int(value):
        raise argparse.ArgumentTypeError(f"size {text!r} is not a whole number of bytes")
    return int(value)


def runtime_dir() -> Path:
    if os.environ.get("DLSLIME_CACHE_RUNTIME_DIR"):
        return Path(os.environ["DLSLIME_CACHE_RUNTIME_DIR"])
    if os.environ.get("XDG_RUNTIME_DIR"):
        return Path(os.environ["XDG_RUNTIME_DIR"]) / "dlslime-cache"
    return Path("/tmp/dlslime-cache")


def service_mode_error(args) -> str | None:
    """Why this combination of options cannot serve data, or None when it is fine."""
    if args.metadata_only:
        return None
    if not args.ctrl:
        return "a data-serving cache needs --ctrl (the NanoCtrl address); use --metadata-only for a directory without memory"
    if args.memory_size <= 0:
        return "a data-serving cache needs a non-zero --memory-size; use --metadata-only for a directory without memory"
    if args.memory_size % args.slab_size != 0:
        return "--memory-size must be a multiple of --slab-size"
    return None


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(prog="dlslime-cache", description="DLSlimeCache service control")
    sub = p.add_subparsers(dest="command", required=True)

    def service_options(sp):
        sp.add_argument("--config", help="JSON file with defaults for the options below")
        sp.add_argument("--host", default="127.0.0.1")
        sp.add_argument("--port", type=int, default=8765)
        sp.add_argument("--ctrl", default=None, help="NanoCtrl URL; enables the PeerAgent data path and discovery")
        sp.add_argument("--scope", default=None)
        sp.add_argument("--alias", default=DEFAULT_AGENT_ALIAS, help="PeerAgent alias of the cache")
        sp.add_argument("--slab-size", type=parse_size, default=DEFAULT_SLAB_SIZE)
        sp.add_argument("--memory-size", type=parse_size, default=0)
        sp.add_argument("--device", default=None, help="cuda:N keeps the cache memory in HBM (reached over NVLink)")
        sp.add_argument("--metadata-only", action="store_true", help="directory only: no memory, no PeerAgent")

    service_options(sub.add_parser("start", help="start a detached cache service"))
    service_options(sub.add_parser("__run", help=argparse.SUPPRESS))
    sub.add_parser("status", help="report whether the detached service is alive and healthy")
    stop = sub.add_parser("stop", help="stop the detached service")
    stop.add_argument("--force", action="store_true")
    return p


def parse_args(argv=None):
    parser = build_parser()
    args = parser.parse_args(argv)
    cfg = getattr(args, "config", None)
    if cfg:
        with open(cfg) as f:
            defaults = json.load(f)
        sp = next(a for a in parser._subparsers._group_actions[0].choices.items() if a[0] == args.command)[1]
        sp.set_defaults(**{k.replace("-", "_"): (parse_size(v) if k.replace("-", "_") in ("slab_size", "memory_size") else v)
                           for k, v in defaults.items()})
        args = parser.parse_args(argv)
    return args


def service_argv(args) -> list[str]:
    """The argument list that reproduces ``args`` for the detached ``__run`` process."""
    out = ["--host", args.host, "--port", str(args.port), "--slab-size", str(args.slab_size), "--memory-size", str(args.memory_size),
           "--alias", args.alias]
    for flag, val in (("--ctrl", args.ctrl), ("--scope", args.scope), ("--device", args.device)):
        if val:
            out += [flag, val]
    if args.metadata_only:
        out.append("--metadata-only")
    return out


def _healthy(host: str, port: int, timeout: float = 1.0) -> bool:
    from .client import get_json

    try:
        return bool(get_json(f"http://{'127.0.0.1' if host in ('', '0.0.0.0') else host}:{port}", "/healthz", timeout=timeout).get("ok"))
    except Exception:
        return False


def _alive(pid: int) -> bool:
    try:
        os.kill(pid, 0)
        return True
    except OSError:
        return False


def cmd_start(args) -> int:
    err = service_mode_error(args)
    if err:
        print(f"dlslime-cache: {err}", file=sys.stderr)
        return 2
    d = runtime_dir()
    d.mkdir(parents=True, exist_ok=True)
    meta_path = d / "cache.json"
    if meta_path.exists():
        meta = json.loads(meta_path.read_text())
        if _alive(meta["pid"]):
            print(f"dlslime-cache is already running (pid {meta['pid']})")
            return 0
    log = d / "cache.log"
    with open(log, "ab") as lf:
        proc = subprocess.Popen([sys.executable, "-m", "dlslime_b200.cache.cli", "__run", *service_argv(args)], stdout=lf, stderr=lf,
                                stdin=subprocess.DEVNULL, start_new_session=True, cwd=str(Path(__file__).resolve().parents[2]))
    meta_path.write_text(json.dumps({"pid": proc.pid, "host": args.host, "port": args.port, "log": str(log), "argv": service_argv(args)}, indent=2))
    (d / "cache.pid").write_text(f"{proc.pid}\n")
    for _ in range(100):
        if _healthy(args.host, args.port):
            print(f"dlslime-cache started (pid {proc.pid}) on http://{args.host}:{args.port}, log {log}")
            return 0
        if proc.poll() is not None:
            break
        time.sleep(0.1)
    print(f"dlslime-cache did not become healthy; see {log}", file=sys.stderr)
    return 1


def cmd_status(_args) -> int:
    meta_path = runtime_dir() / "cache.json"
    if not meta_path.exists():
        print(f"dlslime-cache: not running (no metadata in {runtime_dir()})")
        return 1
    meta = json.loads(meta_path.read_text())
    alive = _alive(meta["pid"])
    ok = alive and _healthy(meta["host"], meta["port"])
    print(f"dlslime-cache: pid {meta['pid']} {'alive' if alive else 'dead'}, http://{meta['host']}:{meta['port']} {'healthy' if ok else 'unreachable'}")
    return 0 if ok else 1


def cmd_stop(args) -> int:
    d = runtime_dir()
    meta_path = d / "cache.json"
    if not meta_path.exists():
        print("dlslime-cache: not running")
        return 0
    meta = json.loads(meta_path.read_text())
    try:
        os.kill(meta["pid"], signal.SIGKILL if args.force else signal.SIGTERM)
        for _ in range(50):
            if not _alive(meta["pid"]):
                break
            time.sleep(0.1)
        print(f"dlslime-cache: stopped pid {meta['pid']}")
    except OSError:
        print(f"dlslime-cache: pid {meta['pid']} is already gone")
    for name in ("cache.json", "cache.pid"):
        (d / name).unlink(missing_ok=True)
    return 0


def cmd_run(args) -> int:
    from .service import CacheServer

    err = service_mode_error(args)
    if err:
        print(f"dlslime-cache: {err}", file=sys.stderr)
        return 2
    srv = CacheServer(args.ctrl, host=args.host, port=args.port, slab_size=args.slab_size, memory_size=args.memory_size,
                      scope=args.scope, alias=args.alias, device=args.device, metadata_only=args.metadata_only)
    stop = {"flag": False}
    signal.signal(signal.SIGTERM, lambda *_: stop.update(flag=True))
    signal.signal(signal.SIGINT, lambda *_: stop.update(flag=True))
    print(f"dlslime-cache serving on {srv.url}", flush=True)
    while not stop["flag"]:
        time.sleep(0.2)
    srv.stop()
    return 0


def main(argv=None) -> int:
    args = parse_args(argv)
    return {"start": cmd_start, "status": cmd_status, "stop": cmd_stop, "__run": cmd_run}[args.command](args)


if __name__ == "__main__":
    sys.exit(main())
