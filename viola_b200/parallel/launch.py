"""``python -m viola_b200 launch --config cfg.yaml script.py [args...]``.

Starts ``num_processes`` ranks (one per GPU) of ``script.py`` on this node through
``torch.distributed.run`` and exports the configuration path as ``$VIOLA_CONFIG`` so that
``violaEngine()`` finds it.  Mirrors the reference launcher (viola/distributed/launch.py:12-24);
the rendezvous is pinned to 127.0.0.1 because container hostnames do not always resolve.
"""

from __future__ import annotations

import argparse
import os
import subprocess
import sys
from pathlib import Path

from .config import read_config


def build_command(config_path, script, script_args, *, python=sys.executable):
    config = read_config(config_path)
    return [python, "-m", "torch.distributed.run", "--standalone", "--local-addr", "127.0.0.1",
            f"--nproc-per-node={config['num_processes']}", script, *script_args]


def main(argv=None):
    parser = argparse.ArgumentParser(prog="viola_b200")
    parser.add_argument("command", choices=("launch",))
    parser.add_argument("--config", required=True)
    parser.add_argument("script")
    parser.add_argument("script_args", nargs=argparse.REMAINDER)
    args = parser.parse_args(argv)
    path = str(Path(args.config).resolve())
    command = build_command(path, args.script, args.script_args)
    raise SystemExit(subprocess.call(command, env=dict(os.environ, VIOLA_CONFIG=path)))


if __name__ == "__main__":
    main()
