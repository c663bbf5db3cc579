"""Option handling in the reference's manner: a value comes from the command line, else from the
environment variable ``IIAN_<FLAG>`` (upper case, dashes as underscores), else from the flat JSON
object named by ``--config``, else from the default (src/iian/cli/args.cpp:152-183, docs/cli.md:75-81).
``--no-x`` switches are plain flags.
"""
from __future__ import annotations

import argparse
import json
import os
from typing import Any, Dict, List, Optional


class Options:
    def __init__(self, prog: str, description: str):
        self.parser = argparse.ArgumentParser(prog=prog, description=description)
        self.parser.add_argument("--config", metavar="FILE", help="JSON object of flag -> value")
        self._defaults: Dict[str, Any] = {}
        self._types: Dict[str, Any] = {}
        self._group = self.parser

    def group(self, title: str) -> None:
        self._group = self.parser.add_argument_group(title)

    def positional(self, name: str, help: str, nargs=None) -> None:
        self.parser.add_argument(name, help=help, nargs=nargs)

    def add(self, flags: str, help: str, metavar: Optional[str] = None, default: Any = None, type=str) -> None:
        names = flags.split(",")
        dest = [n for n in names if n.startswith("--")][0][2:].replace("-", "_")
        self._defaults[dest] = default
        self._types[dest] = type
        shown = f"{help} (default: {default})" if default is not None else help
        self._group.add_argument(*names, dest=dest, metavar=metavar, default=None, type=type, help=shown)

    def flag(self, flags: str, help: str) -> None:
        names = flags.split(",")
        dest = [n for n in names if n.startswith("--")][0][2:].replace("-", "_")
        self._defaults[dest] = False
        self._types[dest] = bool
        self._group.add_argument(*names, dest=dest, action="store_const", const=True, default=None, help=help)

    def parse(self, argv: List[str]) -> argparse.Namespace:
        ns = self.parser.parse_args(argv)
        file_vals: Dict[str, Any] = {}
        if ns.config:
            with open(os.path.expanduser(ns.config), "r", encoding="utf-8") as f:
                raw = json.load(f)
            if not isinstance(raw, dict):
                self.parser.error(f"--config file {ns.config} must contain a JSON object of flag -> value")
            for k, v in raw.items():
                dest = k.replace("-", "_")
                if dest not in self._defaults:
                    self.parser.error(f"unknown option '{k}' in {ns.config}")
                file_vals[dest] = v
        ns.given = set()
        for dest, default in self._defaults.items():
            if getattr(ns, dest) is not None:
                ns.given.add(dest)
                continue
            env = os.environ.get("IIAN_" + dest.upper())
            if env is not None:
                val: Any = env
                ns.given.add(dest)
            elif dest in file_vals:
                val = file_vals[dest]
                ns.given.add(dest)
            else:
                val = default
            t = self._types[dest]
            if val is not None:
                if t is bool:
                    val = val if isinstance(val, bool) else str(val).lower() in ("1", "true", "yes", "on")
                else:
                    val = t(val)
            setattr(ns, dest, val)
        return ns
