"""Reference arm of bench.py: runs the unmodified reference package installed under
`baseline/_ref` through its own public API for the same metric and config."""

from __future__ import annotations

import json


def run(args):
    print(json.dumps({"impl": "reference", "unavailable": "reference arm not wired yet"}), flush=True)
