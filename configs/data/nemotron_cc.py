"""Nemotron-CC split into five quality tiers (reference: configs/data/nemotron_cc_{high,
medium_high,medium,medium_low,low,200b}.py, one shard table per tier).

The per-shard record counts are site data: `scripts/tools/gather_dataset.py <root> --out
<root>/shards.json` writes them next to the converted copy and this file reads them from there,
so the tier specs follow whatever conversion is on disk. Without that index the tiers are
empty and building a dataset from them reports the missing file.
"""

import json
import os

from halite_b200.conf import field

root = os.environ.get("HB_NEMOTRON_CC_ROOT", "/data/nemotron-cc")
TIERS = ("high", "medium-high", "medium", "medium-low", "low")


def _index():
    path = os.path.join(root, "shards.json")
    if not os.path.exists(path):
        return {}
    with open(path) as f:
        data = json.load(f)
    return data.get("shards", data)


_shards = _index()


def tier(name):
    """Spec of one tier alone."""
    return field(root=root, ratios={name: 1.0}, shards={name: dict(_shards.get(name, {}))})


def mixture(ratios):
    """Spec that samples the tiers with the given ratios (`{"high": 0.2, ...}`)."""
    return field(root=root, ratios=ratios, shards={name: dict(_shards.get(name, {})) for name in ratios})


high, medium_high, medium, medium_low, low = (tier(t) for t in TIERS)
uniform = mixture({t: 0.2 for t in TIERS})
conf = uniform
