"""The 200B-token Nemotron-CC sample as one source named `nemotron-cc` (reference:
configs/data/nemotron_cc_200b.py, whose shard table is site data). The record counts come from
`<root>/shards.json`, written by `scripts/tools/gather_dataset.py`; the root is taken from
`HB_NEMOTRON_CC_200B_ROOT` (the folder that holds the `nemotron-cc` directory)."""

import json
import os

from halite_b200.conf import field

root = os.environ.get("HB_NEMOTRON_CC_200B_ROOT", "/data")


def _index():
    path = os.path.join(root, "shards.json")
    if not os.path.exists(path):
        return {}
    with open(path) as f:
        data = json.load(f)
    return data.get("shards", data)


conf = field(root=root, ratios={"nemotron-cc": 1.0}, shards={"nemotron-cc": dict(_index().get("nemotron-cc", {}))})
