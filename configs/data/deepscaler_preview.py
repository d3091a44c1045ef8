"""Shard specification of the DeepScaleR preview problems (40,315 prompts with reference answers)
converted to one record file. Point `root` at the converted copy."""

from halite_b200.conf import field

_NAME = "agentica-org_DeepScaleR-Preview-Dataset"
conf = field(root="/data/halite/", ratios={_NAME: 1.0}, shards={_NAME: {"train-1-of-1.hbrec": 40315}})
