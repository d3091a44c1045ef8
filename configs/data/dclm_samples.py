"""Shard specification of a DCLM-baseline sample converted to record files (20 shards). Point
`root` at the converted copy and regenerate the counts with scripts/tools/gather_dataset.py."""

from halite_b200.conf import field

_COUNTS = [4223649, 4313832, 4329181, 4245980, 4275956, 4275462, 4146856, 4166429, 4217758, 4212483,
           4217677, 4195569, 4230000, 4230000, 4230000, 4230000, 4230000, 4230000, 4230000, 4230000]
_NAME = "dclm-baseline-1.0"

conf = field(root="/data/halite/", ratios={_NAME: 1.0},
             shards={_NAME: {f"data-{i + 1:02d}-of-20.hbrec": n for i, n in enumerate(_COUNTS)}})
