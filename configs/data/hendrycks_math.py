"""Shard specification of the Hendrycks MATH dataset converted to record files
(`root/<dataset>/<shard>`: number of records). Point `root` at the converted copy."""

from halite_b200.conf import field

_SUBJECTS = {"algebra": (1744, 1187), "counting_and_probability": (771, 474), "geometry": (870, 479),
             "intermediate_algebra": (1295, 903), "number_theory": (869, 540), "prealgebra": (1205, 871),
             "precalculus": (746, 546)}
_NAME = "EleutherAI_hendrycks_math"
root = "/data/halite/"

train = field(root=root, ratios={_NAME: 1.0},
              shards={_NAME: {f"{s}-train-1-of-1.bag": n for s, (n, _) in _SUBJECTS.items()}})
test = field(root=root, ratios={_NAME: 1.0},
             shards={_NAME: {f"{s}-test-1-of-1.bag": n for s, (_, n) in _SUBJECTS.items()}})
conf = field(train=train, test=test)
