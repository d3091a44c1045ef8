"""Nemotron-CC, the `medium-high` quality tier alone (reference: configs/data/nemotron_cc_medium_high.py, whose shard
table is site data; here it comes from the `shards.json` index read by `nemotron_cc.py`)."""

from .nemotron_cc import medium_high as conf
