"""Nemotron-CC, the `medium-low` quality tier alone (reference: configs/data/nemotron_cc_medium_low.py, whose shard
table is site data; here it comes from the `shards.json` index read by `nemotron_cc.py`)."""

from .nemotron_cc import medium_low as conf
