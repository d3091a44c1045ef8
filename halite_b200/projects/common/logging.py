"""Run naming from hyper-parameters (reference: projects/common/logging.py:1-2).

An experiment config puts `partial(hparam_to_name, format="...")` under `conf.output.name`; the
training entry points call it with `conf.hparams` once references are resolved.
"""

from __future__ import annotations


def hparam_to_name(hparams: dict, format: str) -> str:
    return format.format(**hparams)
