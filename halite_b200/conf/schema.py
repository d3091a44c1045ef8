"""pydantic bases for experiment schemas: `Config`, `MainConfig`, and the `Instance` field type
that holds an un-instantiated object config (a recorded call).

Matches how the reference declares its schemas (projects/common/config.py:51-96,
projects/lm/config.py:7-11): `model: Instance | None = None` fields, `MainConfig` roots that
also carry free-form `hparams`.
"""

from __future__ import annotations

from typing import Any

from pydantic import BaseModel, ConfigDict
from pydantic_core import core_schema

from .node import FN, PATCH, TARGET, Field, from_plain, normalize, to_plain


class Instance(Field):
    """A recorded call (`{"__target": ...}`), a partial, or a function reference."""

    def __init__(self, *args, **kwargs):
        super().__init__()
        for a in args:
            for k, v in dict(a).items():
                dict.__setitem__(self, k, from_plain(v) if not isinstance(v, Field) else v)
        for k, v in kwargs.items():
            dict.__setitem__(self, k, normalize(v))

    @classmethod
    def __get_pydantic_core_schema__(cls, source, handler):
        def validate(v):
            if isinstance(v, Instance):
                return v
            if isinstance(v, dict):
                if not (TARGET in v or FN in v or PATCH in v):
                    raise ValueError("an Instance must be a recorded call (has no __target / __fn)")
                return Instance(v)
            raise ValueError(f"cannot use {type(v).__name__} as an Instance")

        return core_schema.no_info_plain_validator_function(
            validate, serialization=core_schema.plain_serializer_function_ser_schema(to_plain))


class Config(BaseModel):
    model_config = ConfigDict(extra="forbid", arbitrary_types_allowed=True, protected_namespaces=(),
                              validate_assignment=False)

    def to_dict(self):
        return to_plain(self.model_dump())


class MainConfig(Config):
    model_config = ConfigDict(extra="allow", arbitrary_types_allowed=True, protected_namespaces=())

    hparams: Any = None

    def __getattr__(self, key):
        # unknown top-level sections read as None instead of raising
        try:
            return super().__getattr__(key)
        except AttributeError:
            if key.startswith("_"):
                raise
            return None
