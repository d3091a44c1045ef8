"""Python-as-config: record library calls in config files, edit the tree, build it later.

Drop-in surface for the config package the reference depends on (`field`, `call`,
`config_fn`, `instantiate`, `select`, `patch_fn`, `tag`, `function`, `external`, `Config`,
`MainConfig`, `Instance`, `load_config`, `load_arg_config`, `summarize`, `deserialize`, ...).
"""

from .build import PatchBuilder, Selection, apply_patches, instantiate, patch, patch_fn, select, summarize
from .loader import apply_overrides, deserialize, load_arg_config, load_config, load_module
from .node import (Field, L, Lazy, Ref, annotate, call, config_fn, exempt, external, field, function,
                   lazy_partial, locate, normalize, tag, to_plain)
from .schema import Config, Instance, MainConfig

__all__ = [
    "Config", "Field", "Instance", "L", "Lazy", "MainConfig", "PatchBuilder", "Ref", "Selection",
    "annotate", "apply_overrides", "apply_patches", "call", "config_fn", "deserialize", "exempt",
    "external", "field", "function", "instantiate", "lazy_partial", "load_arg_config",
    "load_config", "load_module", "locate", "normalize", "patch", "patch_fn", "select",
    "summarize", "tag", "to_plain",
]
