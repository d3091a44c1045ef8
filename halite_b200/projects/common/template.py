"""Prompt templating (reference: projects/common/template.py).

`get_render_fn(template)` compiles a jinja2 template (strict about undefined names, blocks
trimmed) into a callable taking either one mapping or keyword arguments; `simple_format(template)`
wraps `str.format`. Without jinja2 a minimal `{{ name }}` substitution stands in.
"""

from __future__ import annotations

import re
from typing import Callable


class Template:
    def __init__(self, template):
        self.template = template

    def __call__(self, *args, **kwargs):
        return self.template.render(*args, **kwargs)


class _FallbackTemplate:
    _VAR = re.compile(r"\{\{\s*([A-Za-z_][A-Za-z0-9_]*)\s*\}\}")

    def __init__(self, text):
        self.text = text

    def render(self, *args, **kwargs):
        ctx = dict(*args, **kwargs)
        return self._VAR.sub(lambda m: str(ctx[m.group(1)]), self.text)


def get_render_fn(template: str, trim_blocks: bool = True, lstrip_blocks: bool = True,
                  keep_trailing_newline: bool = True, filters: dict[str, Callable] | None = None):
    try:
        from jinja2 import Environment, StrictUndefined
    except ImportError:
        return Template(_FallbackTemplate(template))
    env = Environment(trim_blocks=trim_blocks, lstrip_blocks=lstrip_blocks,
                      keep_trailing_newline=keep_trailing_newline, undefined=StrictUndefined)
    for name, fn in (filters or {}).items():
        env.filters[name] = fn
    return Template(env.from_string(template))


class SimpleFormat:
    def __init__(self, template: str):
        self.template = template

    def __call__(self, *args, **kwargs):
        return self.template.format(*args, **kwargs)


def simple_format(template: str) -> SimpleFormat:
    return SimpleFormat(template)
