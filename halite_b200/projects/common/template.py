"""Prompt templating (reference: projects/common/template.py): jinja templates when jinja2 is
importable, `str.format`-style `{{ name }}` substitution otherwise."""

from __future__ import annotations

import re


def simple_format(template, record):
    def sub(m):
        return str(record[m.group(1)])

    return re.sub(r"\{\{\s*([A-Za-z_][A-Za-z0-9_]*)\s*\}\}", sub, template)


def get_render_fn(template):
    try:
        import jinja2

        compiled = jinja2.Environment().from_string(template)
        return lambda record: compiled.render(**record)
    except ImportError:
        return lambda record: simple_format(template, record)
