"""Loading config files: Python source whose library imports arrive as lazy stand-ins.

The source is parsed, every `import` / `from ... import` statement is rewritten into a call
of the loader's import function, and the result is executed as a module. Rules:

* relative imports and absolute imports that resolve inside the config root load other
  config files the same way (their functions and `conf` objects are real);
* this package (also under the alias `slickconf`) is imported for real;
* standard-library modules are real, except `functools.partial`, which records;
* everything else (torch, the framework's classes) becomes `Lazy`, unless marked `@exempt`
  or `@config_fn`.

The CLI surface follows the reference's scripts (scripts/lm.py:278 `load_arg_config(Schema)`,
scripts/tools/convert_checkpoint.py:38 `load_config(path, config_name=...)`).
"""

from __future__ import annotations

import ast
import importlib
import json
import os
import sys
import types

from . import node as _node
from .node import Field, Lazy, from_plain, lazy_partial, normalize, resolve_refs, wrap_lazy

_CONF_ALIASES = ("slickconf", "halite_b200.conf")
_modules: dict[str, types.ModuleType] = {}
_roots: list[str] = []


def _stdlib(name: str) -> bool:
    return name.split(".")[0] in sys.stdlib_module_names


def _config_root(path: str) -> str:
    """Nearest ancestor directory called `configs`; the file's own directory when there is none."""
    d = os.path.dirname(os.path.abspath(path))
    cur = d
    while True:
        if os.path.basename(cur) == "configs":
            return cur
        parent = os.path.dirname(cur)
        if parent == cur:
            return d
        cur = parent


def _module_name(path: str, root: str) -> str:
    rel = os.path.relpath(os.path.abspath(path), os.path.dirname(root))
    rel = rel[:-3] if rel.endswith(".py") else rel
    parts = [p for p in rel.split(os.sep) if p not in ("", ".")]
    if parts and parts[-1] == "__init__":
        parts = parts[:-1]
    return "_hbconf_." + ".".join(parts)


class _ImportRewriter(ast.NodeTransformer):
    def visit_Import(self, node):
        out = []
        for alias in node.names:
            target = alias.asname or alias.name.split(".")[0]
            call = ast.Call(
                func=ast.Name(id="__hb_import__", ctx=ast.Load()),
                args=[ast.Constant(alias.name), ast.Constant(None), ast.Constant(0),
                      ast.Constant(alias.asname is not None)],
                keywords=[])
            out.append(ast.Assign(targets=[ast.Name(id=target, ctx=ast.Store())], value=call))
        return [ast.copy_location(o, node) for o in out]

    def visit_ImportFrom(self, node):
        out = []
        for alias in node.names:
            if alias.name == "*":
                raise SyntaxError("config files cannot use `from x import *`")
            target = alias.asname or alias.name
            call = ast.Call(
                func=ast.Name(id="__hb_import__", ctx=ast.Load()),
                args=[ast.Constant(node.module), ast.Constant(alias.name), ast.Constant(node.level),
                      ast.Constant(True)],
                keywords=[])
            out.append(ast.Assign(targets=[ast.Name(id=target, ctx=ast.Store())], value=call))
        return [ast.copy_location(o, node) for o in out]


def _find_config_file(modname: str, roots) -> str | None:
    rel = modname.replace(".", os.sep)
    for root in roots:
        for base in (os.path.dirname(root), root):
            for cand in (os.path.join(base, rel + ".py"), os.path.join(base, rel, "__init__.py")):
                if os.path.exists(cand) and os.path.abspath(cand).startswith(os.path.abspath(root)):
                    return cand
    return None


def _make_importer(file: str, root: str):
    here = os.path.dirname(os.path.abspath(file))

    def importer(module, name, level, bind_leaf):
        # ---- relative: another config file
        if level > 0:
            base = here
            for _ in range(level - 1):
                base = os.path.dirname(base)
            target_dir = os.path.join(base, *(module.split(".") if module else []))
            cand_mod = target_dir + ".py"
            if name is not None and os.path.exists(os.path.join(target_dir, name + ".py")):
                return load_module(os.path.join(target_dir, name + ".py"), root)
            if name is not None and os.path.isdir(os.path.join(target_dir, name)):
                return _namespace(os.path.join(target_dir, name), root)
            if os.path.exists(cand_mod):
                mod = load_module(cand_mod, root)
            elif os.path.exists(os.path.join(target_dir, "__init__.py")):
                mod = load_module(os.path.join(target_dir, "__init__.py"), root)
            elif os.path.isdir(target_dir):
                mod = _namespace(target_dir, root)
            else:
                raise ImportError(f"config import {'.' * level}{module or ''} not found from {file}")
            return mod if name is None else getattr(mod, name)
        # ---- this package (and its slickconf alias): real
        for alias in _CONF_ALIASES:
            if module == alias or module.startswith(alias + "."):
                real = "halite_b200.conf" + module[len(alias):]
                mod = importlib.import_module(real)
                return mod if name is None else getattr(mod, name)
        # ---- absolute import of a config file under the root
        cfg = _find_config_file(module if name is None else module, [root] + _roots)
        if cfg is not None:
            mod = load_module(cfg, root)
            if name is None:
                return mod
            if hasattr(mod, name):
                return getattr(mod, name)
        if name is not None:
            cfg = _find_config_file(f"{module}.{name}", [root] + _roots)
            if cfg is not None:
                return load_module(cfg, root)
        # ---- standard library: real, except functools.partial
        if _stdlib(module):
            mod = importlib.import_module(module)
            if name is None:
                return mod if bind_leaf else importlib.import_module(module.split(".")[0])
            if module == "functools" and name == "partial":
                return lazy_partial
            return getattr(mod, name)
        # ---- libraries: lazy
        mod = importlib.import_module(module)
        if name is None:
            top = mod if bind_leaf else importlib.import_module(module.split(".")[0])
            return Lazy(top, top.__name__)
        try:
            val = getattr(mod, name)
        except AttributeError:
            val = importlib.import_module(f"{module}.{name}")
        path = f"{module}.{name}"
        return wrap_lazy(val, path)

    return importer


def _namespace(directory: str, root: str):
    return _LazyDir(directory, root)


class _LazyDir:
    def __init__(self, directory, root):
        self._d = directory
        self._root = root

    def __getattr__(self, name):
        cand = os.path.join(self._d, name + ".py")
        if os.path.exists(cand):
            return load_module(cand, self._root)
        if os.path.isdir(os.path.join(self._d, name)):
            return _LazyDir(os.path.join(self._d, name), self._root)
        raise AttributeError(name)


def load_module(path: str, root: str | None = None) -> types.ModuleType:
    """Execute a config file (once per path) and return its module object."""
    path = os.path.abspath(path)
    if path in _modules:
        return _modules[path]
    if root is None:
        root = _config_root(path)
    if root not in _roots:
        _roots.append(root)
    with open(path) as f:
        source = f.read()
    tree = ast.parse(source, filename=path)
    tree = _ImportRewriter().visit(tree)
    ast.fix_missing_locations(tree)
    code = compile(tree, path, "exec")
    name = _module_name(path, root)
    mod = types.ModuleType(name)
    mod.__file__ = path
    mod.__dict__["__hb_import__"] = _make_importer(path, root)
    _modules[path] = mod
    try:
        exec(code, mod.__dict__)
    except BaseException:
        _modules.pop(path, None)
        raise
    for k, v in list(mod.__dict__.items()):
        if isinstance(v, (types.FunctionType, type)) and getattr(v, "__module__", None) == name:
            try:
                v.__hb_file__ = path
            except (AttributeError, TypeError):
                pass
    return mod


def _locate_config_module(path: str):
    if not path.startswith("_hbconf_."):
        return None
    parts = path.split(".")
    for mod in _modules.values():
        mparts = mod.__name__.split(".")
        if parts[:len(mparts)] == mparts:
            obj = mod
            try:
                for p in parts[len(mparts):]:
                    obj = getattr(obj, p)
            except AttributeError:
                continue
            return obj
    return None


_node.register_locator(_locate_config_module)


def _parse_value(text: str):
    try:
        return json.loads(text)
    except json.JSONDecodeError:
        pass
    low = text.lower()
    if low in ("true", "false"):
        return low == "true"
    if low in ("none", "null"):
        return None
    try:
        return ast.literal_eval(text)
    except (ValueError, SyntaxError):
        return text


def apply_overrides(conf, overrides):
    """`a.b.c=value` strings (or a dict) applied to a config tree; list indices allowed."""
    if isinstance(overrides, dict):
        items = list(overrides.items())
    else:
        items = []
        for o in overrides or []:
            if "=" not in o:
                raise ValueError(f"override {o!r} is not key=value")
            k, v = o.split("=", 1)
            items.append((k.lstrip("-"), _parse_value(v)))
    for key, value in items:
        cur = conf
        parts = key.split(".")
        for p in parts[:-1]:
            if isinstance(cur, list):
                cur = cur[int(p)]
            else:
                if p not in cur:
                    cur[p] = Field()
                cur = cur[p]
        last = parts[-1]
        if isinstance(cur, list):
            cur[int(last)] = normalize(value)
        else:
            cur[last] = value
    return conf


def load_config(path: str, config_name: str | None = None, overrides=None, schema=None):
    """Load `path`; the config is the module's `conf`, or the result of calling the function
    `config_name` defined in it. Overrides apply before references resolve."""
    mod = load_module(path)
    if config_name:
        fn = getattr(mod, config_name)
        conf = fn()
    else:
        conf = getattr(mod, "conf")
    apply_overrides(conf, overrides)
    conf = resolve_refs(conf)
    if schema is not None:
        return schema(**conf)
    return conf


def load_arg_config(schema=None, args=None):
    """CLI entry: `script.py [--conf] CONF.py [config_name] [key=value ...]`."""
    args = list(sys.argv[1:] if args is None else args)
    if args and args[0] == "--conf":
        args.pop(0)
    elif args and args[0].startswith("--conf="):
        args[0] = args[0][len("--conf="):]
    if not args:
        raise SystemExit("usage: <script> [--conf] CONFIG.py [config_name] [key=value ...]")
    path = args.pop(0)
    name = None
    if args and "=" not in args[0]:
        name = args.pop(0)
    return load_config(path, config_name=name, overrides=args, schema=schema)


def deserialize(source):
    """Config tree from a JSON file path, a JSON string or an already-parsed dict."""
    if isinstance(source, (dict, list)):
        return from_plain(source)
    if os.path.exists(source):
        with open(source) as f:
            return from_plain(json.load(f))
    return from_plain(json.loads(source))
