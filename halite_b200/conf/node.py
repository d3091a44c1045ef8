"""Config tree primitives: attribute dictionaries, recorded calls, lazy imports, refs and tags.

A config file is ordinary Python. Classes and functions it imports from libraries arrive as
`Lazy` stand-ins: calling one records `{"__target": "pkg.mod.Class", **kwargs}` instead of
constructing the object. The recorded tree is plain data (dict / list / str / number), can be
edited, serialised to JSON and built later with `instantiate`.

The capabilities mirror what the reference's config files use from its external config
package (configs/models/transformer.py:55-430, configs/models/llama/llama3_2_3b.py:14-57,
configs/lm/farseer.py:45,126-142 in the reference tree).
"""

from __future__ import annotations

import copy
import enum
import functools
import importlib
import inspect
import operator
from typing import Any, Callable

TARGET = "__target"
ARGS = "__args"
PARTIAL = "__partial"
FN = "__fn"
TAG = "__tag"
TUPLE = "__tuple"
PATCH = "__patch"
META = "__meta"
FILE = "__file"

_SPECIAL = (TARGET, ARGS, PARTIAL, FN, TAG, TUPLE, PATCH, META, FILE)


class Field(dict):
    """Dictionary with attribute access; the node type of every config tree."""

    def __getattr__(self, key):
        if key == "ref":
            return Ref(self, ())
        try:
            return self[key]
        except KeyError as e:
            raise AttributeError(key) from e

    def __getitem__(self, key):
        if isinstance(key, int) and not isinstance(key, bool) and key not in self.keys():
            return dict.__getitem__(self, ARGS)[key]  # positional argument of a recorded call
        return dict.__getitem__(self, key)

    def __setattr__(self, key, value):
        self[key] = normalize(value)

    def __delattr__(self, key):
        try:
            del self[key]
        except KeyError as e:
            raise AttributeError(key) from e

    def __setitem__(self, key, value):
        super().__setitem__(key, normalize(value))

    def __deepcopy__(self, memo):
        out = type(self)()
        memo[id(self)] = out
        for k, v in self.items():
            dict.__setitem__(out, k, copy.deepcopy(v, memo))
        return out

    def to_dict(self):
        return to_plain(self)

    def update_dict(self, values):
        for k, v in values.items():
            self[k] = v
        return self


def field(*args, **kwargs) -> Field:
    out = Field()
    for a in args:
        for k, v in dict(a).items():
            out[k] = v
    for k, v in kwargs.items():
        out[k] = v
    return out


class Annotated:
    """A positional argument that carries its parameter name (`annotate("layer_id", 3)`)."""

    def __init__(self, name, value):
        self.name = name
        self.value = value


def annotate(name, value):
    return Annotated(name, value)


def tag(name) -> Field:
    """Placeholder filled by `instantiate(conf, _tags_={name: value})`."""
    return Field({TAG: name})


# ----------------------------------------------------------------------------- paths

def object_path(obj) -> str:
    if isinstance(obj, Lazy):
        return obj._hb_path
    mod = getattr(obj, "__module__", None)
    qual = getattr(obj, "__qualname__", None) or getattr(obj, "__name__", None)
    if mod is None or qual is None:
        raise TypeError(f"cannot name {obj!r} in a config")
    return f"{mod}.{qual}"


_locators: list[Callable[[str], Any]] = []


def register_locator(fn):
    """Extra resolver tried before importlib (the loader registers config-file modules)."""
    _locators.append(fn)


def locate(path: str):
    """Resolve 'pkg.mod.Class.attr' to the object."""
    for loc in _locators:
        found = loc(path)
        if found is not None:
            return found
    parts = path.split(".")
    for i in range(len(parts), 0, -1):
        try:
            obj = importlib.import_module(".".join(parts[:i]))
        except ImportError:
            continue
        try:
            for p in parts[i:]:
                obj = getattr(obj, p)
        except AttributeError:
            continue
        return obj
    raise ImportError(f"cannot locate {path!r}")


# ----------------------------------------------------------------------------- lazy objects

_PLAIN = (str, bytes, int, float, bool, type(None), complex)


class Lazy:
    """Stand-in for an imported library object inside a config file."""

    __slots__ = ("_hb_obj", "_hb_path")

    def __init__(self, obj, path):
        object.__setattr__(self, "_hb_obj", obj)
        object.__setattr__(self, "_hb_path", path)

    def __call__(self, *args, **kwargs):
        return record_call(self._hb_obj, self._hb_path, args, kwargs)

    def __getattr__(self, name):
        val = getattr(self._hb_obj, name)
        return wrap_lazy(val, f"{self._hb_path}.{name}")

    def __getitem__(self, item):
        # typing-style subscripts (Class[int]) keep the same target
        return self

    def __repr__(self):
        return f"Lazy({self._hb_path})"

    def __eq__(self, other):
        if isinstance(other, Lazy):
            return self._hb_path == other._hb_path
        return self._hb_obj is other

    def __hash__(self):
        return hash(self._hb_path)


def wrap_lazy(val, path):
    if isinstance(val, _PLAIN) or isinstance(val, (Field, Lazy, Ref)):
        return val
    if isinstance(val, enum.Enum):
        return Field({FN: f"{object_path(type(val))}.{val.name}"})
    if getattr(val, "__hb_exempt__", False) or getattr(val, "__hb_config_fn__", False):
        return val
    if isinstance(val, (list, tuple, dict, set)):
        return val
    return Lazy(val, canonical_path(val, path))


_canon_cache: dict = {}


def canonical_path(val, fallback: str) -> str:
    """Name classes and functions by their defining module when that name resolves back to
    the same object, so `nn.Linear` and `from torch.nn import Linear` record the same target."""
    if not (isinstance(val, type) or inspect.isfunction(val) or inspect.isbuiltin(val)):
        return fallback
    key = id(val)
    hit = _canon_cache.get(key)
    if hit is not None and hit[0] is val:
        return hit[1]
    path = fallback
    try:
        real = object_path(val)
        if real != fallback and "<locals>" not in real and _try_locate(real) is val:
            path = real
    except TypeError:
        pass
    _canon_cache[key] = (val, path)
    return path


def unwrap(obj):
    return obj._hb_obj if isinstance(obj, Lazy) else obj


def record_call(obj, path, args, kwargs, partial=False) -> Field:
    """Record `obj(*args, **kwargs)` as a node, binding positionals to parameter names."""
    node = Field()
    dict.__setitem__(node, TARGET, path)
    if partial:
        dict.__setitem__(node, PARTIAL, True)
    args = list(args)
    named = {}
    # annotated positionals become keywords
    rest = []
    for a in args:
        if isinstance(a, Annotated):
            named[a.name] = a.value
        else:
            rest.append(a)
    args = rest
    leftover = []
    if args:
        names = None if partial else _positional_names(obj)
        if names is None:
            # partials keep positionals positional (they prefix the later call); so do
            # callables whose signature is unknown or takes *args
            leftover = args
        else:
            taken = set(named) | set(kwargs)
            free = [n for n in names if n not in taken]
            for n, a in zip(free, args):
                named[n] = a
            leftover = args[len(free):]
    if leftover:
        dict.__setitem__(node, ARGS, [normalize(a) for a in leftover])
    for k, v in {**named, **kwargs}.items():
        node[k] = v
    src = getattr(obj, "__hb_file__", None)      # defined inside a config file: remember where
    if src:
        dict.__setitem__(node, FILE, src)
    return node


def _positional_names(obj):
    try:
        sig = inspect.signature(obj)
    except (TypeError, ValueError):
        return None
    names, varargs = [], False
    for p in sig.parameters.values():
        if p.kind in (p.POSITIONAL_ONLY,):
            return None
        if p.kind == p.POSITIONAL_OR_KEYWORD:
            names.append(p.name)
        elif p.kind == p.VAR_POSITIONAL:
            varargs = True
    if varargs:
        # positionals after the named ones would land in *args: keep everything positional
        return None
    return names


def lazy_partial(fn, *args, **kwargs) -> Field:
    """`functools.partial` inside a config file: recorded, built into a real partial later."""
    if isinstance(fn, Field):
        if fn.get(PARTIAL):
            node = copy.deepcopy(fn)
            if args:
                dict.__setitem__(node, ARGS, list(node.get(ARGS, [])) + [normalize(a) for a in args])
            for k, v in kwargs.items():
                node[k] = v
            return node
        if FN in fn:
            path = fn[FN]
            node = record_call(_try_locate(path), path, args, kwargs, partial=True)
            if FILE in fn:
                dict.__setitem__(node, FILE, fn[FILE])
            return node
        raise TypeError("partial() of a config node that is not callable")
    obj = unwrap(fn)
    node = record_call(obj, object_path(fn), args, kwargs, partial=True)
    src = getattr(obj, "__hb_file__", None)
    if src:
        dict.__setitem__(node, FILE, src)
    return node


def _try_locate(path):
    try:
        return locate(path)
    except ImportError:
        return None


class _Subscript:
    def __init__(self, fn):
        self._fn = fn

    def __getitem__(self, obj):
        return functools.partial(self._fn, obj)


def _call_now(obj, *args, **kwargs):
    return unwrap(obj)(*args, **kwargs)


def _external(obj, *args, **kwargs):
    return record_call(unwrap(obj), object_path(obj), args, kwargs)


#: `call[fn](...)` runs fn at config time (a config function, `int`, ...).
call = _Subscript(_call_now)
#: `external[Cls](...)` records a call to an object that was imported for real.
external = _Subscript(_external)
L = external


def function(fn) -> Field:
    """Reference to the callable itself (not a call)."""
    obj = unwrap(fn)
    node = Field({FN: object_path(fn)})
    src = getattr(obj, "__hb_file__", None)
    if src:
        dict.__setitem__(node, FILE, src)
    return node


def config_fn(fn):
    """Function whose body runs while the config is written; library calls inside it record."""
    fn.__hb_config_fn__ = True
    return fn


def exempt(fn):
    """Library function that config files call for real (e.g. `load_model(path)`)."""
    fn.__hb_exempt__ = True
    return fn


# ----------------------------------------------------------------------------- refs

class Ref:
    """Deferred lookup `conf.hparams.ref.lr`, usable in arithmetic; resolved by `resolve_refs`."""

    def __init__(self, root, path, expr=None):
        object.__setattr__(self, "_root", root)
        object.__setattr__(self, "_path", tuple(path))
        object.__setattr__(self, "_expr", expr)

    def __getattr__(self, key):
        if key.startswith("_"):
            raise AttributeError(key)
        return Ref(self._root, self._path + (key,))

    def __getitem__(self, key):
        return Ref(self._root, self._path + (key,))

    def _value(self):
        if self._expr is not None:
            op, operands = self._expr
            vals = [o._value() if isinstance(o, Ref) else o for o in operands]
            return op(*vals)
        cur = self._root
        for p in self._path:
            cur = cur[p]
        if isinstance(cur, Ref):
            cur = cur._value()
        return cur

    def _bin(self, other, op, swap=False):
        ops = (other, self) if swap else (self, other)
        return Ref(None, (), (op, ops))

    def __add__(self, o): return self._bin(o, operator.add)
    def __radd__(self, o): return self._bin(o, operator.add, True)
    def __sub__(self, o): return self._bin(o, operator.sub)
    def __rsub__(self, o): return self._bin(o, operator.sub, True)
    def __mul__(self, o): return self._bin(o, operator.mul)
    def __rmul__(self, o): return self._bin(o, operator.mul, True)
    def __truediv__(self, o): return self._bin(o, operator.truediv)
    def __rtruediv__(self, o): return self._bin(o, operator.truediv, True)
    def __floordiv__(self, o): return self._bin(o, operator.floordiv)
    def __rfloordiv__(self, o): return self._bin(o, operator.floordiv, True)
    def __pow__(self, o): return self._bin(o, operator.pow)
    def __rpow__(self, o): return self._bin(o, operator.pow, True)
    def __mod__(self, o): return self._bin(o, operator.mod)
    def __neg__(self): return Ref(None, (), (operator.neg, (self,)))


def resolve_refs(node):
    """Replace every Ref in the tree by its current value (in place); returns the tree."""
    if isinstance(node, Ref):
        return resolve_refs(node._value())
    if isinstance(node, dict):
        for k in list(node.keys()):
            dict.__setitem__(node, k, resolve_refs(node[k]))
        return node
    if isinstance(node, list):
        for i, v in enumerate(node):
            node[i] = resolve_refs(v)
        return node
    if isinstance(node, tuple):
        return tuple(resolve_refs(v) for v in node)
    return node


# ----------------------------------------------------------------------------- normalisation

def normalize(value):
    """Turn a value written in a config file into tree data."""
    if isinstance(value, (Field, Ref)) or isinstance(value, _PLAIN):
        return value
    if isinstance(value, Lazy):
        node = Field()
        dict.__setitem__(node, FN, value._hb_path)
        return node
    if isinstance(value, Annotated):
        return normalize(value.value)
    if isinstance(value, enum.Enum):
        return Field({FN: f"{object_path(type(value))}.{value.name}"})
    if isinstance(value, dict):
        out = Field()
        for k, v in value.items():
            dict.__setitem__(out, k, normalize(v))
        return out
    if isinstance(value, list):
        return [normalize(v) for v in value]
    if isinstance(value, tuple):
        return tuple(normalize(v) for v in value)
    if isinstance(value, functools.partial):
        return lazy_partial(value.func, *value.args, **value.keywords)
    if hasattr(value, "model_dump") and hasattr(value, "model_fields"):
        return value  # pydantic objects pass through
    if callable(value) and hasattr(value, "__qualname__") and "<lambda>" not in value.__qualname__ \
            and "<locals>" not in value.__qualname__:
        return function(value)
    return value


def to_plain(node):
    """JSON-ready copy of a tree (tuples are tagged so they survive the round trip)."""
    if isinstance(node, Ref):
        return to_plain(node._value())
    if isinstance(node, dict):
        return {str(k): to_plain(v) for k, v in node.items()}
    if isinstance(node, tuple):
        return {TUPLE: [to_plain(v) for v in node]}
    if isinstance(node, list):
        return [to_plain(v) for v in node]
    if isinstance(node, _PLAIN):
        return node
    if hasattr(node, "model_dump"):
        return to_plain(node.model_dump())
    if isinstance(node, Lazy):
        return {FN: node._hb_path}
    try:
        import torch

        if isinstance(node, torch.dtype):
            return str(node).replace("torch.", "")
    except ImportError:  # pragma: no cover
        pass
    return repr(node)


def from_plain(data):
    """Inverse of `to_plain`: dicts become Fields, tagged tuples become tuples."""
    if isinstance(data, dict):
        if set(data.keys()) == {TUPLE}:
            return tuple(from_plain(v) for v in data[TUPLE])
        out = Field()
        for k, v in data.items():
            dict.__setitem__(out, k, from_plain(v))
        return out
    if isinstance(data, list):
        return [from_plain(v) for v in data]
    return data


def is_target(node) -> bool:
    return isinstance(node, dict) and (TARGET in node or FN in node)


def public_items(node):
    return [(k, v) for k, v in node.items() if k not in _SPECIAL]
