"""Turning a recorded config tree into live objects, and rewriting trees (`select` / `patch`)."""

from __future__ import annotations

import copy
import functools

from .node import (ARGS, FILE, FN, META, PARTIAL, PATCH, TAG, TARGET, TUPLE, Field, Lazy, Ref,
                   is_target, locate, normalize, object_path, public_items, unwrap)


def _resolve(path, node=None):
    if node is not None and FILE in node:
        # a function or class defined inside a config file: re-load that file
        from .loader import load_module

        mod = load_module(node[FILE])
        prefix = mod.__name__ + "."
        qual = path[len(prefix):] if path.startswith(prefix) else path.rsplit(".", 1)[-1]
        obj = mod
        for p in qual.split("."):
            obj = getattr(obj, p)
        return _runtime_function(mod, unwrap(obj))
    return unwrap(locate(path))


_runtime_globals: dict = {}


def _runtime_function(mod, fn):
    """A plain function or class defined in a config file sees library imports as recording
    stand-ins. When it is used at run time (a hook named with `function(...)`, a reward class
    built with `external[...]`), re-bind its code to a copy of the module's globals in which the
    stand-ins are the real objects, so `torch.cat(...)` inside it computes instead of
    recording."""
    import types

    is_fn = isinstance(fn, types.FunctionType) and not getattr(fn, "__hb_config_fn__", False)
    is_cls = isinstance(fn, type) and getattr(fn, "__module__", None) == mod.__name__
    if not (is_fn or is_cls):
        return fn
    key = id(mod)
    if key not in _runtime_globals:
        real = {}
        for k, v in mod.__dict__.items():
            real[k] = unwrap(v) if isinstance(v, Lazy) else v
        lazy_import = mod.__dict__.get("__hb_import__")
        if lazy_import is not None:
            # imports written inside function bodies must also yield real objects at run time
            real["__hb_import__"] = lambda *a: unwrap(lazy_import(*a))

        def rebind(f):
            g = types.FunctionType(f.__code__, real, f.__name__, f.__defaults__, f.__closure__)
            g.__kwdefaults__ = f.__kwdefaults__
            g.__qualname__ = f.__qualname__
            g.__doc__ = f.__doc__
            return g

        for k, v in list(real.items()):
            if isinstance(v, types.FunctionType) and v.__globals__ is mod.__dict__ and \
                    not getattr(v, "__hb_config_fn__", False):
                real[k] = rebind(v)
            elif isinstance(v, type) and getattr(v, "__module__", None) == mod.__name__:
                body = {}
                for name, attr in vars(v).items():
                    if name in ("__dict__", "__weakref__"):
                        continue
                    if isinstance(attr, types.FunctionType) and attr.__globals__ is mod.__dict__:
                        attr = rebind(attr)
                    elif isinstance(attr, (staticmethod, classmethod)) and \
                            getattr(attr.__func__, "__globals__", None) is mod.__dict__:
                        attr = type(attr)(rebind(attr.__func__))
                    body[name] = attr
                real[k] = type(v)(v.__name__, v.__bases__, body)
        _runtime_globals[key] = real
    return _runtime_globals[key].get(fn.__name__, fn)


def instantiate(node, *args, _tags_: dict | None = None, **kwargs):
    """Build the object(s) a config tree describes.

    Nodes with `__target` are called with their instantiated arguments; partial nodes become
    `functools.partial`; `__fn` nodes become the callable itself; `tag(name)` placeholders take
    their value from `_tags_`. Extra positional / keyword arguments are passed to the root call.
    """
    tags = _tags_ or {}
    return _build(node, tags, args, kwargs, root=True)


def _build(node, tags, extra_args=(), extra_kwargs=None, root=False):
    extra_kwargs = extra_kwargs or {}
    if isinstance(node, Ref):
        return _build(node._value(), tags)
    if isinstance(node, Lazy):
        return node._hb_obj
    if hasattr(node, "model_dump") and hasattr(type(node), "model_fields") and not isinstance(node, dict):
        return node
    if isinstance(node, dict):
        if TAG in node:
            name = node[TAG]
            if name not in tags:
                raise KeyError(f"config tag {name!r} was not supplied to instantiate(_tags_=...)")
            return tags[name]
        if TUPLE in node and len(node) == 1:
            return tuple(_build(v, tags) for v in node[TUPLE])
        if FN in node:
            fn = _resolve(node[FN], node)
            if extra_args or extra_kwargs:
                return fn(*extra_args, **extra_kwargs)
            return fn
        if TARGET in node:
            fn = _resolve(node[TARGET], node)
            a = [_build(v, tags) for v in node.get(ARGS, [])]
            kw = {k: _build(v, tags) for k, v in public_items(node)}
            if node.get(PARTIAL):
                if extra_args or extra_kwargs:
                    return functools.partial(fn, *a, **kw)(*extra_args, **extra_kwargs)
                return functools.partial(fn, *a, **kw) if (a or kw) else fn
            kw.update(extra_kwargs)
            return fn(*a, *extra_args, **kw)
        if PATCH in node:
            return node
        out = Field() if isinstance(node, Field) else {}
        for k, v in node.items():
            dict.__setitem__(out, k, _build(v, tags))
        return out
    if isinstance(node, list):
        return [_build(v, tags) for v in node]
    if isinstance(node, tuple):
        return tuple(_build(v, tags) for v in node)
    return node


# ----------------------------------------------------------------------------- select / patch

def _walk(node, visit):
    """Depth-first, parents before children, in insertion order."""
    if isinstance(node, dict):
        visit(node)
        for v in list(node.values()):
            _walk(v, visit)
    elif isinstance(node, (list, tuple)):
        for v in node:
            _walk(v, visit)


def _replace(node, pred, fn):
    """Return a tree where every dict node satisfying `pred` is replaced by fn(node);
    replacement happens bottom-up so nested matches are rewritten first."""
    if isinstance(node, dict):
        out = type(node)() if isinstance(node, Field) else Field()
        for k, v in node.items():
            dict.__setitem__(out, k, _replace(v, pred, fn))
        if pred(out):
            return normalize(fn(out))
        return out
    if isinstance(node, list):
        return [_replace(v, pred, fn) for v in node]
    if isinstance(node, tuple):
        return tuple(_replace(v, pred, fn) for v in node)
    return node


def _target_path(cls) -> str:
    if isinstance(cls, str):
        return cls
    return object_path(cls)


def _is_instance(node, path) -> bool:
    return isinstance(node, dict) and node.get(TARGET) == path and not node.get(PARTIAL)


def _subst(value, node, index):
    """'$name' -> node[name]; '$index' -> running index of the match."""
    if isinstance(value, str) and value.startswith("$"):
        key = value[1:]
        if key == "index":
            return index
        return node.get(key, _MISSING)
    return value


_MISSING = object()


class Selection:
    """`select(conf).instance(Cls).update_dict({...})` / `.map(fn)` on a copy of `conf`."""

    def __init__(self, conf):
        self._conf = conf
        self._path = None
        self._key = None

    def instance(self, cls):
        self._path = _target_path(cls)
        return self

    def at(self, key):
        self._key = key
        return self

    def _pred(self):
        path = self._path
        return lambda n: _is_instance(n, path)

    def update_dict(self, values):
        def fn(n):
            for k, v in values.items():
                n[k] = v
            return n

        return _replace(self._conf, self._pred(), fn)

    def map(self, fn):
        return _replace(self._conf, self._pred(), fn)

    def map_instance(self, cls, **kwargs):
        return apply_patches(self._conf, [_map_instance_op(self._path, cls, kwargs)])

    def set(self, value):
        key = self._key
        return self.update_dict({key: value})

    def set_sequence(self, value="$index"):
        return apply_patches(self._conf, [Field({PATCH: [
            {"op": "instance", "target": self._path},
            {"op": "at", "key": self._key},
            {"op": "set_sequence", "value": value},
        ]})])


def select(conf) -> Selection:
    return Selection(conf)


def _map_instance_op(src_path, cls, kwargs):
    return Field({PATCH: [
        {"op": "instance", "target": src_path},
        {"op": "map_instance", "target": _target_path(cls), "kwargs": normalize(dict(kwargs))},
    ]})


class PatchBuilder:
    """Deferred, serialisable rewrite: `patch_fn.select().instance(A).map_instance(B, k="$k").chain()`."""

    def __init__(self, ops=None):
        self._ops = list(ops or [])

    def select(self):
        return PatchBuilder([])

    def instance(self, cls):
        return PatchBuilder(self._ops + [{"op": "instance", "target": _target_path(cls)}])

    def at(self, key):
        return PatchBuilder(self._ops + [{"op": "at", "key": key}])

    def map_instance(self, cls, **kwargs):
        return PatchBuilder(self._ops + [
            {"op": "map_instance", "target": _target_path(cls), "kwargs": normalize(dict(kwargs))}])

    def update_dict(self, values):
        return PatchBuilder(self._ops + [{"op": "update_dict", "values": normalize(dict(values))}])

    def set(self, value):
        return PatchBuilder(self._ops + [{"op": "set", "value": value}])

    def set_sequence(self, value="$index"):
        return PatchBuilder(self._ops + [{"op": "set_sequence", "value": value}])

    def chain(self):
        return Field({PATCH: [normalize(o) for o in self._ops]})


patch_fn = PatchBuilder()


def apply_patches(conf, patches):
    conf = copy.deepcopy(conf)
    for p in patches:
        ops = p[PATCH] if isinstance(p, dict) else p
        target = None
        key = None
        for op in ops:
            kind = op["op"]
            if kind == "instance":
                target = op["target"]
            elif kind == "at":
                key = op["key"]
            elif kind == "map_instance":
                new_target, kw = op["target"], op["kwargs"]
                counter = [0]

                def fn(n, new_target=new_target, kw=kw, counter=counter):
                    out = Field()
                    dict.__setitem__(out, TARGET, new_target)
                    for k, v in kw.items():
                        val = _subst(v, n, counter[0])
                        if val is _MISSING:
                            continue
                        out[k] = copy.deepcopy(val)
                    counter[0] += 1
                    return out

                conf = _replace(conf, lambda n, t=target: _is_instance(n, t), fn)
            elif kind == "update_dict":
                vals = op["values"]
                conf = _replace(conf, lambda n, t=target: _is_instance(n, t),
                                lambda n, vals=vals: n.update_dict(copy.deepcopy(dict(vals))))
            elif kind in ("set", "set_sequence"):
                # document order (parents first) so "$index" follows the order of appearance
                matches = []
                _walk(conf, lambda n, t=target: matches.append(n) if _is_instance(n, t) else None)
                for i, n in enumerate(matches):
                    n[key] = _subst(op["value"], n, i)
            else:
                raise ValueError(f"unknown patch op {kind!r}")
    return conf


def patch(conf, patches=()):
    """Apply recorded patches to a config tree; returns the rewritten copy."""
    return apply_patches(conf, list(patches))


# ----------------------------------------------------------------------------- summary

def summarize(conf, indent: int = 0, max_list: int = 4) -> str:
    """Readable multi-line rendering of a config tree (repeated list items are folded)."""
    from .node import to_plain

    if hasattr(conf, "model_dump") and not isinstance(conf, dict):
        conf = conf.model_dump()
    lines: list[str] = []
    _summarize(to_plain(conf), indent, lines, max_list, key=None)
    return "\n".join(lines)


def _summarize(node, indent, lines, max_list, key):
    pad = "  " * indent
    head = f"{pad}{key}: " if key is not None else pad
    if isinstance(node, dict):
        if TUPLE in node and len(node) == 1:
            lines.append(f"{head}{tuple(node[TUPLE])!r}")
            return
        if FN in node:
            lines.append(f"{head}<{node[FN]}>")
            return
        if TARGET in node:
            name = node[TARGET].split(".")[-1]
            tagp = "partial " if node.get(PARTIAL) else ""
            lines.append(f"{head}{tagp}{name}(")
            for i, a in enumerate(node.get(ARGS, [])):
                _summarize(a, indent + 1, lines, max_list, key=f"[{i}]")
            for k, v in node.items():
                if k.startswith("__"):
                    continue
                _summarize(v, indent + 1, lines, max_list, key=k)
            lines.append(f"{pad})")
            return
        lines.append(f"{head}{{" if key is not None else f"{pad}{{")
        for k, v in node.items():
            _summarize(v, indent + 1, lines, max_list, key=k)
        lines.append(f"{pad}}}")
        return
    if isinstance(node, list):
        if not node or all(not isinstance(v, (dict, list)) for v in node):
            lines.append(f"{head}{node!r}")
            return
        lines.append(f"{head}[")
        i = 0
        while i < len(node):
            j = i
            while j + 1 < len(node) and _similar(node[j + 1], node[i]):
                j += 1
            _summarize(node[i], indent + 1, lines, max_list, key=f"({i})" if j == i else f"({i}-{j}) x{j - i + 1}")
            i = j + 1
        lines.append(f"{pad}]")
        return
    lines.append(f"{head}{node!r}")


def _similar(a, b):
    """Same structure up to per-layer indices (used to fold repeated transformer blocks)."""
    if isinstance(a, dict) and isinstance(b, dict):
        if a.keys() != b.keys():
            return False
        return all(_similar(a[k], b[k]) for k in a if k not in ("layer_id",))
    if isinstance(a, list) and isinstance(b, list):
        return len(a) == len(b) and all(_similar(x, y) for x, y in zip(a, b))
    return a == b
