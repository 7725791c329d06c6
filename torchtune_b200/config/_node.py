"""Self-contained config container used by every recipe.

The reference framework builds its config objects with OmegaConf
(torchtune/config/_parse.py:58-60, torchtune/config/_utils.py:198-202).  This
package owns an equivalent, PyYAML-based container so that no third-party
config library is required: attribute *and* item access, ``${a.b}``
interpolation (including inside longer strings), dotlist merging,
``to_container``/``to_yaml``/``save``, and custom resolvers
(``${eval:'...'}`` style).
"""
from __future__ import annotations

import copy
import io
import re
from typing import Any, Callable, Dict, Iterable, Iterator, List, Optional, Sequence, Union

import yaml

_INTERP = re.compile(r"\$\{([^${}]+)\}")
_RESOLVERS: Dict[str, Callable[..., Any]] = {}


def _arithmetic(expr: Any) -> Any:
    """``${eval:'<expr>'}``: numbers combined with ``+ - * / // % **`` and parentheses (the async GRPO configs derive queue and
    batch sizes this way).  Evaluated on the syntax tree — names, calls and attribute access are rejected."""
    import ast
    import operator as op

    ops = {ast.Add: op.add, ast.Sub: op.sub, ast.Mult: op.mul, ast.Div: op.truediv, ast.FloorDiv: op.floordiv, ast.Mod: op.mod, ast.Pow: op.pow, ast.USub: op.neg, ast.UAdd: op.pos}

    def ev(node):
        if isinstance(node, ast.Constant) and isinstance(node.value, (int, float)):
            return node.value
        if isinstance(node, ast.BinOp) and type(node.op) in ops:
            return ops[type(node.op)](ev(node.left), ev(node.right))
        if isinstance(node, ast.UnaryOp) and type(node.op) in ops:
            return ops[type(node.op)](ev(node.operand))
        raise InterpolationError(f"eval resolver accepts arithmetic on numbers only, got {expr!r}")

    if isinstance(expr, (int, float)):
        return expr
    return ev(ast.parse(str(expr).strip().strip("'\""), mode="eval").body)


_RESOLVERS["eval"] = _arithmetic


class ConfigKeyError(KeyError, AttributeError):
    """Raised for missing keys through either access style."""


class InterpolationError(ValueError):
    pass


class _YamlLoader(yaml.SafeLoader):
    """SafeLoader that also reads ``1e-5`` style floats as floats (YAML 1.2)."""


_YamlLoader.add_implicit_resolver(
    "tag:yaml.org,2002:float",
    re.compile(
        r"""^(?:[-+]?(?:[0-9][0-9_]*)\.[0-9_]*(?:[eE][-+]?[0-9]+)?
        |[-+]?(?:[0-9][0-9_]*)(?:[eE][-+]?[0-9]+)
        |\.[0-9_]+(?:[eE][-+]?[0-9]+)?
        |[-+]?\.(?:inf|Inf|INF)
        |\.(?:nan|NaN|NAN))$""",
        re.X,
    ),
    list("-+0123456789."),
)


def _wrap(value: Any, parent: Optional["_Node"], key: Any) -> Any:
    if isinstance(value, _Node):
        if value._parent is not None and value._parent is not parent:
            value = copy.deepcopy(value)
        value._parent, value._key = parent, key
        return value
    if isinstance(value, dict):
        return DictConfig(value, _parent=parent, _key=key)
    if isinstance(value, (list, tuple)):
        return ListConfig(value, _parent=parent, _key=key)
    return value


class _Node:
    _parent: Optional["_Node"]
    _key: Any

    def _root(self) -> "_Node":
        node = self
        while node._parent is not None:
            node = node._parent
        return node

    # -- interpolation -------------------------------------------------
    def _lookup_path(self, path: str) -> Any:
        path = path.strip()
        node: Any = self._root()
        if path.startswith("."):
            # relative: one dot = sibling, each extra dot = one level up
            node = self
            stripped = path.lstrip(".")
            for _ in range(len(path) - len(stripped) - 1):
                node = node._parent if node._parent is not None else node
            path = stripped
        for part in _split_dotpath(path):
            if isinstance(node, DictConfig):
                if part not in node._data:
                    raise InterpolationError(f"interpolation key '{path}' not found")
                node = node._get_resolved(part)
            elif isinstance(node, ListConfig):
                node = node._get_resolved(int(part))
            else:
                raise InterpolationError(f"interpolation key '{path}' not found")
        return node

    def _resolve_value(self, value: Any) -> Any:
        if not isinstance(value, str) or "${" not in value:
            return value
        whole = _INTERP.fullmatch(value)
        if whole:
            return self._resolve_expr(whole.group(1))
        prev = None
        while prev != value and "${" in value:
            prev = value
            value = _INTERP.sub(lambda m: str(self._resolve_expr(m.group(1))), value)
        return value

    def _resolve_expr(self, expr: str) -> Any:
        if ":" in expr:
            name, _, arg = expr.partition(":")
            name = name.strip()
            if name in _RESOLVERS:
                args = [_parse_scalar(a.strip()) for a in _split_args(arg)]
                args = [self._resolve_value(a) for a in args]
                return _RESOLVERS[name](*args)
            if name == "oc.env":
                import os

                parts = _split_args(arg)
                if parts[0] in os.environ:
                    return os.environ[parts[0]]
                if len(parts) > 1:
                    return _parse_scalar(parts[1])
                raise InterpolationError(f"environment variable {parts[0]} not set")
            raise InterpolationError(f"unknown resolver '{name}'")
        return self._lookup_path(expr)


def _split_args(arg: str) -> List[str]:
    out, depth, cur, quote = [], 0, "", None
    for ch in arg:
        if quote:
            cur += ch
            if ch == quote:
                quote = None
            continue
        if ch in "'\"":
            quote = ch
            cur += ch
        elif ch in "([{":
            depth += 1
            cur += ch
        elif ch in ")]}":
            depth -= 1
            cur += ch
        elif ch == "," and depth == 0:
            out.append(cur)
            cur = ""
        else:
            cur += ch
    out.append(cur)
    return out


def _split_dotpath(path: str) -> List[str]:
    parts: List[str] = []
    for piece in path.split("."):
        m = re.fullmatch(r"([^\[\]]*)((?:\[\d+\])*)", piece)
        if m and m.group(2):
            if m.group(1):
                parts.append(m.group(1))
            parts.extend(re.findall(r"\[(\d+)\]", m.group(2)))
        else:
            parts.append(piece)
    return [p for p in parts if p != ""]


def _parse_scalar(text: str) -> Any:
    """Parse a CLI/YAML scalar the way a YAML document would type it."""
    if not isinstance(text, str):
        return text
    try:
        return yaml.load(text, Loader=_YamlLoader)
    except yaml.YAMLError:
        return text


class DictConfig(_Node):
    """Mapping node with attribute access and lazy interpolation."""

    def __init__(self, content: Optional[dict] = None, _parent=None, _key=None):
        object.__setattr__(self, "_data", {})
        object.__setattr__(self, "_parent", _parent)
        object.__setattr__(self, "_key", _key)
        for k, v in (content or {}).items():
            self._data[k] = _wrap(v, self, k)

    # raw / resolved access
    def _get_resolved(self, key: Any) -> Any:
        return self._resolve_value(self._data[key])

    def __getitem__(self, key: Any) -> Any:
        if key not in self._data:
            raise ConfigKeyError(f"Missing key {key}")
        return self._get_resolved(key)

    def __getattr__(self, key: str) -> Any:
        if key.startswith("__") and key.endswith("__"):
            raise AttributeError(key)
        data = object.__getattribute__(self, "_data")
        if key not in data:
            raise ConfigKeyError(f"Missing key {key}")
        return self._get_resolved(key)

    def __setitem__(self, key: Any, value: Any) -> None:
        self._data[key] = _wrap(value, self, key)

    def __setattr__(self, key: str, value: Any) -> None:
        if key in ("_data", "_parent", "_key"):
            object.__setattr__(self, key, value)
        else:
            self[key] = value

    def __delitem__(self, key: Any) -> None:
        del self._data[key]

    def __delattr__(self, key: str) -> None:
        if key not in self._data:
            raise ConfigKeyError(key)
        del self._data[key]

    def __contains__(self, key: Any) -> bool:
        return key in self._data

    def __iter__(self) -> Iterator:
        return iter(self._data)

    def __len__(self) -> int:
        return len(self._data)

    def __bool__(self) -> bool:
        return bool(self._data)

    def keys(self):
        return self._data.keys()

    def values(self):
        return [self._get_resolved(k) for k in self._data]

    def items(self):
        return [(k, self._get_resolved(k)) for k in self._data]

    def get(self, key: Any, default: Any = None) -> Any:
        if key in self._data:
            value = self._get_resolved(key)
            return default if value is None else value
        return default

    def pop(self, key: Any, *default: Any) -> Any:
        if key in self._data:
            value = self._get_resolved(key)
            del self._data[key]
            return value
        if default:
            return default[0]
        raise ConfigKeyError(f"Missing key {key}")

    def update(self, other: Union[dict, "DictConfig"]) -> None:
        for k in other:
            self[k] = other[k] if not isinstance(other, DictConfig) else other._data[k]

    def copy(self) -> "DictConfig":
        return copy.deepcopy(self)

    def __deepcopy__(self, memo):
        new = DictConfig()
        for k, v in self._data.items():
            new._data[k] = _wrap(copy.deepcopy(v, memo) if not isinstance(v, _Node) else _detached_copy(v, memo), new, k)
        # keep interpolation context for detached copies of sub-nodes
        object.__setattr__(new, "_parent", None)
        if self._parent is not None:
            object.__setattr__(new, "_ctx", self._root())
        return new

    def _lookup_path(self, path: str) -> Any:  # honour stored context of sub-node copies
        ctx = self.__dict__.get("_ctx") if self._parent is None else None
        if ctx is not None and not path.strip().startswith("."):
            try:
                return _Node._lookup_path(self, path)
            except InterpolationError:
                return ctx._lookup_path(path)
        return _Node._lookup_path(self, path)

    def __eq__(self, other: Any) -> bool:
        if isinstance(other, DictConfig):
            return OmegaConf.to_container(self, resolve=True) == OmegaConf.to_container(other, resolve=True)
        if isinstance(other, dict):
            return OmegaConf.to_container(self, resolve=True) == other
        return NotImplemented

    def __repr__(self) -> str:
        return repr(OmegaConf.to_container(self, resolve=False))

    def __getstate__(self):
        return {"data": OmegaConf.to_container(self, resolve=False)}

    def __setstate__(self, state):
        self.__init__(state["data"])


def _detached_copy(node: _Node, memo) -> _Node:
    if isinstance(node, DictConfig):
        new = DictConfig()
        for k, v in node._data.items():
            new._data[k] = _wrap(_detached_copy(v, memo) if isinstance(v, _Node) else copy.deepcopy(v, memo), new, k)
        return new
    new_l = ListConfig()
    for i, v in enumerate(node._data):
        new_l._data.append(_wrap(_detached_copy(v, memo) if isinstance(v, _Node) else copy.deepcopy(v, memo), new_l, i))
    return new_l


class ListConfig(_Node):
    """Sequence node; recipes test ``isinstance(x, ListConfig)`` to detect multi-dataset configs."""

    def __init__(self, content: Optional[Iterable] = None, _parent=None, _key=None):
        self._data: List[Any] = []
        self._parent = _parent
        self._key = _key
        for i, v in enumerate(content or []):
            self._data.append(_wrap(v, self, i))

    def _get_resolved(self, idx: int) -> Any:
        return self._resolve_value(self._data[idx])

    def __getitem__(self, idx):
        if isinstance(idx, slice):
            return [self._resolve_value(v) for v in self._data[idx]]
        return self._get_resolved(idx)

    def __setitem__(self, idx: int, value: Any) -> None:
        self._data[idx] = _wrap(value, self, idx)

    def __len__(self) -> int:
        return len(self._data)

    def __iter__(self) -> Iterator:
        for i in range(len(self._data)):
            yield self._get_resolved(i)

    def __contains__(self, item: Any) -> bool:
        return any(v == item for v in self)

    def append(self, value: Any) -> None:
        self._data.append(_wrap(value, self, len(self._data)))

    def __deepcopy__(self, memo):
        new = _detached_copy(self, memo)
        return new

    def __eq__(self, other: Any) -> bool:
        if isinstance(other, ListConfig):
            return OmegaConf.to_container(self, resolve=True) == OmegaConf.to_container(other, resolve=True)
        if isinstance(other, (list, tuple)):
            return OmegaConf.to_container(self, resolve=True) == list(other)
        return NotImplemented

    def __repr__(self) -> str:
        return repr(OmegaConf.to_container(self, resolve=False))


class OmegaConf:
    """Static helpers mirroring the handful of OmegaConf calls recipes rely on
    (load, create, merge, resolve, to_container, to_yaml, save, from_dotlist,
    is_dict, is_list, register_new_resolver)."""

    @staticmethod
    def create(obj: Any = None) -> Union[DictConfig, ListConfig]:
        if obj is None:
            return DictConfig({})
        if isinstance(obj, str):
            obj = yaml.load(obj, Loader=_YamlLoader)
            if obj is None:
                return DictConfig({})
        if isinstance(obj, _Node):
            return copy.deepcopy(obj)
        if isinstance(obj, dict):
            return DictConfig(copy.deepcopy(obj))
        if isinstance(obj, (list, tuple)):
            return ListConfig(copy.deepcopy(list(obj)))
        raise TypeError(f"cannot create a config from {type(obj)}")

    @staticmethod
    def load(path_or_file: Any) -> Union[DictConfig, ListConfig]:
        if hasattr(path_or_file, "read"):
            data = yaml.load(path_or_file.read(), Loader=_YamlLoader)
        else:
            with open(path_or_file, "r") as f:
                data = yaml.load(f.read(), Loader=_YamlLoader)
        return OmegaConf.create(data if data is not None else {})

    @staticmethod
    def is_dict(obj: Any) -> bool:
        return isinstance(obj, DictConfig)

    @staticmethod
    def is_list(obj: Any) -> bool:
        return isinstance(obj, ListConfig)

    @staticmethod
    def is_config(obj: Any) -> bool:
        return isinstance(obj, _Node)

    @staticmethod
    def to_container(cfg: Any, resolve: bool = False) -> Any:
        if isinstance(cfg, DictConfig):
            out = {}
            for k, v in cfg._data.items():
                if isinstance(v, _Node):
                    out[k] = OmegaConf.to_container(v, resolve)
                else:
                    out[k] = cfg._resolve_value(v) if resolve else v
                    if isinstance(out[k], _Node):
                        out[k] = OmegaConf.to_container(out[k], resolve)
            return out
        if isinstance(cfg, ListConfig):
            out_l = []
            for v in cfg._data:
                if isinstance(v, _Node):
                    out_l.append(OmegaConf.to_container(v, resolve))
                else:
                    r = cfg._resolve_value(v) if resolve else v
                    out_l.append(OmegaConf.to_container(r, resolve) if isinstance(r, _Node) else r)
            return out_l
        return cfg

    @staticmethod
    def to_object(cfg: Any) -> Any:
        return OmegaConf.to_container(cfg, resolve=True)

    @staticmethod
    def resolve(cfg: _Node) -> None:
        """Replace every interpolation in-place by its value."""
        if isinstance(cfg, DictConfig):
            keys: Sequence = list(cfg._data.keys())
        else:
            keys = range(len(cfg._data))
        for k in keys:
            v = cfg._data[k]
            if isinstance(v, _Node):
                OmegaConf.resolve(v)
            else:
                r = cfg._resolve_value(v)
                cfg._data[k] = _wrap(copy.deepcopy(r), cfg, k) if isinstance(r, _Node) else r

    @staticmethod
    def to_yaml(cfg: Any, resolve: bool = False, sort_keys: bool = False) -> str:
        data = OmegaConf.to_container(cfg, resolve=resolve)
        return yaml.safe_dump(data, sort_keys=sort_keys, default_flow_style=False, allow_unicode=True)

    @staticmethod
    def save(config: Any, f: Any, resolve: bool = False) -> None:
        text = OmegaConf.to_yaml(config, resolve=resolve)
        if isinstance(f, io.IOBase) or hasattr(f, "write"):
            f.write(text)
        else:
            with open(f, "w") as fh:
                fh.write(text)

    @staticmethod
    def from_dotlist(dotlist: Sequence[str]) -> DictConfig:
        cfg = DictConfig({})
        for item in dotlist:
            key, sep, value = item.partition("=")
            if not sep:
                raise ValueError(f"dotlist entry '{item}' is not of the form key=value")
            OmegaConf.update(cfg, key, _parse_scalar(value) if value != "" else None)
        return cfg

    @staticmethod
    def update(cfg: DictConfig, dotpath: str, value: Any) -> None:
        parts = _split_dotpath(dotpath)
        node: Any = cfg
        for i, part in enumerate(parts[:-1]):
            if isinstance(node, ListConfig):
                node = node._data[int(part)]
                continue
            nxt = node._data.get(part)
            if not isinstance(nxt, _Node):
                nxt = DictConfig({}, _parent=node, _key=part)
                node._data[part] = nxt
            node = nxt
        last = parts[-1]
        if isinstance(node, ListConfig):
            node[int(last)] = value
        else:
            node[last] = value

    @staticmethod
    def select(cfg: _Node, dotpath: str, default: Any = None) -> Any:
        try:
            return cfg._lookup_path(dotpath)
        except (InterpolationError, IndexError, ValueError):
            return default

    @staticmethod
    def merge(*configs: Any) -> Union[DictConfig, ListConfig]:
        """Later configs win; dicts merge recursively, everything else is replaced."""
        result = OmegaConf.create(configs[0]) if not isinstance(configs[0], _Node) else copy.deepcopy(configs[0])
        for other in configs[1:]:
            other = other if isinstance(other, _Node) else OmegaConf.create(other)
            if isinstance(result, DictConfig) and isinstance(other, DictConfig):
                _merge_into(result, other)
            else:
                result = copy.deepcopy(other)
        return result

    @staticmethod
    def register_new_resolver(name: str, fn: Callable[..., Any], replace: bool = False) -> None:
        if name in _RESOLVERS and not replace:
            raise ValueError(f"resolver '{name}' is already registered")
        _RESOLVERS[name] = fn

    @staticmethod
    def has_resolver(name: str) -> bool:
        return name in _RESOLVERS

    @staticmethod
    def clear_resolver(name: str) -> None:
        _RESOLVERS.pop(name, None)


def _merge_into(dst: DictConfig, src: DictConfig) -> None:
    for k, v in src._data.items():
        cur = dst._data.get(k)
        if isinstance(cur, DictConfig) and isinstance(v, DictConfig):
            _merge_into(cur, v)
        else:
            dst[k] = _detached_copy(v, {}) if isinstance(v, _Node) else copy.deepcopy(v)
