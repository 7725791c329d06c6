"""Import-time stand-ins for two third-party packages the reference imports but this image
does not ship (``torchao``, ``omegaconf``).

The reference refuses to import without them, although the bf16 full-finetune path the
benchmark exercises never calls into either.  ``install()`` registers a meta-path finder
that fabricates empty modules for ``torchao.*`` / ``omegaconf.*`` whose attributes are inert
placeholder classes (subclassable, callable, usable as decorators).  Nothing of the reference
is modified; any real *use* of a placeholder raises.
"""
from __future__ import annotations

import importlib.abc
import importlib.machinery
import sys
import types

_ROOTS = ("torchao", "omegaconf")


class _PlaceholderMeta(type):
    def __getattr__(cls, name):
        if name.startswith("__"):
            raise AttributeError(name)
        return _make_placeholder(f"{cls.__name__}.{name}")

    def __call__(cls, *args, **kwargs):
        # used as a decorator factory / decorator: hand back the decorated object unchanged
        if len(args) == 1 and callable(args[0]) and not kwargs and not isinstance(args[0], _PlaceholderMeta):
            return args[0]
        return lambda obj=None, *a, **k: obj

    def __instancecheck__(cls, instance):
        return False


def _make_placeholder(name: str):
    return _PlaceholderMeta(name, (), {"__module__": "missing_deps"})


class _StubModule(types.ModuleType):
    def __getattr__(self, name):
        if name.startswith("__"):
            raise AttributeError(name)
        value = _make_placeholder(name)
        setattr(self, name, value)
        return value


class _Finder(importlib.abc.MetaPathFinder, importlib.abc.Loader):
    def find_spec(self, fullname, path=None, target=None):
        if fullname.split(".")[0] in _ROOTS:
            return importlib.machinery.ModuleSpec(fullname, self, is_package=True)
        return None

    def create_module(self, spec):
        mod = _StubModule(spec.name)
        mod.__path__ = []
        mod.__version__ = "0.0.0+stub"
        return mod

    def exec_module(self, module):
        pass


def install() -> None:
    if not any(isinstance(f, _Finder) for f in sys.meta_path):
        sys.meta_path.append(_Finder())
