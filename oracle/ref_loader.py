"""Import the upstream ``qutai`` package (pure Python, written for Python >= 3.14) under
Python 3.12 so that its CPU float64 path can generate golden vectors.

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package imports this file; it is used by
``tests/golden/make_golden.py`` (fixture generation) and by the optional cross-check tests that
run only where a checkout of the upstream sources is present.

Two load-time source transforms are applied, neither of which touches arithmetic:

* ``from __future__ import annotations`` is prepended to every module, because the upstream
  sources use unquoted forward references in annotations (legal with deferred evaluation only);
* ``contextvars.ContextVar`` is replaced by a thin wrapper whose ``set()`` returns a token that
  also works as a context manager (``with var.set(x): ...``), a Python 3.14 feature the upstream
  code relies on (src/qutai/core/context.py:8-20, src/qutai/backends/precision.py:10-11,
  src/qutai/lm/recompute.py:52).
"""
from __future__ import annotations

import contextvars
import importlib.abc
import importlib.util
import os
import sys
import types

_SHIM_NAME = "_qutai_py312_shim"


class _Token:
    def __init__(self, var, token):
        self._var, self._token = var, token

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self._var.reset(self._token)
        return False


class _Var:
    def __init__(self, name, **kw):
        self._var = contextvars.ContextVar(name, **kw)

    def get(self, *default):
        return self._var.get(*default)

    def set(self, value):
        return _Token(self._var, self._var.set(value))

    def reset(self, token):
        self._var.reset(token._token if isinstance(token, _Token) else token)


def _install_shim():
    if _SHIM_NAME not in sys.modules:
        module = types.ModuleType(_SHIM_NAME)
        module.ContextVar = _Var
        module.Token = _Token
        sys.modules[_SHIM_NAME] = module


class _Loader(importlib.abc.SourceLoader):
    def __init__(self, fullname, path):
        self._fullname, self._path = fullname, path

    def get_filename(self, fullname):
        return self._path

    def get_data(self, path):
        with open(path, "rb") as handle:
            data = handle.read()
        if not path.endswith(".py"):
            return data
        text = data.decode("utf-8")
        text = text.replace("from contextvars import", f"from {_SHIM_NAME} import")
        if text.strip():
            text = "from __future__ import annotations\n" + text
        return text.encode("utf-8")

    def path_stats(self, path):
        raise OSError  # never read or write byte-code caches (the source tree may be read-only)

    def set_data(self, path, data):
        return None


class _Finder(importlib.abc.MetaPathFinder):
    def __init__(self, root):
        self._root = root

    def find_spec(self, fullname, path=None, target=None):
        if fullname != "qutai" and not fullname.startswith("qutai."):
            return None
        base = os.path.join(self._root, *fullname.split("."))
        if os.path.isdir(base) and os.path.isfile(os.path.join(base, "__init__.py")):
            filename = os.path.join(base, "__init__.py")
            return importlib.util.spec_from_file_location(
                fullname, filename, loader=_Loader(fullname, filename),
                submodule_search_locations=[base])
        if os.path.isfile(base + ".py"):
            return importlib.util.spec_from_file_location(
                fullname, base + ".py", loader=_Loader(fullname, base + ".py"))
        return None


def reference_root():
    """Directory holding the upstream ``src/qutai`` tree, or None when it is not mounted."""
    # QUTAI_REFERENCE_SRC, else a checkout named "reference" next to this repository
    beside = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "reference", "src")
    root = os.environ.get("QUTAI_REFERENCE_SRC", beside)
    return root if os.path.isfile(os.path.join(root, "qutai", "__init__.py")) else None


def load():
    """Return the imported upstream ``qutai`` package (raises ImportError when absent)."""
    if "qutai" in sys.modules:
        return sys.modules["qutai"]
    root = reference_root()
    if root is None:
        raise ImportError("upstream qutai sources are not present on this machine")
    _install_shim()
    sys.dont_write_bytecode = True
    sys.meta_path.insert(0, _Finder(root))
    import qutai  # noqa: F401

    return sys.modules["qutai"]
