"""Import-name compatibility: code written against the reference imports ``nkigen`` (and its
submodules); here the implementation lives in ``nkipy_b200.nkigen``.  Importing ``nkigen`` or any
``nkigen.x.y`` returns the very same module objects as ``nkipy_b200.nkigen`` / ``nkipy_b200.nkigen.x.y``."""

import importlib
import importlib.abc
import importlib.util
import sys

_ALIAS, _REAL = "nkigen", "nkipy_b200.nkigen"


class _AliasFinder(importlib.abc.MetaPathFinder, importlib.abc.Loader):
    def find_spec(self, fullname, path=None, target=None):
        if fullname.startswith(_ALIAS + "."):
            real = _REAL + fullname[len(_ALIAS):]
            try:
                if importlib.util.find_spec(real) is None:
                    return None
            except (ImportError, ValueError):
                return None
            return importlib.util.spec_from_loader(fullname, self)
        return None

    def create_module(self, spec):
        module = importlib.import_module(_REAL + spec.name[len(_ALIAS):])
        self._own_spec = getattr(self, "_own_spec", {})
        self._own_spec[spec.name] = (module.__spec__, getattr(module, "__loader__", None))
        return module

    def exec_module(self, module):
        # the import machinery has just stamped the alias spec on the shared module object: give it its own
        # back, or its relative imports would see a package name that differs from its spec's parent
        for name, (own, loader) in list(getattr(self, "_own_spec", {}).items()):
            if getattr(module, "__spec__", None) is not None and module.__spec__.name == name:
                module.__spec__ = own
                if loader is not None:
                    module.__loader__ = loader
                del self._own_spec[name]
        return None


if not any(isinstance(f, _AliasFinder) for f in sys.meta_path):
    sys.meta_path.insert(0, _AliasFinder())

_impl = importlib.import_module(_REAL)
globals().update({k: v for k, v in vars(_impl).items() if not k.startswith("__")})
__all__ = getattr(_impl, "__all__", [k for k in vars(_impl) if not k.startswith("_")])
