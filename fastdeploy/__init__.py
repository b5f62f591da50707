"""``import fastdeploy`` for programs written against PaddlePaddle/FastDeploy 1.x: every ``fastdeploy[.x.y]`` module IS the
``fastdeploy_b200[.x.y]`` module (one module object under two names, so classes and ``isinstance`` agree whichever name a
program imported them by)."""
import importlib
import importlib.abc
import importlib.machinery
import sys

_ALIAS, _REAL = "fastdeploy", "fastdeploy_b200"


class _AliasFinder(importlib.abc.MetaPathFinder, importlib.abc.Loader):
    def find_spec(self, fullname, path=None, target=None):
        if fullname != _ALIAS and not fullname.startswith(_ALIAS + "."):
            return None
        real = _REAL + fullname[len(_ALIAS):]
        try:
            module = importlib.import_module(real)
        except ModuleNotFoundError as e:
            if e.name == real:
                return None
            raise
        spec = importlib.machinery.ModuleSpec(fullname, self, is_package=hasattr(module, "__path__"))
        spec._aliased = module
        return spec

    def create_module(self, spec):
        return spec._aliased

    def exec_module(self, module):
        pass


if not any(isinstance(f, _AliasFinder) for f in sys.meta_path):
    sys.meta_path.insert(0, _AliasFinder())
_impl = importlib.import_module(_REAL)
sys.modules[_ALIAS] = _impl
