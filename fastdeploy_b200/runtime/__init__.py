"""``fastdeploy.runtime`` (python/fastdeploy/runtime.py): ``Runtime`` and ``RuntimeOption`` are importable from here too."""
from .option import RuntimeOption  # noqa: F401
from .runtime import Runtime  # noqa: F401
