"""``fastdeploy.model`` (python/fastdeploy/model.py): the base class under the reference's module path."""
from .runtime.model import FastDeployModel  # noqa: F401
