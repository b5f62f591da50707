"""Directories of the local model hub (python/fastdeploy/utils/hub_env.py:26-55): ``HUB_HOME`` is ``$HUB_HOME`` or
``~/.fastdeploy``; models, configuration and example resources live in sub-directories of it. Importing this module only
computes the paths; a directory is created by whoever first writes into it."""
import os


def _get_user_home() -> str:
    return os.path.expanduser("~")


def _get_hub_home() -> str:
    home = os.environ.get("HUB_HOME")
    if home:
        if os.path.exists(home) and not os.path.isdir(home):
            raise RuntimeError("The environment variable HUB_HOME {} is not a directory.".format(home))
        return home
    return os.path.join(_get_user_home(), ".fastdeploy")


def _get_sub_home(directory: str) -> str:
    return os.path.join(_get_hub_home(), directory)


USER_HOME = _get_user_home()
HUB_HOME = _get_hub_home()
MODEL_HOME = _get_sub_home("models")
CONF_HOME = _get_sub_home("conf")
RESOURCE_HOME = _get_sub_home("resources")
