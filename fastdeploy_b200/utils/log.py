"""Logger with the reference's prefixes and global switches
(fastdeploy/utils/utils.cc:22-48: ``[INFO]`` / ``[WARNING]`` / ``[ERROR]`` + file(line)::function)."""
from __future__ import annotations

import inspect
import json
import os
import sys
import time

_enable_info = True
_enable_warning = True
_json_lines = os.environ.get("FDX_LOG_JSON", "0") == "1"


def set_logger(enable_info: bool = True, enable_warning: bool = True) -> None:
    global _enable_info, _enable_warning
    _enable_info, _enable_warning = bool(enable_info), bool(enable_warning)


def _emit(level: str, msg: str, stream) -> None:
    fr = inspect.stack()[2]
    where = f"{os.path.basename(fr.filename)}({fr.lineno})::{fr.function}"
    if _json_lines:
        stream.write(json.dumps({"ts": time.time(), "level": level, "where": where, "msg": msg}) + "\n")
    else:
        stream.write(f"[{level}] {where}\t{msg}\n")
    stream.flush()


def info(msg: str) -> None:
    if _enable_info:
        _emit("INFO", msg, sys.stdout)


def warning(msg: str) -> None:
    if _enable_warning:
        _emit("WARNING", msg, sys.stdout)


def error(msg: str) -> None:
    _emit("ERROR", msg, sys.stderr)


class FDAssertionError(RuntimeError):
    pass


def fdassert(cond: bool, msg: str) -> None:
    """The reference aborts the process (fastdeploy/utils/utils.h:95-102); here it raises."""
    if not cond:
        error(msg)
        raise FDAssertionError(msg)
