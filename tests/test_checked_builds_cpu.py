"""Checked variants of the native libraries: the host library under AddressSanitizer and
UndefinedBehaviorSanitizer runs the tokenizer, scheduler and core tests clean."""
import os
import subprocess
import sys

import pytest

from fastdeploy_b200._native import build as B

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HOST_TESTS = ["tests/test_text_cpu.py", "tests/test_serving_cpu.py", "tests/test_core_functions.py",
              "tests/test_function_native_cpu.py"]


def _env(mode):
    rt = B.sanitizer_runtime(mode)
    if not rt:
        pytest.skip(f"the {mode} runtime is not installed with this compiler")
    cxx_rt = subprocess.run(["g++", "-print-file-name=libstdc++.so"], stdout=subprocess.PIPE, text=True).stdout.strip()
    env = dict(os.environ)
    # the C++ runtime goes in with the sanitizer: the interpreter is a C program, and the sanitizer resolves the
    # exception entry points it wraps when it starts
    env["LD_PRELOAD"] = rt + " " + cxx_rt
    env["FDX_NATIVE_VARIANT"] = mode
    env["ASAN_OPTIONS"] = "detect_leaks=0:halt_on_error=1"
    env["UBSAN_OPTIONS"] = "halt_on_error=1:print_stacktrace=1"
    return env


@pytest.mark.parametrize("mode", ["asan", "ubsan"])
def test_host_library_is_clean_under_sanitizer(mode):
    lib = B.build_variant(mode)
    env = _env(mode)
    where = subprocess.run([sys.executable, "-c", "from fastdeploy_b200 import _native; print(_native.cpu()._name)"],
                           cwd=ROOT, env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=300)
    assert where.returncode == 0 and where.stdout.strip().endswith(os.path.relpath(lib, ROOT)), where.stdout[-2000:]
    run = subprocess.run([sys.executable, "-m", "pytest", "-q", "-x", "-p", "no:cacheprovider"] + HOST_TESTS,
                         cwd=ROOT, env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=900)
    assert run.returncode == 0, run.stdout[-4000:]
    assert "runtime error" not in run.stdout and "AddressSanitizer" not in run.stdout


def test_unknown_mode_is_refused():
    with pytest.raises(ValueError):
        B.build_variant("fast")
