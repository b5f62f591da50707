"""The CMake build: host library, plan runner and tool build and install, and a consumer project finds the package."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
NVCC = shutil.which("nvcc") or ("/usr/local/cuda/bin/nvcc" if os.path.exists("/usr/local/cuda/bin/nvcc") else None)
pytestmark = pytest.mark.skipif(shutil.which("cmake") is None or NVCC is None, reason="cmake and nvcc are needed")

CONSUMER = """cmake_minimum_required(VERSION 3.24)
project(consumer LANGUAGES C CXX)
find_package(FastDeployB200 REQUIRED)
add_executable(smoke smoke.c)
target_include_directories(smoke PRIVATE ${FastDeployB200_INCLUDE_DIR})
target_link_libraries(smoke PRIVATE FastDeployB200::fdb200_runner)
"""


def test_cmake_build_install_and_find_package(tmp_path):
    gen = ["-G", "Ninja"] if shutil.which("ninja") else []
    env = dict(os.environ, CUDACXX=NVCC)
    build, inst = str(tmp_path / "b"), str(tmp_path / "inst")
    # the kernel library is left out here: its build is the long one and `python -m fastdeploy_b200._native.build`
    # already covers it; its target is configured in the last step below
    subprocess.run(["cmake", "-S", ROOT, "-B", build, "-DFDB_BUILD_KERNELS=OFF"] + gen, check=True, env=env,
                   stdout=subprocess.DEVNULL)
    subprocess.run(["cmake", "--build", build], check=True, env=env, stdout=subprocess.DEVNULL)
    subprocess.run(["cmake", "--install", build, "--prefix", inst], check=True, env=env, stdout=subprocess.DEVNULL)
    for rel in ("lib/libfdb200_cpu.so", "lib/libfdb200_runner.so", "bin/fdplan_run", "include/fastdeploy_b200/fd_plan_runner.h",
                "lib/cmake/FastDeployB200/FastDeployB200Config.cmake"):
        assert os.path.exists(os.path.join(inst, rel)), rel
    usage = subprocess.run([os.path.join(inst, "bin", "fdplan_run")], capture_output=True, text=True)
    assert usage.returncode == 2 and "usage" in usage.stderr
    cons = tmp_path / "consumer"
    cons.mkdir()
    (cons / "CMakeLists.txt").write_text(CONSUMER)
    shutil.copy(os.path.join(ROOT, "tests", "plan_runner_smoke.c"), cons / "smoke.c")
    subprocess.run(["cmake", "-S", str(cons), "-B", str(cons / "b"), f"-DCMAKE_PREFIX_PATH={inst}"] + gen, check=True,
                   env=env, stdout=subprocess.DEVNULL)
    subprocess.run(["cmake", "--build", str(cons / "b")], check=True, env=env, stdout=subprocess.DEVNULL)
    junk = tmp_path / "junk.fdplan"
    junk.write_bytes(b"junk")
    run = subprocess.run([str(cons / "b" / "smoke"), "/nonexistent/kernels.so", str(tmp_path / "absent"), str(junk)],
                         capture_output=True, text=True, env=dict(env, LD_LIBRARY_PATH=os.path.join(inst, "lib")))
    assert run.returncode == 0 and run.stdout.count("null") == 3, run.stdout + run.stderr
    # the full configuration (kernels on, sm_100a only) at least configures
    subprocess.run(["cmake", "-S", ROOT, "-B", str(tmp_path / "full")] + gen, check=True, env=env, stdout=subprocess.DEVNULL)
    cache = (tmp_path / "full" / "CMakeCache.txt").read_text()
    assert "CMAKE_CUDA_ARCHITECTURES" in cache and "100a" in cache
