"""Builds the native libraries in-tree with nvcc / g++ (no JIT cache involved).

Two shared objects are produced next to this file:

* ``libfdb200_kernels.so`` - every CUDA kernel, compiled only for sm_100a
  (``-gencode arch=compute_100a,code=sm_100a``), exposing a plain C ABI.
* ``libfdb200_cpu.so`` - the host-side runtime pieces written in C++
  (post-processing oracles, tokenizer, schedulers, crypto, C API).

Run ``python -m fastdeploy_b200._native.build`` to (re)build; objects are cached
by source mtime under ``build/``.

Checked variants (``--mode``) are written under ``build/<mode>/`` and never replace the release libraries:

* ``boundscheck`` - the kernel library with ``-DFDB_BOUNDS_CHECK``: data-dependent indices that the release
  build clamps are counted and the first offender kept (``fdb_bounds_report``). Load it with
  ``FDX_NATIVE_VARIANT=boundscheck``.
* ``asan`` / ``tsan`` / ``ubsan`` - the host library with the matching ``-fsanitize=`` flag and frame
  pointers; run a host test with it by pre-loading the sanitizer runtime (``sanitizer_runtime(mode)``)
  and ``FDX_NATIVE_VARIANT=<mode>``.
"""
from __future__ import annotations

import concurrent.futures as cf
import glob
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
CSRC = os.path.join(ROOT, "csrc")
OBJ_DIR = os.path.join(ROOT, "build", "obj")

KERNEL_LIB = os.path.join(HERE, "libfdb200_kernels.so")
CPU_LIB = os.path.join(HERE, "libfdb200_cpu.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
    "-Xptxas", "-v",
]
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-fvisibility=hidden", "-pthread", "-Wall"]


def _nvcc() -> str:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found")
    return cand


def _newer(src: str, dst: str, deps: list[str]) -> bool:
    if not os.path.exists(dst):
        return True
    t = os.path.getmtime(dst)
    return any(os.path.getmtime(p) > t for p in [src] + deps)


def _compile(cmd: list[str], log_path: str) -> tuple[int, str]:
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    with open(log_path, "w") as f:
        f.write(" ".join(cmd) + "\n" + proc.stdout)
    return proc.returncode, proc.stdout


SANITIZERS = {"asan": "address", "tsan": "thread", "ubsan": "undefined"}


def variant_dir(mode: str) -> str:
    return os.path.join(ROOT, "build", mode)


def variant_lib(mode: str) -> str:
    """Path of the checked library of ``mode`` (kernels for ``boundscheck``, the host library for sanitizers)."""
    name = "libfdb200_kernels.so" if mode == "boundscheck" else "libfdb200_cpu.so"
    return os.path.join(variant_dir(mode), name)


def sanitizer_runtime(mode: str) -> str:
    """Shared runtime of the sanitizer (to be put in LD_PRELOAD of the process that loads the checked library)."""
    cxx = shutil.which("g++") or "g++"
    name = {"asan": "libasan.so", "tsan": "libtsan.so", "ubsan": "libubsan.so"}[mode]
    out = subprocess.run([cxx, "-print-file-name=" + name], stdout=subprocess.PIPE, text=True).stdout.strip()
    return out if os.path.isabs(out) and os.path.exists(out) else ""


def build_variant(mode: str, verbose: bool = False, force: bool = False) -> str:
    """Builds one checked library into ``build/<mode>/`` (objects cached by source mtime) and returns its path."""
    out_dir = variant_dir(mode)
    os.makedirs(out_dir, exist_ok=True)
    lib = variant_lib(mode)
    if mode == "boundscheck":
        nvcc = _nvcc()
        srcs = sorted(glob.glob(os.path.join(CSRC, "kernels", "*.cu")))
        jobs = [(s, [nvcc] + NVCC_FLAGS + ["-DFDB_BOUNDS_CHECK=1", "-I", os.path.join(CSRC, "kernels"), "-c", s, "-o",
                                           os.path.join(out_dir, os.path.basename(s) + ".o")],
                 os.path.join(out_dir, os.path.basename(s) + ".log")) for s in srcs]
        link = [nvcc, "-shared", "-o", lib] + [j[1][-1] for j in jobs] + \
               ["-gencode", "arch=compute_100a,code=sm_100a", "-cudart", "static", "-ldl"]
    elif mode in SANITIZERS:
        cxx = shutil.which("g++") or "g++"
        flags = [f for f in CXX_FLAGS if f != "-O2"] + ["-O1", "-g", "-fno-omit-frame-pointer",
                                                         "-fsanitize=" + SANITIZERS[mode]]
        srcs = sorted(glob.glob(os.path.join(CSRC, "cpu", "*.cc")))
        jobs = [(s, [cxx] + flags + ["-I", os.path.join(CSRC, "cpu"), "-I", os.path.join(CSRC, "capi"), "-c", s, "-o",
                                     os.path.join(out_dir, "cpu_" + os.path.basename(s) + ".o")],
                 os.path.join(out_dir, "cpu_" + os.path.basename(s) + ".log")) for s in srcs]
        link = [cxx, "-shared", "-o", lib] + [j[1][-1] for j in jobs] + ["-pthread", "-fsanitize=" + SANITIZERS[mode]]
    else:
        raise ValueError(f"unknown build mode {mode!r}: boundscheck, asan, tsan or ubsan")
    sub = "kernels" if mode == "boundscheck" else "cpu"
    hdrs = [h for pat in ("*.h", "*.cuh") for h in glob.glob(os.path.join(CSRC, sub, pat))]
    todo = [j for j in jobs if force or _newer(j[0], j[1][-1], hdrs)]
    if not todo and os.path.exists(lib):
        return lib
    with cf.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as ex:
        futs = {ex.submit(_compile, cmd, log): src for src, cmd, log in todo}
        for fut in cf.as_completed(futs):
            rc, out = fut.result()
            if verbose or rc != 0:
                print(out)
            if rc != 0:
                raise RuntimeError(f"compiling {futs[fut]} for mode {mode} failed")
    rc, out = _compile(link, os.path.join(out_dir, "link.log"))
    if rc != 0:
        print(out)
        raise RuntimeError(f"linking {lib} failed")
    return lib


def build_kernels(verbose: bool = False, force: bool = False) -> str:
    os.makedirs(OBJ_DIR, exist_ok=True)
    srcs = sorted(glob.glob(os.path.join(CSRC, "kernels", "*.cu")))
    hdrs = glob.glob(os.path.join(CSRC, "kernels", "*.h")) + glob.glob(os.path.join(CSRC, "kernels", "*.cuh"))
    nvcc = _nvcc()
    jobs = []
    objs = []
    for s in srcs:
        o = os.path.join(OBJ_DIR, os.path.basename(s) + ".o")
        objs.append(o)
        if force or _newer(s, o, hdrs):
            jobs.append((s, [nvcc] + NVCC_FLAGS + ["-I", os.path.join(CSRC, "kernels"), "-c", s, "-o", o],
                         o + ".log"))
    with cf.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as ex:
        futs = {ex.submit(_compile, cmd, log): src for src, cmd, log in jobs}
        for fut in cf.as_completed(futs):
            rc, out = fut.result()
            if verbose or rc != 0:
                print(out)
            if rc != 0:
                raise RuntimeError(f"nvcc failed on {futs[fut]}")
    if force or jobs or not os.path.exists(KERNEL_LIB):
        cmd = [nvcc, "-shared", "-o", KERNEL_LIB] + objs + ["-gencode", "arch=compute_100a,code=sm_100a",
                                                           "-cudart", "static", "-ldl"]
        rc, out = _compile(cmd, os.path.join(OBJ_DIR, "link_kernels.log"))
        if rc != 0:
            print(out)
            raise RuntimeError("linking libfdb200_kernels.so failed")
    return KERNEL_LIB


def build_cpu(verbose: bool = False, force: bool = False) -> str:
    os.makedirs(OBJ_DIR, exist_ok=True)
    srcs = sorted(glob.glob(os.path.join(CSRC, "cpu", "*.cc")))
    if not srcs:
        return ""
    hdrs = glob.glob(os.path.join(CSRC, "cpu", "*.h"))
    cxx = shutil.which("g++") or "g++"
    jobs = []
    objs = []
    for s in srcs:
        o = os.path.join(OBJ_DIR, "cpu_" + os.path.basename(s) + ".o")
        objs.append(o)
        if force or _newer(s, o, hdrs):
            jobs.append((s, [cxx] + CXX_FLAGS + ["-I", os.path.join(CSRC, "cpu"), "-I", os.path.join(CSRC, "capi"),
                                                 "-c", s, "-o", o], o + ".log"))
    with cf.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as ex:
        futs = {ex.submit(_compile, cmd, log): src for src, cmd, log in jobs}
        for fut in cf.as_completed(futs):
            rc, out = fut.result()
            if verbose or rc != 0:
                print(out)
            if rc != 0:
                raise RuntimeError(f"g++ failed on {futs[fut]}")
    if force or jobs or not os.path.exists(CPU_LIB):
        cmd = [cxx, "-shared", "-o", CPU_LIB] + objs + ["-pthread"]
        rc, out = _compile(cmd, os.path.join(OBJ_DIR, "link_cpu.log"))
        if rc != 0:
            print(out)
            raise RuntimeError("linking libfdb200_cpu.so failed")
    return CPU_LIB


CAPI_LIB = os.path.join(HERE, "libfastdeploy_capi.so")


def build_capi(verbose: bool = False, force: bool = False) -> str:
    """C API shared library (embeds the interpreter: links libpython of the running Python)."""
    import sysconfig
    srcs = sorted(glob.glob(os.path.join(CSRC, "capi", "*.cc")))
    if not srcs:
        return ""
    hdrs = glob.glob(os.path.join(CSRC, "capi", "*.h"))
    if not force and os.path.exists(CAPI_LIB) and not any(_newer(s, CAPI_LIB, hdrs) for s in srcs):
        return CAPI_LIB
    inc = sysconfig.get_paths()["include"]
    if not os.path.exists(os.path.join(inc, "Python.h")):
        return ""            # no interpreter headers on this machine: the C API is optional
    libdir = sysconfig.get_config_var("LIBDIR") or ""
    ver = sysconfig.get_config_var("LDVERSION") or sysconfig.get_python_version()
    cxx = shutil.which("g++") or "g++"
    cmd = [cxx] + CXX_FLAGS + ["-shared", "-I", inc, "-I", os.path.join(CSRC, "capi")] + srcs + \
          ["-o", CAPI_LIB, "-L", libdir, f"-lpython{ver}", f"-Wl,-rpath,{libdir}"]
    os.makedirs(OBJ_DIR, exist_ok=True)
    rc, out = _compile(cmd, os.path.join(OBJ_DIR, "link_capi.log"))
    if verbose or rc != 0:
        print(out)
    if rc != 0:
        raise RuntimeError("building libfastdeploy_capi.so failed")
    return CAPI_LIB


RUNNER_LIB = os.path.join(HERE, "libfdb200_runner.so")
RUNNER_TOOL = os.path.join(HERE, "fdplan_run")


def build_runner(verbose: bool = False, force: bool = False) -> str:
    """Plan runner: a library and a command-line tool that replay an exported plan without Python."""
    src = os.path.join(CSRC, "runner", "plan_runner.cu")
    if not os.path.exists(src):
        return ""
    nvcc = _nvcc()
    common = ["-O2", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-cudart", "static", "-ldl"]
    os.makedirs(OBJ_DIR, exist_ok=True)
    for out, extra in ((RUNNER_LIB, ["-shared", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden"]),
                       (RUNNER_TOOL, ["-DFDPLAN_MAIN"])):
        if force or _newer(src, out, []):
            rc, log_text = _compile([nvcc] + common + extra + ["-o", out, src],
                                    os.path.join(OBJ_DIR, os.path.basename(out) + ".log"))
            if verbose or rc != 0:
                print(log_text)
            if rc != 0:
                raise RuntimeError(f"building {os.path.basename(out)} failed")
    return RUNNER_LIB


def build_all(verbose: bool = False, force: bool = False) -> None:
    build_runner(verbose=verbose, force=force)
    build_kernels(verbose=verbose, force=force)
    build_cpu(verbose=verbose, force=force)
    build_capi(verbose=verbose, force=force)


if __name__ == "__main__":
    if "--mode" in sys.argv:
        print("built:", build_variant(sys.argv[sys.argv.index("--mode") + 1], verbose="-v" in sys.argv,
                                      force="-f" in sys.argv))
    else:
        build_all(verbose="-v" in sys.argv, force="-f" in sys.argv)
        print("built:", KERNEL_LIB, CPU_LIB if os.path.exists(CPU_LIB) else "")
