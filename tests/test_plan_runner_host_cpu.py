"""The plan runner built without a GPU (device memory = host memory) against a stand-in kernel library: a plan file
written by hand in the documented layout is read, relocated, run and read back; corrupt files are refused."""
import ctypes
import os
import shutil
import struct
import subprocess

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
pytestmark = pytest.mark.skipif(shutil.which("g++") is None, reason="no C++ compiler")


@pytest.fixture(scope="module")
def libs(tmp_path_factory):
    d = tmp_path_factory.mktemp("runner_host")
    src = d / "plan_runner_host.cc"
    shutil.copy(os.path.join(ROOT, "csrc", "runner", "plan_runner.cu"), src)
    runner, fake = str(d / "libfdb200_runner_host.so"), str(d / "libfake_kernels.so")
    subprocess.run(["g++", "-std=c++17", "-O1", "-DFDPLAN_HOST_ONLY", "-fPIC", "-shared", "-o", runner, str(src), "-ldl"],
                   check=True)
    subprocess.run(["g++", "-std=c++17", "-O1", "-fPIC", "-shared", "-o", fake, os.path.join(ROOT, "tests", "fake_kernels.cc")],
                   check=True)
    lib = ctypes.CDLL(runner)
    lib.fdplan_load.restype = ctypes.c_void_p
    lib.fdplan_load.argtypes = [ctypes.c_char_p, ctypes.c_char_p]
    lib.fdplan_last_error.restype = ctypes.c_char_p
    lib.fdplan_io_name.restype = ctypes.c_char_p
    lib.fdplan_io_name.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int]
    lib.fdplan_io_bytes.restype = ctypes.c_ulonglong
    lib.fdplan_io_bytes.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int]
    lib.fdplan_io_desc.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.POINTER(ctypes.c_int),
                                   ctypes.POINTER(ctypes.c_longlong)]
    for fn in ("fdplan_num_ops", "fdplan_num_inputs", "fdplan_num_outputs", "fdplan_run", "fdplan_destroy"):
        getattr(lib, fn).argtypes = [ctypes.c_void_p]
    lib.fdplan_set_input.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p, ctypes.c_ulonglong]
    lib.fdplan_get_output.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p, ctypes.c_ulonglong]
    lib.fdplan_time.restype = ctypes.c_double
    lib.fdplan_time.argtypes = [ctypes.c_void_p, ctypes.c_int]
    lib._paths = (runner, fake)
    return lib, fake.encode()


def _plan_bytes():
    """x [4, 6] fp32 (input, rows padded to a pitch of 8) -> t = 2 x + 1 -> out = t + w + t (table of three addresses,
    one of them null) ; output `out` [4, 6] dense. Buffers: 0 x (pitch 8), 1 t, 2 w (constant), 3 out, 4 table."""
    n = 24
    w = np.arange(n, dtype=np.float32) * 0.5
    out = bytearray(b"FDPLAN1\0")
    bufs = [(4 * 8 * 4 + 64, None), (n * 4, None), (n * 4, w.tobytes()), (n * 4, None), (4 * 8, None)]
    out += struct.pack("<I", len(bufs))
    for size, data in bufs:
        out += struct.pack("<QB", size, 1 if data is not None else 0)
        if data is not None:
            out += data
    ops = []
    # the scale op reads the input through a dense copy made by a strided-copy op of the plan itself
    gen = bytearray(4 * 8 + 48 * 8 + 4 * 4)
    ints = [2, 2, 2, 4, 6, 0, 0, 0, 0, 8, 1, 0, 0, 0, 0, 6, 1, 0, 0, 0, 0]              # nd, dtypes, shape, strides
    struct.pack_into(f"<{len(ints)}q", gen, 32, *ints)
    ops.append((b"fdb_generic_create", 0, bytes(gen), [(0, 0, 64), (8, 3, 0)]))           # x (offset 64) -> out as scratch
    scale = struct.pack("<QQqff", 0, 0, n, 2.0, 1.0)
    ops.append((b"fdb_fake_scale_create", -1, scale, [(0, 3, 0), (8, 1, 0)]))            # t = 2 * dense(x) + 1
    tsum = struct.pack("<QiiQq", 0, 4, 0, 0, n)
    ops.append((b"fdb_fake_table_sum_create", 7, tsum, [(0, 4, 0), (16, 3, 0)]))         # out = table[0] + ... + table[3]
    out += struct.pack("<I", len(ops))
    for name, kind, desc, relocs in ops:
        out += struct.pack("<H", len(name)) + name + struct.pack("<iI", kind, len(desc)) + desc
        out += struct.pack("<I", len(relocs))
        for off, b, o in relocs:
            out += struct.pack("<IIQ", off, b, o)
    out += struct.pack("<I", 1)                                                           # one pointer table
    out += struct.pack("<IQI", 4, 0, 4)
    for b, o in ((1, 0), (2, 0), (-1, 0), (1, 0)):                                        # t, w, null, t
        out += struct.pack("<iQ", b, o)
    out += struct.pack("<I", 2)
    out += struct.pack("<BH", 0, 1) + b"x" + struct.pack("<IQBB", 0, 64, 2, 2) + struct.pack("<2q", 4, 6) + struct.pack("<2q", 8, 1)
    out += struct.pack("<BH", 1, 3) + b"out" + struct.pack("<IQBB", 3, 0, 2, 2) + struct.pack("<2q", 4, 6) + struct.pack("<2q", 6, 1)
    return bytes(out), w


def test_hand_written_plan_is_relocated_run_and_read_back(libs, tmp_path):
    lib, fake = libs
    blob, w = _plan_bytes()
    path = tmp_path / "toy.fdplan"
    path.write_bytes(blob)
    h = lib.fdplan_load(str(path).encode(), fake)
    assert h, lib.fdplan_last_error().decode()
    assert (lib.fdplan_num_ops(h), lib.fdplan_num_inputs(h), lib.fdplan_num_outputs(h)) == (3, 1, 1)
    assert lib.fdplan_io_name(h, 0, 0) == b"x" and lib.fdplan_io_name(h, 1, 0) == b"out"
    dt, dims = ctypes.c_int(), (ctypes.c_longlong * 8)()
    assert lib.fdplan_io_desc(h, 0, 0, ctypes.byref(dt), dims) == 2 and dt.value == 2 and list(dims[:2]) == [4, 6]
    assert lib.fdplan_io_bytes(h, 0, 0) == 96 and lib.fdplan_io_bytes(h, 1, 0) == 96
    for seed in (0, 1, 2):                                   # three runs: eager, then whatever replay the build has
        x = np.random.default_rng(seed).standard_normal((4, 6)).astype(np.float32)
        assert lib.fdplan_set_input(h, 0, x.ctypes.data, x.nbytes) == 0
        assert lib.fdplan_run(h) == 0, lib.fdplan_last_error().decode()
        got = np.empty((4, 6), np.float32)
        assert lib.fdplan_get_output(h, 0, got.ctypes.data, got.nbytes) == 0
        t = 2 * x.reshape(-1) + 1
        assert np.allclose(got.reshape(-1), t + w + t)
    assert lib.fdplan_set_input(h, 0, x.ctypes.data, 8) != 0 and b"96 bytes" in lib.fdplan_last_error()
    assert lib.fdplan_set_input(h, 3, x.ctypes.data, 96) != 0
    assert lib.fdplan_time(h, 3) >= 0.0
    lib.fdplan_destroy(h)


def test_corrupt_plan_files_are_refused_not_followed(libs, tmp_path):
    lib, fake = libs
    blob, _ = _plan_bytes()
    cases = {"truncated": blob[:len(blob) // 2], "tail_cut": blob[:-5], "bad_magic": b"FDPLAN9\0" + blob[8:]}
    # a relocation that points past its buffer, and one that points past its descriptor
    first_reloc = blob.index(b"fdb_generic_create") + len(b"fdb_generic_create") + 8 + (4 * 8 + 48 * 8 + 16) + 4
    bad_buffer = bytearray(blob)
    struct.pack_into("<IIQ", bad_buffer, first_reloc, 0, 0, 1 << 40)
    cases["reloc_outside_buffer"] = bytes(bad_buffer)
    bad_desc = bytearray(blob)
    struct.pack_into("<IIQ", bad_desc, first_reloc, 1 << 20, 0, 64)
    cases["reloc_outside_descriptor"] = bytes(bad_desc)
    unknown = blob.replace(b"fdb_fake_scale_create", b"fdb_fake_scale_creatX")
    cases["unknown_creation_function"] = unknown
    for name, data in cases.items():
        p = tmp_path / f"{name}.fdplan"
        p.write_bytes(data)
        h = lib.fdplan_load(str(p).encode(), fake)
        assert not h, name
        assert len(lib.fdplan_last_error()) > 0, name


def test_python_front_of_the_runner(libs, tmp_path):
    from fastdeploy_b200.runtime.plan_runner import PlanRunner
    lib, _ = libs
    runner_path, fake_path = lib._paths
    blob, w = _plan_bytes()
    path = tmp_path / "toy.fdplan"
    path.write_bytes(blob)
    with PlanRunner(str(path), kernels_lib=fake_path, runner_lib=runner_path) as r:
        assert r.num_ops == 3 and [t.name for t in r.inputs] == ["x"] and r.outputs[0].shape == [4, 6]
        assert r.inputs[0].dtype == "float32" and "x" in repr(r.inputs[0])
        x = np.arange(24, dtype=np.float64).reshape(4, 6)                  # converted to the plan's float32
        out = r.infer({"x": x})[0]
        t = 2 * x.reshape(-1) + 1
        assert out.dtype == np.float32 and np.allclose(out.reshape(-1), t + w + t)
        out2 = r.infer([x.astype(np.float32) * 0])[0]
        assert np.allclose(out2.reshape(-1), 2 + w)
        with pytest.raises(ValueError):
            r.set_input("x", np.zeros((2, 2), np.float32))
        with pytest.raises(KeyError):
            r.set_input("nope", x)
        assert r.time(2) >= 0.0
    with pytest.raises(FileNotFoundError):
        PlanRunner(str(tmp_path / "absent.fdplan"), kernels_lib=fake_path, runner_lib=runner_path)
    junk = tmp_path / "junk.fdplan"
    junk.write_bytes(b"nope")
    with pytest.raises(RuntimeError, match="not a plan file"):
        PlanRunner(str(junk), kernels_lib=fake_path, runner_lib=runner_path)
