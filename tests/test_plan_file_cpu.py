"""Host-side pieces of the plan file writer: which bytes of a descriptor are device addresses."""
import ctypes

from fastdeploy_b200.runtime.plan_file import MAGIC, _pointer_slots


def test_pointer_slots_cover_pointer_fields_and_pointer_arrays_only():
    class D(ctypes.Structure):
        _fields_ = [("a", ctypes.c_void_p), ("n", ctypes.c_int), ("tab", ctypes.c_void_p * 3), ("f", ctypes.c_float),
                    ("ints", ctypes.c_longlong * 4), ("z", ctypes.c_void_p)]
    d = D()
    slots = _pointer_slots(d)
    assert slots == [D.a.offset, D.tab.offset, D.tab.offset + 8, D.tab.offset + 16, D.z.offset]
    assert all(s % 8 == 0 for s in slots) and D.ints.offset not in slots
    assert MAGIC == b"FDPLAN1\x00" and len(MAGIC) == 8


def test_every_native_descriptor_type_is_covered():
    """The descriptors the op wrappers fill are plain structures of scalars, pointers and arrays of them: nothing a
    plan file could not carry (no nested structures, no unions, no pointers hidden in integer fields by type)."""
    from fastdeploy_b200.ops import conv_gemm, generic, nhwc, nms, preproc, stem_conv, transformer
    seen = 0
    for mod in (conv_gemm, generic, nhwc, nms, preproc, stem_conv, transformer):
        for name in dir(mod):
            obj = getattr(mod, name)
            if isinstance(obj, type) and issubclass(obj, ctypes.Structure) and obj is not ctypes.Structure:
                seen += 1
                for fname, ctype in obj._fields_:
                    base = ctype._type_ if isinstance(ctype, type) and issubclass(ctype, ctypes.Array) else ctype
                    assert base in (ctypes.c_void_p, ctypes.c_int, ctypes.c_uint, ctypes.c_longlong, ctypes.c_ulonglong,
                                    ctypes.c_float, ctypes.c_double, ctypes.c_ubyte, ctypes.c_char), (name, fname, base)
    assert seen >= 7
