import base64
import hashlib

import numpy as np
import pytest

from fastdeploy_b200 import encryption as E


def test_round_trip_and_container_layout():
    key = E.generate_key()
    assert len(base64.b64decode(key)) == 32
    plain = bytes(range(256)) * 7
    blob = E.encrypt_bytes(plain, key)
    assert blob[:6] == b"PADDLE" and blob[6:7] == b"1"
    assert blob[7:71] == hashlib.sha256(base64.b64decode(key)).hexdigest().encode()
    assert len(blob) == 6 + 1 + 128 + len(plain) + 16
    assert E.decrypt_bytes(blob, key) == plain
    text, k2 = E.encrypt("hello model")
    assert E.decrypt(text, k2) == "hello model"


def test_wrong_key_and_tampering_are_detected():
    key, other = E.generate_key(), E.generate_key()
    blob = bytearray(E.encrypt_bytes(b"weights" * 100, key))
    with pytest.raises(E.EncryptionError, match="key does not match"):
        E.decrypt_bytes(bytes(blob), other)
    blob[200] ^= 1
    with pytest.raises(E.EncryptionError, match="authentication failed"):
        E.decrypt_bytes(bytes(blob), key)
    with pytest.raises(E.EncryptionError):
        E.decrypt_bytes(b"not a model", key)
    with pytest.raises(E.EncryptionError, match="key length"):
        E.encrypt_bytes(b"x", base64.b64encode(b"short").decode())


def test_runtime_loads_an_encrypted_model(tmp_path):
    import fastdeploy_b200 as fd
    from fastdeploy_b200.core.types import ModelFormat
    from fastdeploy_b200.models.resnet import resnet18_like_onnx
    plain = str(tmp_path / "m.onnx")
    resnet18_like_onnx(plain, seed=1)
    key = E.generate_key()
    enc = str(tmp_path / "enc.onnx")
    E.encrypt_file(plain, enc, key)
    opt = fd.RuntimeOption(); opt.use_cpu(); opt.set_model_path(plain, "", ModelFormat.ONNX)
    rt0 = fd.Runtime(opt)
    info = rt0.get_input_info(0)
    shape = [d if isinstance(d, int) and d > 0 else 1 for d in info.shape]
    x = np.random.default_rng(0).standard_normal(shape).astype(np.float32)
    ref = rt0.infer({info.name: x})[0]
    opt2 = fd.RuntimeOption(); opt2.use_cpu(); opt2.set_model_path(enc, "", ModelFormat.ONNX); opt2.set_encryption_key(key)
    rt = fd.Runtime(opt2)
    out = rt.infer({info.name: x})[0]
    assert np.allclose(ref, out)
