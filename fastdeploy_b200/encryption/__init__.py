"""Model encryption (fastdeploy/encryption/src/{encrypt,decrypt}.cc, python/fastdeploy/encryption):
AES-256-GCM with the reference's container - ``"PADDLE"`` magic, version ``"1"``, a 128-byte tag whose
first 64 characters are the SHA-256 hex digest of the 32-byte key (the rest is random filler), then the
ciphertext with its 16-byte GCM tag. The key is 32 random bytes, base64; the IV is bytes 16..32 of the
key, as in the reference. ``encrypt`` / ``decrypt`` exchange base64 text like the reference's string API;
``encrypt_bytes`` / ``decrypt_bytes`` work on raw buffers (what ``Runtime`` uses for model files).
"""
from __future__ import annotations

import base64
import hashlib
import os
import secrets
import string
from typing import List, Tuple

MAGIC = b"PADDLE"
VERSION = b"1"
TAG_LEN = 128
KEY_LEN = 32
IV_LEN = 16
GCM_TAG_LEN = 16


class EncryptionError(ValueError):
    pass


def _aesgcm(key: bytes):
    from cryptography.hazmat.primitives.ciphers.aead import AESGCM
    return AESGCM(key)


def generate_key() -> str:
    """32 random bytes, base64 (``GenerateRandomKey``)."""
    return base64.b64encode(os.urandom(KEY_LEN)).decode()


def _key_bytes(key: str) -> bytes:
    try:
        raw = base64.b64decode(key.encode(), validate=True)
    except Exception as e:
        raise EncryptionError("key is not valid base64") from e
    if len(raw) != KEY_LEN:
        raise EncryptionError("key length abnormal: expected 32 bytes")
    return raw


def encrypt_bytes(plain: bytes, key: str) -> bytes:
    raw = _key_bytes(key)
    cipher = _aesgcm(raw).encrypt(raw[16:16 + IV_LEN], bytes(plain), None)
    digest = hashlib.sha256(raw).hexdigest().encode()          # 64 characters
    filler = "".join(secrets.choice(string.ascii_letters + string.digits) for _ in range(TAG_LEN - len(digest))).encode()
    return MAGIC + VERSION + digest + filler + cipher


def is_encrypted(blob: bytes) -> bool:
    return len(blob) >= len(MAGIC) + 1 + TAG_LEN + GCM_TAG_LEN and bytes(blob[:len(MAGIC)]) == MAGIC


def decrypt_bytes(blob: bytes, key: str) -> bytes:
    raw = _key_bytes(key)
    blob = bytes(blob)
    if not is_encrypted(blob):
        raise EncryptionError("not an encrypted model (magic number mismatch)")
    if blob[len(MAGIC):len(MAGIC) + 1] != VERSION:
        raise EncryptionError("unsupported container version")
    tag = blob[len(MAGIC) + 1:len(MAGIC) + 1 + TAG_LEN]
    if tag[:64] != hashlib.sha256(raw).hexdigest().encode():
        raise EncryptionError("key does not match the encrypted model")
    try:
        return _aesgcm(raw).decrypt(raw[16:16 + IV_LEN], blob[len(MAGIC) + 1 + TAG_LEN:], None)
    except Exception as e:
        raise EncryptionError("AES-GCM authentication failed") from e


def encrypt(input, key: str = "") -> List[str]:
    """``[base64(ciphertext container), key]``; a key is generated when none is given."""
    key = key or generate_key()
    data = input if isinstance(input, (bytes, bytearray)) else str(input).encode("latin-1")
    return [base64.b64encode(encrypt_bytes(bytes(data), key)).decode(), key]


def decrypt(cipher, key: str):
    """Inverse of :func:`encrypt`. Accepts the base64 text form (returns ``str`` through latin-1, the
    byte-preserving mapping) or the raw container bytes (returns ``bytes``)."""
    if isinstance(cipher, (bytes, bytearray)):
        blob = bytes(cipher)
        if not is_encrypted(blob):
            blob = base64.b64decode(blob)
        return decrypt_bytes(blob, key)
    return decrypt_bytes(base64.b64decode(cipher.encode()), key).decode("latin-1")


def encrypt_file(src: str, dst: str, key: str = "") -> str:
    key = key or generate_key()
    with open(src, "rb") as f:
        blob = encrypt_bytes(f.read(), key)
    with open(dst, "wb") as f:
        f.write(blob)
    return key
