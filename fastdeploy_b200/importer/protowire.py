"""Schema-driven protobuf wire-format codec (no protoc, no generated code).

A schema is ``{field_number: (name, kind, repeated)}`` where ``kind`` is one of
``int`` (varint, two's complement 64-bit), ``uint``, ``bool``, ``float`` (fixed32),
``double`` (fixed64), ``bytes``, ``str`` or a nested schema dict. Messages decode to
plain dicts; repeated fields decode to lists (packed and unpacked encodings are both
accepted). Unknown fields are skipped on decode and never emitted on encode.

Replaces the protobuf runtime that the reference links for ``.pdmodel`` and ONNX
parsing (paddle2onnx/parser/parser.cc:180-260, paddle2onnx/onnx_reader.cc).
"""
from __future__ import annotations

import struct
from typing import Any, Dict, Tuple, Union

Schema = Dict[int, Tuple[str, Any, bool]]

_MASK64 = (1 << 64) - 1


class WireError(ValueError):
    pass


def _read_varint(buf: bytes, pos: int) -> Tuple[int, int]:
    result = 0
    shift = 0
    while True:
        if pos >= len(buf):
            raise WireError("truncated varint")
        b = buf[pos]
        pos += 1
        result |= (b & 0x7F) << shift
        if not b & 0x80:
            return result, pos
        shift += 7
        if shift > 70:
            raise WireError("varint too long")


def _write_varint(out: bytearray, v: int) -> None:
    v &= _MASK64
    while True:
        b = v & 0x7F
        v >>= 7
        if v:
            out.append(b | 0x80)
        else:
            out.append(b)
            return


def _to_signed(v: int) -> int:
    return v - (1 << 64) if v & (1 << 63) else v


def _scalar_from_varint(kind: str, v: int):
    if kind == "int":
        return _to_signed(v)
    if kind == "bool":
        return bool(v)
    return v


def decode(buf: Union[bytes, bytearray, memoryview], schema: Schema) -> Dict[str, Any]:
    buf = bytes(buf)
    msg: Dict[str, Any] = {}
    for _, (name, _, rep) in schema.items():
        if rep:
            msg[name] = []
    pos, end = 0, len(buf)
    while pos < end:
        key, pos = _read_varint(buf, pos)
        fnum, wt = key >> 3, key & 7
        spec = schema.get(fnum)
        if wt == 0:
            v, pos = _read_varint(buf, pos)
            if spec is None:
                continue
            name, kind, rep = spec
            val = _scalar_from_varint(kind, v)
        elif wt == 1:
            if pos + 8 > end:
                raise WireError("truncated fixed64")
            raw = buf[pos:pos + 8]
            pos += 8
            if spec is None:
                continue
            name, kind, rep = spec
            val = struct.unpack("<d", raw)[0] if kind == "double" else struct.unpack("<q", raw)[0]
        elif wt == 5:
            if pos + 4 > end:
                raise WireError("truncated fixed32")
            raw = buf[pos:pos + 4]
            pos += 4
            if spec is None:
                continue
            name, kind, rep = spec
            val = struct.unpack("<f", raw)[0] if kind == "float" else struct.unpack("<i", raw)[0]
        elif wt == 2:
            ln, pos = _read_varint(buf, pos)
            if pos + ln > end:
                raise WireError("truncated length-delimited field")
            raw = buf[pos:pos + ln]
            pos += ln
            if spec is None:
                continue
            name, kind, rep = spec
            if isinstance(kind, dict):
                val = decode(raw, kind)
            elif kind == "bytes":
                val = raw
            elif kind == "str":
                val = raw.decode("utf-8", errors="replace")
            elif rep and kind in ("int", "uint", "bool"):
                p2 = 0
                while p2 < ln:
                    v, p2 = _read_varint(raw, p2)
                    msg[name].append(_scalar_from_varint(kind, v))
                continue
            elif rep and kind == "float":
                msg[name].extend(struct.unpack("<%df" % (ln // 4), raw))
                continue
            elif rep and kind == "double":
                msg[name].extend(struct.unpack("<%dd" % (ln // 8), raw))
                continue
            else:
                raise WireError(f"field {fnum}: length-delimited data for scalar kind {kind}")
        else:
            raise WireError(f"unsupported wire type {wt}")
        if rep:
            msg[name].append(val)
        else:
            msg[name] = val
    return msg


def _encode_scalar(out: bytearray, fnum: int, kind, val) -> None:
    if isinstance(kind, dict):
        body = encode(val, kind)
        _write_varint(out, (fnum << 3) | 2)
        _write_varint(out, len(body))
        out += body
    elif kind in ("int", "uint", "bool"):
        _write_varint(out, (fnum << 3) | 0)
        _write_varint(out, int(val))
    elif kind == "float":
        _write_varint(out, (fnum << 3) | 5)
        out += struct.pack("<f", val)
    elif kind == "double":
        _write_varint(out, (fnum << 3) | 1)
        out += struct.pack("<d", val)
    elif kind == "bytes":
        b = bytes(val)
        _write_varint(out, (fnum << 3) | 2)
        _write_varint(out, len(b))
        out += b
    elif kind == "str":
        b = val.encode("utf-8") if isinstance(val, str) else bytes(val)
        _write_varint(out, (fnum << 3) | 2)
        _write_varint(out, len(b))
        out += b
    else:
        raise WireError(f"unknown kind {kind}")


def encode(msg: Dict[str, Any], schema: Schema, packed: bool = True) -> bytes:
    out = bytearray()
    for fnum in sorted(schema):
        name, kind, rep = schema[fnum]
        if name not in msg or msg[name] is None:
            continue
        val = msg[name]
        if not rep:
            _encode_scalar(out, fnum, kind, val)
            continue
        if len(val) == 0:
            continue
        if packed and kind in ("int", "uint", "bool", "float", "double"):
            body = bytearray()
            if kind == "float":
                body += struct.pack("<%df" % len(val), *val)
            elif kind == "double":
                body += struct.pack("<%dd" % len(val), *val)
            else:
                for v in val:
                    _write_varint(body, int(v))
            _write_varint(out, (fnum << 3) | 2)
            _write_varint(out, len(body))
            out += body
        else:
            for v in val:
                _encode_scalar(out, fnum, kind, v)
    return bytes(out)
