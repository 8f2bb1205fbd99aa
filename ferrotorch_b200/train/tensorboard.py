"""Minimal TensorBoard event writer: TFRecord framing + masked CRC32C + hand-encoded ``Event``
protobufs, like the reference's writer (ferrotorch-train/src/tensorboard.rs:314-418)."""
from __future__ import annotations

import os
import socket
import struct
import time

_CRC_TABLE = []
for _i in range(256):
    _c = _i
    for _ in range(8):
        _c = (_c >> 1) ^ 0x82F63B78 if _c & 1 else _c >> 1
    _CRC_TABLE.append(_c)


def crc32c(data: bytes) -> int:
    c = 0xFFFFFFFF
    for b in data:
        c = _CRC_TABLE[(c ^ b) & 0xFF] ^ (c >> 8)
    return c ^ 0xFFFFFFFF


def masked_crc(data: bytes) -> int:
    c = crc32c(data)
    return (((c >> 15) | (c << 17)) + 0xA282EAD8) & 0xFFFFFFFF


def _varint(n: int) -> bytes:
    out = bytearray()
    while True:
        b = n & 0x7F
        n >>= 7
        if n:
            out.append(b | 0x80)
        else:
            out.append(b)
            return bytes(out)


def _field(num: int, wire: int, payload: bytes) -> bytes:
    return _varint((num << 3) | wire) + payload


def _bytes_field(num: int, b: bytes) -> bytes:
    return _field(num, 2, _varint(len(b)) + b)


def encode_scalar_event(tag: str, value: float, step: int, wall_time: float) -> bytes:
    """Event{wall_time=1 (double), step=2 (int64), summary=5{value=1{tag=1, simple_value=2 (float)}}}."""
    val = _bytes_field(1, tag.encode()) + _field(2, 5, struct.pack("<f", value))
    summary = _bytes_field(1, val)
    return _field(1, 1, struct.pack("<d", wall_time)) + _field(2, 0, _varint(step)) + _bytes_field(5, summary)


def encode_file_version_event(wall_time: float) -> bytes:
    return _field(1, 1, struct.pack("<d", wall_time)) + _bytes_field(3, b"brain.Event:2")


def record(data: bytes) -> bytes:
    hdr = struct.pack("<Q", len(data))
    return hdr + struct.pack("<I", masked_crc(hdr)) + data + struct.pack("<I", masked_crc(data))


def read_records(path: str) -> list[bytes]:
    out = []
    with open(path, "rb") as f:
        buf = f.read()
    p = 0
    while p < len(buf):
        (n,) = struct.unpack_from("<Q", buf, p)
        hdr = buf[p:p + 8]
        (hc,) = struct.unpack_from("<I", buf, p + 8)
        data = buf[p + 12:p + 12 + n]
        (dc,) = struct.unpack_from("<I", buf, p + 12 + n)
        if hc != masked_crc(hdr) or dc != masked_crc(data):
            raise ValueError("corrupt TFRecord at offset %d" % p)
        out.append(data)
        p += 16 + n
    return out


class TensorBoardWriter:
    def __init__(self, log_dir: str):
        os.makedirs(log_dir, exist_ok=True)
        self._log_dir = log_dir
        self.path = os.path.join(log_dir, "events.out.tfevents.%d.%s" % (int(time.time()), socket.gethostname()))
        self._f = open(self.path, "wb")
        self._f.write(record(encode_file_version_event(time.time())))

    def log_dir(self) -> str:
        return self._log_dir

    def add_scalar(self, tag: str, value: float, step: int) -> None:
        self._f.write(record(encode_scalar_event(tag, float(value), int(step), time.time())))

    def add_scalars(self, main_tag: str, values: dict, step: int) -> None:
        for k, v in values.items():
            self.add_scalar("%s/%s" % (main_tag, k), v, step)

    def flush(self) -> None:
        self._f.flush()

    def close(self) -> None:
        self._f.close()
