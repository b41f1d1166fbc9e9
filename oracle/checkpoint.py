"""CPU restatement of the reference's NVFP4 checkpoint container (test infrastructure only).

Only the test-suite may import this module.  `write_checkpoint` follows
src/checkpoint/format/writer.rs:15-38 (header: magic, u32 version, u32 tensor count; per tensor: u32 name_len,
u64 len, u64 byte_len, u64 scale_len, f32 global_scale, name, bytes, scales; all little-endian) with the constants
of src/checkpoint/format.rs:7-8; `read_checkpoint` follows src/checkpoint/format/reader.rs:22-67 and raises the
reference's two header errors; `validate_for_upload` is src/checkpoint/load/tensor.rs:27-39.

Parity pinned by: the reference's repository holds no checkpoint file and no test of the format; the byte layout
above is read from the two source files, which are unambiguous (fixed-width little-endian fields in a fixed
order).
"""
from __future__ import annotations

import struct
from typing import List, Tuple

MAGIC = b"GPT2_NVFP4_CHECKPOINT\n"  # format.rs:7
VERSION = 2                         # format.rs:8

Tensor = Tuple[str, int, float, bytes, bytes]  # name, len, global_scale, bytes, scales


def write_checkpoint(tensors: List[Tensor]) -> bytes:
    out = [MAGIC, struct.pack("<I", VERSION), struct.pack("<I", len(tensors))]       # writer.rs:15-19
    for name, length, global_scale, data, scales in tensors:                        # writer.rs:21-38
        raw = name.encode("utf-8")
        out.append(struct.pack("<I", len(raw)))
        out.append(struct.pack("<Q", length))
        out.append(struct.pack("<Q", len(data)))
        out.append(struct.pack("<Q", len(scales)))
        out.append(struct.pack("<f", global_scale))
        out.append(raw)
        out.append(bytes(data))
        out.append(bytes(scales))
    return b"".join(out)


def read_checkpoint(blob: bytes) -> List[Tensor]:
    pos = len(MAGIC)
    if blob[:pos] != MAGIC:                                                         # reader.rs:25-27
        raise ValueError("invalid GPT2 NVFP4 checkpoint magic")
    (version,) = struct.unpack_from("<I", blob, pos)
    pos += 4
    if version != VERSION:                                                          # reader.rs:30-32
        raise ValueError(f"unsupported checkpoint version {version}")
    (count,) = struct.unpack_from("<I", blob, pos)
    pos += 4
    tensors = []
    for _ in range(count):                                                          # reader.rs:37-66
        name_len, length, byte_len, scale_len, global_scale = struct.unpack_from("<IQQQf", blob, pos)
        pos += struct.calcsize("<IQQQf")
        name = blob[pos:pos + name_len].decode("utf-8")
        pos += name_len
        data = blob[pos:pos + byte_len]
        pos += byte_len
        scales = blob[pos:pos + scale_len]
        pos += scale_len
        if len(data) != byte_len or len(scales) != scale_len:
            raise ValueError("truncated checkpoint")
        tensors.append((name, length, global_scale, data, scales))
    return tensors


def validate_for_upload(tensor: Tensor) -> None:
    name, length, _, data, scales = tensor                                          # load/tensor.rs:27-39
    if len(data) != length // 2:
        raise ValueError(f"{name} has {len(data)} bytes; expected {length // 2}")
    if len(scales) != length // 16:
        raise ValueError(f"{name} has {len(scales)} scales; expected {length // 16}")
