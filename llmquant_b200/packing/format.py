"""The single-file container, byte-compatible with llmquant/packing/format.py:29-118.

    b"LLMQUANT" | u64 little-endian header length | JSON header | tensor bytes

The JSON header is {"version": 1, "meta": {...}, "tensors": {name: {dtype, shape, offset,
nbytes}}}; offsets count from the first byte after the header and every tensor starts on a
64-byte multiple of that origin. bfloat16 payloads are the raw 16-bit patterns.
"""

import json
import mmap
import struct
from pathlib import Path

import numpy as np
import torch

MAGIC = b"LLMQUANT"
VERSION = 1
ALIGNMENT = 64
HEADER_LENGTH_BYTES = 8

_NUMPY_OF = {"uint8": np.uint8, "int8": np.int8, "float32": np.float32, "bfloat16": np.uint16}


def _payload(tensor: torch.Tensor) -> bytes:
    host = tensor.detach().cpu().contiguous()
    if host.dtype == torch.bfloat16:
        host = host.view(torch.uint16)
    return host.numpy().tobytes()


def write_packed(path, tensors: dict, meta: dict) -> Path:
    path = Path(path)
    path.parent.mkdir(parents=True, exist_ok=True)
    entries, cursor, chunks = {}, 0, []
    for name, tensor in tensors.items():
        gap = -cursor % ALIGNMENT
        if gap:
            chunks.append(bytes(gap))
            cursor += gap
        data = _payload(tensor)
        entries[name] = {
            "dtype": str(tensor.dtype).removeprefix("torch."),
            "shape": list(tensor.shape),
            "offset": cursor,
            "nbytes": len(data),
        }
        chunks.append(data)
        cursor += len(data)
    header = json.dumps({"version": VERSION, "meta": meta, "tensors": entries}).encode("utf-8")
    with open(path, "wb") as out:
        out.write(MAGIC + struct.pack("<Q", len(header)) + header)
        out.writelines(chunks)
    return path


def _read_prefix(handle):
    if handle.read(len(MAGIC)) != MAGIC:
        raise ValueError(f"{handle.name} is not a llmquant weight file")
    (length,) = struct.unpack("<Q", handle.read(HEADER_LENGTH_BYTES))
    header = json.loads(handle.read(length).decode("utf-8"))
    if header["version"] != VERSION:
        raise ValueError(f"unsupported file version {header['version']}, expected {VERSION}")
    return header, len(MAGIC) + HEADER_LENGTH_BYTES + length


def read_header(path) -> dict:
    with open(path, "rb") as handle:
        return _read_prefix(handle)[0]


def _tensor_from(view, entry) -> torch.Tensor:
    if entry["dtype"] not in _NUMPY_OF:
        raise ValueError(f"unsupported tensor dtype {entry['dtype']!r} in packed file")
    raw = view[entry["offset"]: entry["offset"] + entry["nbytes"]]
    array = np.frombuffer(raw, dtype=_NUMPY_OF[entry["dtype"]]).copy()
    tensor = torch.from_numpy(array)
    if entry["dtype"] == "bfloat16":
        tensor = tensor.view(torch.bfloat16)
    return tensor.reshape(entry["shape"])


def read_packed(path):
    """(tensors, meta). The file is mapped, each tensor copied out once."""
    with open(path, "rb") as handle:
        header, data_start = _read_prefix(handle)
        if not header["tensors"]:
            return {}, header["meta"]
        with mmap.mmap(handle.fileno(), 0, access=mmap.ACCESS_READ) as mapped:
            view = memoryview(mapped)[data_start:]
            try:
                tensors = {name: _tensor_from(view, entry) for name, entry in header["tensors"].items()}
            finally:
                view.release()
    return tensors, header["meta"]
