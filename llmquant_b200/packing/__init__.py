"""The single-file format for a quantized model (`model.bin`)."""

from llmquant_b200.packing.format import read_header, read_packed, write_packed
from llmquant_b200.packing.model_io import (
    describe_packed,
    load_packed_model,
    packed_dtypes,
    save_packed_model,
)
from llmquant_b200.packing.packing import pack_int4, pack_weight, unpack_int4, unpack_weight

__all__ = [
    "describe_packed", "load_packed_model", "pack_int4", "pack_weight", "packed_dtypes",
    "read_header", "read_packed", "save_packed_model", "unpack_int4", "unpack_weight",
    "write_packed",
]
