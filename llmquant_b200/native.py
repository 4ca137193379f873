"""ctypes binding of libllmquant_b200.so (the C ABI in include/llmquant_b200.h).

The library is built offline by `python -m llmquant_b200.build`; there is no JIT and no
fallback. Loading fails loudly if the shared object is missing, and every non-zero status
from the library is raised as a RuntimeError carrying the library's message.
"""

import ctypes
import functools
import os
import pathlib
import re

import torch

PKG = pathlib.Path(__file__).resolve().parent
# LLMQUANT_B200_LIBRARY points at another build of the same sources (a diagnostic build, say)
LIB_PATH = pathlib.Path(os.environ.get("LLMQUANT_B200_LIBRARY") or PKG / "libllmquant_b200.so")
HEADER = PKG.parent / "include" / "llmquant_b200.h"

LQ_F32, LQ_F16, LQ_BF16 = 0, 1, 2
GEMM_FOLD_SCALES, GEMM_SERIAL = 1, 2  # lq_wq_gemm_prefill flags
ATTN_AUTO, ATTN_SIMT, ATTN_MMA, ATTN_CLUSTER = 0, 1, 2, 3  # lq_attn_decode_fused impl
DTYPE_ID = {torch.float32: LQ_F32, torch.float16: LQ_F16, torch.bfloat16: LQ_BF16}

_P, _I, _L = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64
_IP = ctypes.POINTER(ctypes.c_int)

# name -> argtypes; every function returns int status unless listed in _RESTYPE
_SIGNATURES = {
    "lq_version": [],
    "lq_last_error": [],
    "lq_fake_quant_group": [_P, _P, _P, _L, _I, _I, _I, _P],
    "lq_quantize_group_i8": [_P, _P, _P, _L, _I, _I, _I, _P],
    "lq_quantize_weight": [_P, _I, _I, _I, _I, _I, _I, _I, _P, _P, _P],
    "lq_residual_add": [_P, _P, _P, _L, _I, _P],
    "lq_gemm_device_error": [],
    "lq_wq_gemm_prefill": [_P, _I, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _P],
    "lq_allreduce_max_world": [],
    "lq_allreduce_device_error": [],
    "lq_allreduce_residual": [_P, _I, _I, _I, _L, _L, _P, _P, _P, _I, _L, _I, _P],
    "lq_pack_int4": [_P, _P, _L, _P],
    "lq_unpack_int4": [_P, _P, _L, _P],
    "lq_dequant_weight": [_P, _P, _P, _I, _I, _I, _I, _I, _P],
    "lq_wq_gemv": [_P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _P],
    "lq_stream_layout_sizes": [_I, _I, _I, _I, _I, _IP, _IP, _IP],
    "lq_gemv_device_error": [],
    "lq_embed_gather": [_P, _P, _P, _I, _I, ctypes.c_int64, _I, _P],
    "lq_next_token": [_P, ctypes.c_int64, _P, _P, _P, ctypes.c_int64, _P, _I, _I, _P],
    "lq_wq_gemv_batched_max_rows": [],
    "lq_wq_gemv_batched": [_P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _P],
    "lq_gemv_tensor_core_ok": [_I, _I, _I, _I],
    "lq_repack_stream": [_P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _P],
    "lq_unrepack_stream": [_P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _P],
    "lq_dequant_stream": [_P, _P, _P, _I, _I, _I, _I, _I, _I, _P],
    "lq_wq_gemv_stream": [_P, _I, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _P],
}
_SIGNATURES.update({
    "lq_kv_write": [_P, _P, _P, _P, _I, _P, _P, _P, _P, _I, _I, _I, _I, _I, _P, _L, _I, _P],
    "lq_kv_dequant": [_P, _P, _P, _I, _I, _I, _I, _I, _I, _P],
    "lq_rope_kv_write": [_P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _P, _L, _I, _I, _P],
    "lq_attn_decode_scratch_bytes": [_I, _I, _I, _I],
    "lq_attn_decode_kv_i8": [_P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _P, _L, _I,
                             ctypes.c_float, _I, _I, _P],
})
_SIGNATURES.update({
    "lq_attn_decode_static_scratch_bytes": [],
    "lq_attn_fused_scratch_bytes": [_I, _I, _I, _I, _I],
    "lq_attn_device_error": [],
    "lq_attn_decode_fused": [_P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _P, _L, _I,
                             ctypes.c_float, _I, _I, _I, _P],
    "lq_attn_decode_kv_i8_static": [_P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _P, _L, _I,
                                    ctypes.c_float, _I, _I, _P],
})
_RESTYPE = {"lq_last_error": ctypes.c_char_p, "lq_attn_decode_scratch_bytes": ctypes.c_int64,
            "lq_attn_decode_static_scratch_bytes": ctypes.c_int64,
            "lq_attn_fused_scratch_bytes": ctypes.c_int64,
            "lq_decode_gemm_workspace_bytes": ctypes.c_int64, "lq_tile_weight_bytes": ctypes.c_int64}


class GemvArgs(ctypes.Structure):
    """Mirror of `lq_gemv_args` (include/llmquant_b200.h)."""

    _fields_ = [
        ("x", _P), ("ldx", _I), ("norm_weight", _P), ("norm_eps", ctypes.c_float),
        ("codes", _P), ("scale_tiles", _P), ("bias", _P), ("residual", _P), ("out", _P),
        ("out_dtype", _I), ("M", _I), ("N", _I), ("K", _I), ("Kd", _I), ("span", _I),
        ("bits", _I), ("epilogue", _I), ("variant", _I), ("pdl", _I), ("tp", _P), ("ldo", _I),
        ("workspace", _P), ("workspace_bytes", _L),
    ]


class GemvTp(ctypes.Structure):
    """Mirror of `lq_gemv_tp` (include/llmquant_b200.h)."""

    _fields_ = [
        ("mode", _I), ("world", _I), ("rank", _I), ("peers", _P), ("data_offset", _L),
        ("parts", _P), ("residual", _P), ("wait_cycles", _L),
    ]


TP_PUSH, TP_SUM = 1, 2

_SIGNATURES["lq_wq_gemv_fused"] = [ctypes.POINTER(GemvArgs), _P]
_SIGNATURES["lq_glue_device_error"] = []
_SIGNATURES["lq_decode_gemm_device_error"] = []
_SIGNATURES["lq_decode_gemm_workspace_bytes"] = [_I, _I, _I]
_SIGNATURES["lq_tile_weight_bytes"] = [_I, _I, _I]
_SIGNATURES["lq_tile_weight"] = [_P, _P, _P, _I, _I, _I, _P]
_SIGNATURES["lq_next_token_tp"] = [_P, _L, _I, _I, _P, _L, _I, _P, _P, _P, _L, _P, _P, _I, _L, _I, _P]


def declared_symbols(header: pathlib.Path = HEADER):
    """Every function name the public header declares."""
    text = re.sub(r"/\*.*?\*/", "", header.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(lq_[a-z0-9_]+)\s*\(", text)))


@functools.lru_cache(maxsize=1)
def library() -> ctypes.CDLL:
    if not LIB_PATH.exists():
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m llmquant_b200.build` "
            "(the CUDA kernels are compiled offline; there is no fallback path)"
        )
    lib = ctypes.CDLL(str(LIB_PATH))
    for name, argtypes in _SIGNATURES.items():
        fn = getattr(lib, name)
        fn.argtypes = argtypes
        fn.restype = _RESTYPE.get(name, ctypes.c_int)
    return lib


def last_error() -> str:
    msg = library().lq_last_error()
    return msg.decode("utf-8", "replace") if msg else ""


def check(status: int):
    if status:
        raise RuntimeError(last_error() or f"libllmquant_b200 returned status {status}")


def stream_ptr(device=None) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def ptr(t) -> int:
    return 0 if t is None else t.data_ptr()


def call(name: str, *args):
    """Invoke one entry point and raise on a non-zero status."""
    check(getattr(library(), name)(*args))


def stream_layout_sizes(n, groups, group_size, head_dim, bits):
    """(Kd, span, NP) of the streaming layout for a canonical [n, groups, group_size] weight."""
    kd, span, np_ = ctypes.c_int(), ctypes.c_int(), ctypes.c_int()
    call("lq_stream_layout_sizes", n, groups, group_size, head_dim or 0, bits,
         ctypes.byref(kd), ctypes.byref(span), ctypes.byref(np_))
    return kd.value, span.value, np_.value
