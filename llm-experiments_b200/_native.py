"""ctypes binding of ``libb2kv.so``, the C-ABI CUDA library (declared in include/b2kv.h).

The library is the only compute path of this package.  If it is missing the import of
this module fails with instructions to build it: there is no CPU or PyTorch fallback.
"""
from __future__ import annotations

import ctypes
import pathlib

_PKG = pathlib.Path(__file__).resolve().parent
LIB_PATH = _PKG / "libb2kv.so"

DTYPE_F32 = 0
DTYPE_BF16 = 1

ERR_BAD_ARG = -1
ERR_ALIGN = -2
ERR_UNSUPPORTED = -3
ERR_WORKSPACE = -4
ERR_CUDA = -5
ERR_STATIC_LIMIT = -6
STATIC_SCRATCH_BYTES = 32 << 20

DEV_STATUS_TEXT = {
    1: "a block-table entry points outside the pool",
    2: "an append position lies outside the cache",
    3: "a bounded wait on a barrier ran out",
    4: "a token id lies outside the embedding table",
}

_vp = ctypes.c_void_p
_i = ctypes.c_int
_i64 = ctypes.c_int64
_sz = ctypes.c_size_t

# name -> (restype, argtypes); kept in the order of include/b2kv.h
SIGNATURES = {
    "b2kv_strerror": (ctypes.c_char_p, [_i]),
    "b2kv_last_cuda_error": (ctypes.c_char_p, []),
    "b2kv_version": (_i, []),
    "b2kv_append": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i64, _i64, _i64, _i, _vp, _vp]),
    "b2kv_append_paged": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _vp, _i, _i, _i, _i, _i, _i, _i64, _i64, _i64, _i,
                               _vp, _vp]),
    "b2kv_append_rows_paged": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _i, _i64, _i64, _i64, _i, _vp, _vp]),
    "b2kv_advance_lengths": (_i, [_vp, _i, _i, _vp]),
    "b2kv_gather": (_i, [_vp, _vp, _vp, _i, _i, _i, _i, _i, _i64, _i64, _i64, _i, _vp]),
    "b2kv_gather_paged": (_i, [_vp, _vp, _vp, _i, _vp, _i, _i, _i, _i, _i, _i, _i, _i64, _i64, _i64, _i, _vp, _vp]),
    "b2kv_decode_workspace_bytes": (_sz, [_i, _i, _i, _i, _i]),
    "b2kv_decode": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i64, _i64, _i64, _i, _vp, _sz, _vp, _vp]),
    "b2kv_decode_paged": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _vp, _i, _i, _i, _i, _i, _i, _i, _i64, _i64, _i64,
                               _i, _vp, _sz, _vp, _vp]),
    "b2kv_decode_allgather": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i64, _i64, _i64, _i, _vp, _sz, _vp, _vp,
                                   _vp, _vp, ctypes.c_uint32, _i, _i, _i, ctypes.c_uint32, _vp, _vp]),
    "b2kv_decode_partial": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i64, _i64, _i64, _i, _vp, _sz, _vp,
                                 _vp]),
    "b2kv_merge_partials": (_i, [_vp, _i, _i, _i, _i, _vp, _i, _vp]),
    "b2kv_decode_static": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i64, _i64, _i64, _i, _vp, _vp]),
    "b2kv_prefill": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i, _i, _i, _i, _i, _i, _vp, _vp]),
    "b2kv_prefill_workspace_bytes": (_sz, [_i, _i, _i, _i, _i]),
    "b2kv_prefill_ws": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i, _i, _i, _i, _i, _i, _vp, _sz,
                             _vp, _vp]),
    "b2kv_prefill_paged": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i64, _i64, _i64, _i, _i, _i, _i, _i,
                                _vp, _vp]),
    "b2kv_layernorm": (_i, [_vp, _vp, _vp, _vp, _i64, _i, ctypes.c_float, _vp]),
    "b2kv_layernorm_bf16": (_i, [_vp, _vp, _vp, _vp, _i64, _i, ctypes.c_float, _vp]),
    "b2kv_extract_last_tokens": (_i, [_vp, _vp, _i, _i, _i, _vp]),
    "b2kv_softmax": (_i, [_vp, _vp, _i64, _i, _vp]),
    "b2kv_argmax": (_i, [_vp, _vp, _i, _i, _vp]),
    "b2kv_extract_last_tokens_bf16": (_i, [_vp, _vp, _i, _i, _i, _vp]),
    "b2kv_argmax_bf16": (_i, [_vp, _vp, _i, _i, _vp]),
    "b2kv_embedding": (_i, [_vp, _vp, _vp, _vp, _i, _vp, _i, _i, _i, _i, _i, _i, _vp, _vp]),
    "b2kv_qkv_append": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i64, _i64, _i64, _i, _vp, _vp]),
    "b2kv_matmul_rows": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _vp]),
    "b2kv_matmul": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _vp, _vp]),
    "b2kv_tune": (_i, [ctypes.c_char_p, _i]),
}


class B2KVError(RuntimeError):
    """A C-ABI call returned a negative status."""

    def __init__(self, status: int, text: str):
        super().__init__(f"b2kv error {status}: {text}")
        self.status = status


def _load() -> ctypes.CDLL:
    if not LIB_PATH.exists():
        raise ImportError(
            f"{LIB_PATH} is missing. Build the CUDA library first: "
            f"`python {_PKG.name}/build.py` (needs nvcc with sm_100a support). "
            "This package has no CPU fallback."
        )
    lib = ctypes.CDLL(str(LIB_PATH))
    for name, (restype, argtypes) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError here means header and library disagree
        fn.restype = restype
        fn.argtypes = argtypes
    return lib


lib = _load()


def check(status: int) -> None:
    """Raise for a negative status of a C-ABI call."""
    if status == 0:
        return
    text = lib.b2kv_strerror(status).decode()
    if status == ERR_CUDA:
        text += ": " + lib.b2kv_last_cuda_error().decode()
    raise B2KVError(status, text)


def tune(name: str, value: int) -> None:
    check(lib.b2kv_tune(name.encode(), int(value)))
