"""ctypes front end of the C oracle (``kv_oracle.c``).  TEST INFRASTRUCTURE ONLY.

Arrays are numpy; bf16 data is passed as ``uint16`` bit patterns.  ``dtype`` is
0 for float32 and 1 for bf16 storage.  See ``kv_oracle.c`` for what each function
follows in the reference.
"""

from __future__ import annotations

import ctypes
import pathlib

import numpy as np

from . import build_oracle

_HERE = pathlib.Path(__file__).resolve().parent
_lib = None

_i32p = ctypes.POINTER(ctypes.c_int32)
_f32p = ctypes.POINTER(ctypes.c_float)


def lib():
    """Load (building first if the source is newer or the library is absent)."""
    global _lib
    if _lib is None:
        path = build_oracle.build()
        L = ctypes.CDLL(str(path))
        L.kvo_num_threads.restype = ctypes.c_int
        L.kvo_set_num_threads.argtypes = [ctypes.c_int]
        L.kvo_append.restype = None
        L.kvo_append.argtypes = [ctypes.c_void_p] * 4 + [_i32p, ctypes.c_int] + [ctypes.c_int] * 3 + [
            ctypes.c_int64] * 3 + [ctypes.c_int, _i32p, ctypes.c_int, ctypes.c_int, ctypes.c_int64]
        L.kvo_decode.restype = None
        L.kvo_decode.argtypes = [ctypes.c_void_p] * 3 + [_f32p, _i32p, ctypes.c_int] + [ctypes.c_int] * 3 + [
            ctypes.c_int64] * 3 + [ctypes.c_int, _i32p, ctypes.c_int, ctypes.c_int, ctypes.c_int64]
        L.kvo_prefill.restype = None
        L.kvo_prefill.argtypes = [ctypes.c_void_p] * 3 + [_f32p, _f32p, _f32p] + [ctypes.c_int] * 5
        _lib = L
    return _lib


def _ptr(a):
    return ctypes.c_void_p(a.ctypes.data)


def _i32(a):
    if a is None:
        return None, None
    a = np.ascontiguousarray(a, dtype=np.int32)
    return a, a.ctypes.data_as(_i32p)


def _dtype_code(a):
    if a.dtype == np.float32:
        return 0
    if a.dtype == np.uint16:
        return 1
    raise TypeError(f"oracle arrays must be float32 or uint16 (bf16 bits), got {a.dtype}")


def num_threads() -> int:
    return int(lib().kvo_num_threads())


def set_num_threads(n: int) -> None:
    lib().kvo_set_num_threads(int(n))


def append(new_k, new_v, k_cache, v_cache, pos, B, H, D, strides, block_table=None, block_size=0, stride_blk=0):
    """In-place append.  ``pos`` int or int32 [B]; ``strides = (sb, st, sh)`` in elements."""
    dt = _dtype_code(k_cache)
    assert new_k.flags.c_contiguous and new_v.flags.c_contiguous
    pos_keep, pos_p = (None, None) if np.isscalar(pos) else _i32(pos)
    bt_keep, bt_p = _i32(block_table)
    max_blocks = 0 if block_table is None else block_table.shape[1]
    lib().kvo_append(_ptr(new_k), _ptr(new_v), _ptr(k_cache), _ptr(v_cache), pos_p,
                     int(pos) if np.isscalar(pos) else 0, B, H, D, strides[0], strides[1], strides[2], dt,
                     bt_p, max_blocks, block_size, stride_blk)


def decode(q, k_cache, v_cache, lens, B, H, D, strides, block_table=None, block_size=0, stride_blk=0):
    """Returns float32 ``[B, H*D]``.  ``lens`` int or int32 [B]."""
    dt = _dtype_code(k_cache)
    assert _dtype_code(q) == dt and q.flags.c_contiguous
    out = np.empty((B, H * D), dtype=np.float32)
    lens_keep, lens_p = (None, None) if np.isscalar(lens) else _i32(lens)
    bt_keep, bt_p = _i32(block_table)
    max_blocks = 0 if block_table is None else block_table.shape[1]
    lib().kvo_decode(_ptr(q), _ptr(k_cache), _ptr(v_cache), out.ctypes.data_as(_f32p), lens_p,
                     int(lens) if np.isscalar(lens) else 0, B, H, D, strides[0], strides[1], strides[2], dt,
                     bt_p, max_blocks, block_size, stride_blk)
    return out


def prefill(Q, K, V, B, N, H, D, want_stats=True):
    """Returns ``(O [B*N, H*D], L [B*N*H], M [B*N*H])`` as float32."""
    dt = _dtype_code(Q)
    for a in (Q, K, V):
        assert a.flags.c_contiguous and _dtype_code(a) == dt
    O = np.empty((B * N, H * D), dtype=np.float32)
    L = np.empty(B * N * H, dtype=np.float32) if want_stats else None
    M = np.empty(B * N * H, dtype=np.float32) if want_stats else None
    lib().kvo_prefill(_ptr(Q), _ptr(K), _ptr(V), O.ctypes.data_as(_f32p),
                      L.ctypes.data_as(_f32p) if want_stats else None,
                      M.ctypes.data_as(_f32p) if want_stats else None, B, N, H, D, dt)
    return O, L, M
