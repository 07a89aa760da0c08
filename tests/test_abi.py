"""The C-ABI library: it loads without a GPU, exports every symbol that include/b2kv.h
declares with the declared number of arguments, and rejects bad arguments before touching
the device (so these checks run on a CPU-only machine)."""
import ctypes
import pathlib
import re

import pytest

ROOT = pathlib.Path(__file__).resolve().parent.parent
HEADER = ROOT / "include" / "b2kv.h"


def header_functions():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    decls = {}
    for m in re.finditer(r"\b([A-Za-z_][\w\s\*]*?)\b(b2kv_\w+)\s*\(([^;{]*?)\)\s*;", text, flags=re.S):
        args = m.group(3).strip()
        n = 0 if args in ("", "void") else len([a for a in args.split(",") if a.strip()])
        decls[m.group(2)] = n
    return decls


def test_header_declares_the_expected_entry_points():
    names = set(header_functions())
    for required in ["b2kv_append", "b2kv_append_paged", "b2kv_gather", "b2kv_gather_paged", "b2kv_decode",
                     "b2kv_decode_paged", "b2kv_decode_workspace_bytes", "b2kv_prefill", "b2kv_strerror",
                     "b2kv_last_cuda_error", "b2kv_version", "b2kv_tune"]:
        assert required in names


def test_library_exports_every_declared_symbol(pkg):
    native = pkg._native
    lib = ctypes.CDLL(str(native.LIB_PATH))
    decls = header_functions()
    for name, nargs in decls.items():
        assert hasattr(lib, name), f"{name} declared in b2kv.h but not exported"
        assert name in native.SIGNATURES, f"{name} has no ctypes signature"
        assert len(native.SIGNATURES[name][1]) == nargs, f"{name}: header has {nargs} args"
    assert set(native.SIGNATURES) == set(decls)


def test_status_text_and_version(pkg):
    lib = pkg._native.lib
    assert lib.b2kv_version() >= 2
    assert lib.b2kv_strerror(0) == b"ok"
    for code in (-1, -2, -3, -4, -5):
        assert len(lib.b2kv_strerror(code)) > 5
    with pytest.raises(pkg._native.B2KVError):
        pkg._native.check(-1)
    assert lib.b2kv_tune(b"no_such_knob", 1) == -1
    assert lib.b2kv_tune(b"decode_grid_per_sm", 0) == 0


def test_argument_checks_return_before_any_launch(pkg):
    lib = pkg._native.lib
    A = 0x1000  # a fake, 16-byte aligned "pointer": these calls must fail before using it
    # null pointer
    assert lib.b2kv_append(None, A, A, A, None, 0, 0, 1, 1, 64, 8, 512, 64, 64, 0, None, None) == -1
    # unsupported dtype
    assert lib.b2kv_append(A, A, A, A, None, 0, 0, 1, 1, 64, 8, 512, 64, 64, 7, None, None) == -3
    # misaligned pointer
    assert lib.b2kv_append(A + 4, A, A, A, None, 0, 0, 1, 1, 64, 8, 512, 64, 64, 0, None, None) == -2
    # stride not a multiple of 16 bytes
    assert lib.b2kv_append(A, A, A, A, None, 0, 0, 1, 1, 64, 8, 513, 64, 64, 0, None, None) == -2
    # position outside the cache
    assert lib.b2kv_append(A, A, A, A, None, 8, 0, 1, 1, 64, 8, 512, 64, 64, 0, None, None) == -1
    # head_dim whose rows are not whole 16-byte chunks
    assert lib.b2kv_append(A, A, A, A, None, 0, 0, 1, 1, 6, 8, 48, 6, 6, 0, None, None) == -3
    # decode: head_dim that is not compiled, missing workspace handled after the shape checks
    assert lib.b2kv_decode(A, A, A, A, None, 4, 0, 1, 1, 48, 8, 384, 48, 48, 0, A, 1 << 20, None, None) == -3
    assert lib.b2kv_decode(A, A, A, A, None, 4, 0, 0, 1, 64, 8, 512, 64, 64, 0, A, 1 << 20, None, None) == -1
    # decode without a workspace argument: the same checks come before the look-up of the built-in array
    assert lib.b2kv_decode_static(None, A, A, A, None, 4, 0, 1, 1, 64, 8, 512, 64, 64, 0, None, None) == -1
    assert lib.b2kv_decode_static(A, A, A, A, None, 4, 0, 1, 1, 64, 8, 512, 64, 64, 7, None, None) == -3
    assert lib.b2kv_decode_static(A, A, A, A, None, 4, 0, 1, 1, 48, 8, 384, 48, 48, 0, None, None) == -3
    assert lib.b2kv_decode_static(A, A + 8, A, A, None, 4, 0, 1, 1, 64, 8, 512, 64, 64, 0, None, None) == -2
    # paged decode: table smaller than the upper bound of the lengths
    assert lib.b2kv_decode_paged(A, A, A, A, None, 4, 0, A, 1, 16, 8, 1, 1, 64, 64, 1024, 64, 1024, 0, A, 1 << 20,
                                 None, None) == -1
    # prefill: K cache given without V cache
    assert lib.b2kv_prefill(A, A, A, A, None, None, A, None, 0, 0, 0, 8, 1, 8, 1, 64, 0, None, None) == -1
    assert lib.b2kv_prefill(A, A, A, A, None, None, None, None, 0, 0, 0, 0, 1, 0, 1, 64, 0, None, None) == -1
    # matmul: fp32 is not taken, a missing operand, an inner dimension whose rows are not whole 16-byte chunks,
    # a misaligned residual
    assert lib.b2kv_matmul(A, A, None, None, A, 256, 128, 128, 0, 0, None, None) == -3
    assert lib.b2kv_matmul(A, None, None, None, A, 256, 128, 128, 0, 1, None, None) == -1
    assert lib.b2kv_matmul(A, A, None, None, A, 256, 100, 128, 0, 1, None, None) == -3
    assert lib.b2kv_matmul(A, A, None, A + 2, A, 256, 128, 128, 0, 1, None, None) == -2
    assert lib.b2kv_matmul(A, A, None, None, A, 256, 128, 128, 2, 1, None, None) == -1
    # length advance: no lengths, no sequences
    assert lib.b2kv_advance_lengths(None, 4, 1, None) == -1
    assert lib.b2kv_advance_lengths(A, 0, 1, None) == -1


def test_workspace_size_grows_with_the_problem(pkg):
    lib = pkg._native.lib
    small = lib.b2kv_decode_workspace_bytes(1, 4, 64, 256, 0)
    big = lib.b2kv_decode_workspace_bytes(64, 32, 128, 8192, 1)
    assert 0 < small < big
    assert lib.b2kv_decode_workspace_bytes(0, 4, 64, 256, 0) == 0
    assert lib.b2kv_decode_workspace_bytes(1, 4, 64, 256, 9) == 0
