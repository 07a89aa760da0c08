"""`b2kv_decode_static`: decode attention for callers that cannot allocate device memory
when they decode (all HBM already given to the KV-cache pool, or a latency budget that rules
out cudaMalloc's device-wide synchronisation).  Its split-K partials live in an array inside
the library instead of a caller-provided workspace.

The test calls the entry point through the C ABI twice in a row, with different inputs, and
compares each result with `b2kv_decode` (caller-provided workspace) on the same inputs: the
second call runs on top of whatever the first one left in the shared array.  It also checks that
a shape whose partials exceed the array is refused before anything is launched.  This file sorts
last on purpose, so that a run stopping at the first failure has already run everything else.
"""
import numpy as np
import pytest
import torch

from tests import kv_util as U

pytestmark = pytest.mark.gpu


def _decode_both(native, q, k, v, lens, B, H, D, T_max, dtype_code, stream):
    lib = native.lib
    strides = (H * T_max * D, D, T_max * D)  # [B, H, T_max, D]
    t_upper = int(lens.max().item())
    out_ws = torch.empty_like(q)
    out_static = torch.empty_like(q)
    nbytes = lib.b2kv_decode_workspace_bytes(B, H, D, T_max, dtype_code)
    ws = torch.empty(nbytes, dtype=torch.uint8, device=q.device)
    native.check(lib.b2kv_decode(q.data_ptr(), k.data_ptr(), v.data_ptr(), out_ws.data_ptr(), lens.data_ptr(), 0, 0,
                                 B, H, D, t_upper, *strides, dtype_code, ws.data_ptr(), ws.numel(), None, stream))
    native.check(lib.b2kv_decode_static(q.data_ptr(), k.data_ptr(), v.data_ptr(), out_static.data_ptr(),
                                        lens.data_ptr(), 0, 0, B, H, D, t_upper, *strides, dtype_code, None, stream))
    torch.cuda.synchronize()
    return out_ws, out_static


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_static_scratch_decode_matches_workspace_decode_twice(pkg, dtype):
    native = pkg._native
    device = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    stream = torch.cuda.current_stream().cuda_stream
    code = native.DTYPE_BF16 if dtype == torch.bfloat16 else native.DTYPE_F32
    D = 128 if dtype == torch.bfloat16 else 64
    B, H, T_max = 6, 8, 3072
    tol = U.TOL[dtype]
    for call, lens_list in enumerate([[3072, 1, 700, 64, 2049, 1500], [5, 3000, 1024, 33, 0, 2500]]):
        lens = torch.tensor(lens_list, dtype=torch.int32, device=device)
        q = U.randn((B, H * D), dtype, device, 10 + call)
        k = U.randn((B, H, T_max, D), dtype, device, 20 + call)
        v = U.randn((B, H, T_max, D), dtype, device, 30 + call)
        out_ws, out_static = _decode_both(native, q, k, v, lens, B, H, D, T_max, code, stream)
        np.testing.assert_allclose(U.to_f32(out_static), U.to_f32(out_ws), **tol)
        assert torch.equal(out_static.view(torch.uint8), out_ws.view(torch.uint8))  # same kernels, same split
        want = U.oracle_decode(q, k.permute(0, 2, 1, 3).contiguous(), v.permute(0, 2, 1, 3).contiguous(), lens_list)
        np.testing.assert_allclose(U.to_f32(out_static), want, **tol)


def test_static_scratch_decode_takes_the_benchmark_shape_and_allocates_nothing(pkg):
    """B = 64, H = 32, D = 128 bf16 (4 MB of partial slots) fits the built-in array and is
    bit-identical to b2kv_decode; the free device memory does not move across a call once the first call on
    the device has looked the array's address up."""
    native = pkg._native
    device = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    stream = torch.cuda.current_stream().cuda_stream
    B, H, D, T_max = 64, 32, 128, 1024
    rng = np.random.default_rng(0)
    lens_list = [int(x) for x in rng.integers(64, T_max + 1, size=B)]
    lens = torch.tensor(lens_list, dtype=torch.int32, device=device)
    q = U.randn((B, H * D), torch.bfloat16, device, 41)
    k = U.randn((B, H, T_max, D), torch.bfloat16, device, 42)
    v = U.randn((B, H, T_max, D), torch.bfloat16, device, 43)
    out_ws, out_static = _decode_both(native, q, k, v, lens, B, H, D, T_max, native.DTYPE_BF16, stream)
    assert torch.equal(out_static.view(torch.uint8), out_ws.view(torch.uint8))
    strides = (H * T_max * D, D, T_max * D)
    out2 = torch.empty_like(q)
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    native.check(native.lib.b2kv_decode_static(q.data_ptr(), k.data_ptr(), v.data_ptr(), out2.data_ptr(),
                                               lens.data_ptr(), 0, 0, B, H, D, T_max, *strides, native.DTYPE_BF16,
                                               None, stream))
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before
    assert torch.equal(out2.view(torch.uint8), out_ws.view(torch.uint8))


def test_static_scratch_decode_refuses_shapes_beyond_its_array(pkg):
    native = pkg._native
    device = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    B, H, D, T_upper = 4096, 32, 128, 8192  # one partial slot per (sequence, head) alone: 68 MB, twice the array
    assert B * H * (D + 2) * 4 > native.STATIC_SCRATCH_BYTES
    tiny = torch.zeros(64, dtype=torch.bfloat16, device=device)  # never dereferenced: the call must fail first
    rc = native.lib.b2kv_decode_static(tiny.data_ptr(), tiny.data_ptr(), tiny.data_ptr(), tiny.data_ptr(), None,
                                       T_upper, 0, B, H, D, T_upper, H * T_upper * D, D, T_upper * D,
                                       native.DTYPE_BF16, None, torch.cuda.current_stream().cuda_stream)
    assert rc == native.ERR_STATIC_LIMIT
    assert b"B2KV_STATIC_SCRATCH_BYTES" in native.lib.b2kv_strerror(rc)
    with pytest.raises(native.B2KVError, match="built-in array"):
        native.check(rc)
    torch.cuda.synchronize()
