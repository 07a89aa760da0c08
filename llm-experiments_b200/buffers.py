"""Buffers: torch CUDA tensors wrapped like the reference's GPUBuffer1D / GPUBuffer2D.

Mirrors simple-llm/src/gpu/gpu_buffer.py (create :58-114, zerofy :117-127, write :130-148,
read :151-208).  The reference stores fp32 / i32 / u32 only (:31-39); a ``dtype`` argument
adds bf16.  Host data may be a numpy array or a CPU torch tensor (numpy has no bf16).
Creation, upload and read-back are plumbing: they use torch copies, not kernels of this
library.
"""
from __future__ import annotations

from typing import Optional

import numpy as np
import torch

from .types import GPUBuffer1D, GPUBuffer2D, GPUBufferAny, GPUContext

_NP_OK = (np.float32, np.uint32, np.int32)


def _as_host_tensor(data, dtype: Optional[torch.dtype]) -> torch.Tensor:
    if isinstance(data, torch.Tensor):
        t = data
    else:
        if data.dtype not in _NP_OK:
            raise ValueError(f"Unsupported dtype: {data.dtype}. Supported: float32, int32, uint32")
        arr = np.ascontiguousarray(data)
        if arr.dtype == np.uint32:
            arr = arr.view(np.int32)
        t = torch.from_numpy(arr)
    if dtype is not None and t.dtype != dtype:
        t = t.to(dtype)
    return t.contiguous()


def _create(ctx: GPUContext, shape, data, dtype) -> torch.Tensor:
    if data is not None:
        host = _as_host_tensor(data, dtype)
        return host.to(ctx.device, non_blocking=True).reshape(shape)
    return torch.empty(shape, dtype=dtype or torch.float32, device=ctx.device)


def gpu_buffer_1d_create(ctx: GPUContext, size: int, data=None, dtype: Optional[torch.dtype] = None) -> GPUBuffer1D:
    if size <= 0:
        raise ValueError(f"Buffer size must be positive, got {size}")
    if data is not None and tuple(data.shape) != (size,):
        raise ValueError(f"Data shape {tuple(data.shape)} doesn't match buffer size ({size},)")
    return GPUBuffer1D(buffer=_create(ctx, (size,), data, dtype), shape=(size,), size=size)


def gpu_buffer_2d_create(ctx: GPUContext, rows: int, cols: int, data=None,
                         dtype: Optional[torch.dtype] = None) -> GPUBuffer2D:
    if rows <= 0 or cols <= 0:
        raise ValueError(f"Buffer dimensions must be positive, got ({rows}, {cols})")
    if data is not None and tuple(data.shape) != (rows, cols):
        raise ValueError(f"Data shape {tuple(data.shape)} doesn't match buffer shape ({rows}, {cols})")
    return GPUBuffer2D(buffer=_create(ctx, (rows, cols), data, dtype), shape=(rows, cols), size=rows * cols)


def gpu_buffer_zerofy(ctx: GPUContext, gpu_buffer: GPUBufferAny) -> None:
    gpu_buffer.buffer.zero_()


def _write(ctx: GPUContext, in_data, buffer: GPUBufferAny) -> None:
    host = _as_host_tensor(in_data, buffer.buffer.dtype)
    buffer.buffer.copy_(host.reshape(buffer.buffer.shape), non_blocking=True)


def gpu_buffer_1d_write(ctx: GPUContext, in_data, buffer: GPUBuffer1D) -> None:
    _write(ctx, in_data, buffer)


def gpu_buffer_2d_write(ctx: GPUContext, in_data, buffer: GPUBuffer2D) -> None:
    _write(ctx, in_data, buffer)


def _read(ctx: GPUContext, buffer: GPUBufferAny, out_data) -> None:
    """Blocking read-back into a pre-allocated numpy array or CPU tensor (as the reference's
    staged map_sync read blocks, gpu_buffer.py:151-182)."""
    if isinstance(out_data, torch.Tensor):
        out_data.copy_(buffer.buffer.reshape(out_data.shape), non_blocking=True)
        torch.cuda.current_stream(ctx.device).synchronize()
    else:
        host = buffer.buffer.to(torch.float32).cpu() if buffer.buffer.dtype == torch.bfloat16 else buffer.buffer.cpu()
        np.copyto(out_data, host.numpy().reshape(out_data.shape))


def gpu_buffer_1d_read(ctx: GPUContext, buffer: GPUBuffer1D, out_data) -> None:
    _read(ctx, buffer, out_data)


def gpu_buffer_2d_read(ctx: GPUContext, buffer: GPUBuffer2D, out_data) -> None:
    _read(ctx, buffer, out_data)
