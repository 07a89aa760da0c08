"""Batches and shape checks (reference: simple-llm/src/gpu/gpu_ops.py).

The reference records compute passes into a command encoder between ``batch_begin`` and
``batch_commit`` and submits them together (:226-250, :343-360).  On CUDA the stream already
is that ordered queue: operations are launched asynchronously as they are added, and
``batch_commit`` only closes the batch.  The observable rules are kept: operations need an
open batch, a batch holds at most ``max_batch_operations`` operations (:277-283), and a second
commit raises (:352-353).
"""
from __future__ import annotations

from typing import Tuple

import torch

from . import _native
from .types import BatchState, GPUBuffer1D, GPUBuffer2D, GPUContext


def validate_buffer_shape_1d(buffer: GPUBuffer1D, expected_size: int, name: str) -> None:
    if expected_size <= 0:
        raise ValueError(f"Invalid expected size for {name}: {expected_size}")
    if tuple(buffer.shape) != (expected_size,):
        raise ValueError(f"{name} shape mismatch: got {buffer.shape}, expected ({expected_size},)")


def validate_buffer_shape_2d(buffer: GPUBuffer2D, expected_shape: Tuple[int, int], name: str) -> None:
    if expected_shape[0] <= 0 or expected_shape[1] <= 0:
        raise ValueError(f"Invalid expected shape for {name}: {expected_shape}")
    if tuple(buffer.shape) != tuple(expected_shape):
        raise ValueError(f"{name} shape mismatch: got {buffer.shape}, expected {expected_shape}")


def batch_begin(ctx: GPUContext, enable_profiling: bool = False) -> None:
    stream = torch.cuda.current_stream(ctx.device)
    ctx.batch_state = BatchState(encoder=stream, retained_buffers=[], enable_profiling=enable_profiling,
                                 operation_count=0)


def batch_op_begin(ctx: GPUContext) -> int:
    """Common prologue of every operation: returns the raw stream handle to launch on."""
    state = ctx.batch_state
    if state is None or state.encoder is None:
        raise RuntimeError("Must call batch_begin before adding operations")
    max_ops = ctx.config.max_batch_operations
    if state.operation_count >= max_ops:
        raise RuntimeError(f"Batch operation limit ({max_ops}) exceeded. Call batch_commit() to flush operations.")
    state.operation_count += 1
    return state.encoder.cuda_stream


def dev_status_ptr(ctx: GPUContext) -> int:
    if ctx.dev_status is None:
        ctx.dev_status = torch.zeros(1, dtype=torch.int32, device=ctx.device)
    return ctx.dev_status.data_ptr()


def batch_commit(ctx: GPUContext) -> None:
    state = ctx.batch_state
    if state is None or state.encoder is None:
        raise RuntimeError("Batch already submitted or not initialized")
    stream = state.encoder
    state.encoder = None
    state.retained_buffers.clear()
    if ctx.config.check_device_status and ctx.dev_status is not None:
        stream.synchronize()
        code = int(ctx.dev_status.item())
        if code != 0:
            ctx.dev_status.zero_()
            raise RuntimeError("device status: " + _native.DEV_STATUS_TEXT.get(code, f"code {code}"))
