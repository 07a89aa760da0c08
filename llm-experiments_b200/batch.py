"""Batches and shape checks (reference: simple-llm/src/gpu/gpu_ops.py).

The reference records compute passes into a command encoder between ``batch_begin`` and
``batch_commit`` and submits them together (:226-250, :343-360).  On CUDA the stream already
is that ordered queue: operations are launched asynchronously as they are added, and
``batch_commit`` only closes the batch.  The observable rules are kept: operations need an
open batch, a batch holds at most ``max_batch_operations`` operations (:277-283), and a second
commit raises (:352-353).
"""
from __future__ import annotations

import functools
from typing import Tuple

import torch

from . import _native
from .types import BatchState, GPUBuffer1D, GPUBuffer2D, GPUContext, KernelTimeStats, PerfMonitor, PerfStats


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
    """Opens a batch on torch's current stream (reference: gpu_ops.py:226-250).  With
    ``enable_profiling`` every operation of the batch is wrapped in an NVTX range named after the
    reference function and bracketed by CUDA events; ``batch_commit`` then synchronises and adds
    the durations to ``ctx.perf_monitor`` (the reference stores the flag, gpu_ops.py:245-250, and
    leaves the recording to the caller, gpu_device.py:569-608)."""
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
    # The kernels go to the batch's stream; the few torch operations beside them (length counters) go to
    # torch's current stream.  They are ordered only when the two are the same stream.
    if torch.cuda.current_stream(ctx.device) != state.encoder:
        raise RuntimeError("The current CUDA stream changed since batch_begin; commit the batch and begin a new one "
                           "on the new stream")
    state.operation_count += 1
    return state.encoder.cuda_stream


def reference_op(name: str):
    """Marks a function ``f(ctx, ...)`` as one operation of the reference's API.  In a batch opened with
    ``enable_profiling`` the call runs inside an NVTX range called ``name`` between two CUDA events
    whose distance ``batch_commit`` records under that name."""

    def wrap(fn):
        @functools.wraps(fn)
        def inner(ctx, *args, **kwargs):
            state = ctx.batch_state
            if state is None or not state.enable_profiling or state.encoder is None:
                return fn(ctx, *args, **kwargs)
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.nvtx.range_push(name)
            try:
                start.record(state.encoder)
                result = fn(ctx, *args, **kwargs)
                end.record(state.encoder)
            finally:
                torch.cuda.nvtx.range_pop()
            state.retained_buffers.append((name, start, end))
            return result

        return inner

    return wrap


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
    if state.enable_profiling:
        stream.synchronize()
        if ctx.perf_monitor is None:
            ctx.perf_monitor = perf_monitor_create()
        for item in state.retained_buffers:
            if isinstance(item, tuple) and len(item) == 3:
                name, start, end = item
                perf_monitor_kernel_time_record(ctx.perf_monitor, name, start.elapsed_time(end))
        perf_monitor_submission_record(ctx.perf_monitor)
    state.retained_buffers.clear()
    if ctx.config.check_device_status and ctx.dev_status is not None:
        stream.synchronize()
        code = int(ctx.dev_status.item())
        if code != 0:
            ctx.dev_status.zero_()
            raise RuntimeError("device status: " + _native.DEV_STATUS_TEXT.get(code, f"code {code}"))


# ---- performance monitor (reference: simple-llm/src/gpu/gpu_device.py:569-608) ----


def perf_monitor_create() -> PerfMonitor:
    return PerfMonitor()


def perf_monitor_kernel_time_record(monitor: PerfMonitor, kernel_name: str, duration_ms: float) -> None:
    monitor.kernel_times.setdefault(kernel_name, []).append(duration_ms)


def perf_monitor_submission_record(monitor: PerfMonitor) -> None:
    monitor.submission_count += 1


def perf_monitor_stats_get(monitor: PerfMonitor) -> PerfStats:
    stats = {}
    for name, times in monitor.kernel_times.items():
        stats[name] = KernelTimeStats(count=len(times), total_ms=sum(times),
                                      avg_ms=sum(times) / len(times) if times else 0,
                                      min_ms=min(times) if times else 0, max_ms=max(times) if times else 0)
    return PerfStats(total_submissions=monitor.submission_count, kernel_times=stats)


def perf_monitor_reset(monitor: PerfMonitor) -> None:
    monitor.kernel_times.clear()
    monitor.memory_usage.clear()
    monitor.submission_count = 0
