"""Facade with the reference's names (simple-llm/src/gpu/gpu.py:82-156), restricted to the
KV-cache attention path and the tail of a generation step: callers write ``from <package> import gpu`` and use
``gpu.kv_cache_update(ctx, ...)`` exactly as with the reference's ``gpu`` module."""
from .attention import flash_attention
from .batch import (
    batch_begin,
    batch_commit,
    perf_monitor_create,
    perf_monitor_kernel_time_record,
    perf_monitor_reset,
    perf_monitor_stats_get,
    perf_monitor_submission_record,
)
from .buffers import (
    gpu_buffer_1d_create,
    gpu_buffer_1d_read,
    gpu_buffer_1d_write,
    gpu_buffer_2d_create,
    gpu_buffer_2d_read,
    gpu_buffer_2d_write,
    gpu_buffer_zerofy,
)
from .device import context_create, device_config_create, device_create, pipeline_cache_create
from .kv_cache import (
    attention_with_kv_cache,
    kv_cache_create,
    kv_cache_gather,
    kv_cache_reset,
    kv_cache_set_lengths,
    kv_cache_update,
)
from .projection import matmul, qkv_project_append
from .step_tail import argmax, embedding, extract_last_tokens, layernorm, softmax
from .types import GPUBuffer1D, GPUBuffer2D, GPUConfig, GPUContext, KVCache, KVCacheConfig, KVCacheLayer

__all__ = [
    "GPUBuffer1D", "GPUBuffer2D", "GPUConfig", "GPUContext", "KVCache", "KVCacheConfig", "KVCacheLayer",
    "device_create", "device_config_create", "pipeline_cache_create", "context_create",
    "gpu_buffer_1d_create", "gpu_buffer_2d_create", "gpu_buffer_1d_write", "gpu_buffer_2d_write",
    "gpu_buffer_1d_read", "gpu_buffer_2d_read", "gpu_buffer_zerofy",
    "flash_attention",
    "batch_begin", "batch_commit",
    "perf_monitor_create", "perf_monitor_kernel_time_record", "perf_monitor_reset", "perf_monitor_stats_get",
    "perf_monitor_submission_record",
    "kv_cache_create", "kv_cache_reset", "kv_cache_update", "attention_with_kv_cache",
    "kv_cache_gather", "kv_cache_set_lengths",
    "embedding", "layernorm", "extract_last_tokens", "softmax", "argmax",
    "qkv_project_append", "matmul",
]
