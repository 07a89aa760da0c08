"""Data carriers of the KV-cache path, shaped like the reference's dataclasses.

Mirrors simple-llm/src/gpu/gpu_types.py: ``GPUConfig`` (:19-201, only the fields this
path reads), ``GPUBuffer1D`` / ``GPUBuffer2D`` (:212-235), ``BatchState`` (:252-261),
``GPUContext`` (:264-270), ``KVCacheLayer`` / ``KVCache`` / ``KVCacheConfig`` (:403-467).
A buffer's ``buffer`` field holds a torch CUDA tensor where the reference holds a
``wgpu.GPUBuffer``.  Fields that the reference does not have carry defaults that keep
its behaviour (fp32, one shared ``current_len``, ``[B*T_max, H*D]`` layout, no paging).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple, Union

import torch


@dataclass
class GPUConfig:
    """Kernel and limit settings (reference: gpu_types.py:19-201).

    The tile-size fields are accepted for compatibility; the CUDA kernels pick their own
    tiles, so only ``flash_attn_max_head_dim``, ``max_batch_operations`` and the extension
    fields below change behaviour.
    """

    flash_attn_bc: int = 32
    flash_attn_br: int = 32
    flash_attn_max_head_dim: int = 128
    max_workgroup_storage_size: int = 16384
    default_workgroup_size: int = 256
    attention_workgroup_size: int = 256
    max_workgroups_per_dim: int = 65535
    max_batch_operations: int = 1000
    layernorm_epsilon: float = 1e-5
    # ---- extensions ----
    enforce_reference_decode_limit: bool = False
    """True: refuse current_len > attention_workgroup_size as the reference does
    (gpu_kv_cache.py:250-257).  The split-K kernel has no such limit, so the default is off."""
    check_device_status: bool = False
    """True: batch_commit synchronises and raises if a kernel recorded a device status."""


@dataclass
class GPUBuffer1D:
    buffer: torch.Tensor
    shape: Tuple[int]
    size: int


@dataclass
class GPUBuffer2D:
    buffer: torch.Tensor
    shape: Tuple[int, int]
    size: int


GPUBufferAny = Union[GPUBuffer1D, GPUBuffer2D]


@dataclass
class PipelineCache:
    """Kept for signature compatibility; CUDA kernels are compiled ahead of time."""

    pipelines: dict = field(default_factory=dict)
    bind_groups: dict = field(default_factory=dict)


@dataclass
class BatchState:
    """An open batch (reference: gpu_types.py:252-261).  ``encoder`` is the CUDA stream the
    batch's operations are issued on; ``None`` after commit, as in the reference."""

    encoder: Optional[Any]
    retained_buffers: List[Any] = field(default_factory=list)
    enable_profiling: bool = False
    operation_count: int = 0


@dataclass
class KernelTimeStats:
    """Reference: gpu_types.py:360-372."""

    count: int
    total_ms: float
    avg_ms: float
    min_ms: float
    max_ms: float


@dataclass
class PerfStats:
    """Reference: gpu_types.py:375-384."""

    total_submissions: int
    kernel_times: Dict[str, KernelTimeStats]


@dataclass
class PerfMonitor:
    """Reference: gpu_types.py:387-395.  ``kernel_times`` is keyed by the name of the reference
    function an operation stands for (``kv_cache_update``, ``flash_attention``, ...)."""

    kernel_times: Dict[str, List[float]] = field(default_factory=dict)
    memory_usage: Dict[str, Any] = field(default_factory=dict)
    submission_count: int = 0


@dataclass
class GPUContext:
    device: torch.device
    config: GPUConfig
    batch_state: Optional[BatchState]
    pipeline_cache: Optional[PipelineCache] = None
    reduction_workspace: Optional[GPUBuffer1D] = None
    dev_status: Optional[torch.Tensor] = None  # int32[1], written by kernels that detect a bad index
    perf_monitor: Optional[PerfMonitor] = None  # filled by batches opened with enable_profiling
    prefill_workspace: Optional[torch.Tensor] = None  # scratch of flash_attention for fp32 prompts, grown on demand


@dataclass
class KVCacheLayer:
    """K and V of one layer.  Reference layout (default): ``[B*T_max, H*D]``.
    ``layout="bhtd"``: ``[B*H*T_max, D]``.  Paged: pools ``[n_blocks*H*block_size, D]``."""

    k_cache: GPUBuffer2D
    v_cache: GPUBuffer2D


@dataclass
class KVCache:
    layers: List[KVCacheLayer]
    batch_size: int
    max_seq_len: int
    current_len: int  # host-side length; with seq_lens set it is the upper bound of all lengths
    n_heads: int
    head_dim: int
    # ---- extensions ----
    dtype: torch.dtype = torch.float32
    layout: str = "bthd"  # "bthd" (reference) or "bhtd"
    seq_lens: Optional[torch.Tensor] = None  # int32[B] on the device: per-sequence lengths
    block_table: Optional[torch.Tensor] = None  # int32[B, max_blocks] on the device
    block_size: int = 0
    n_blocks: int = 0
    workspace: Optional[torch.Tensor] = None  # decode scratch, allocated on first use


@dataclass
class KVCacheConfig:
    batch_size: int
    max_seq_len: int
    n_layers: int
    n_heads: int
    head_dim: int
    # ---- extensions ----
    dtype: torch.dtype = torch.float32
    layout: str = "bthd"
    ragged: bool = False  # keep per-sequence lengths on the device
    block_size: int = 0  # > 0: paged cache with blocks of this many tokens
    n_blocks: int = 0  # pool size in blocks (paged)
