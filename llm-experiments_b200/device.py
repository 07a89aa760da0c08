"""Device and configuration set-up (reference: simple-llm/src/gpu/gpu_device.py).

The reference opens a WebGPU adapter, builds a ``GPUConfig`` from vendor presets and keeps a
cache of compiled pipelines (:40-42, :163-192, :343-431).  On CUDA the kernels are compiled
ahead of time, so only the calls that the reference's callers make are kept:
``device_create``, ``device_config_create``, ``pipeline_cache_create`` and a convenience
``context_create``.
"""
from __future__ import annotations

import torch

from . import _native  # noqa: F401  (fails loudly when the CUDA library is missing)
from .types import GPUConfig, GPUContext, PipelineCache


def device_create(index: int = None) -> torch.device:
    if not torch.cuda.is_available():
        raise RuntimeError("No CUDA device: this package runs on B200 (sm_100a) only and has no CPU fallback")
    if index is None:
        index = torch.cuda.current_device()
    torch.cuda.set_device(index)
    return torch.device("cuda", index)


def device_config_create(device: torch.device) -> GPUConfig:
    return GPUConfig()


def pipeline_cache_create(device: torch.device) -> PipelineCache:
    return PipelineCache()


def context_create(index: int = None) -> GPUContext:
    device = device_create(index)
    return GPUContext(device=device, config=device_config_create(device), batch_state=None,
                      pipeline_cache=pipeline_cache_create(device))
