#!/usr/bin/env python3
"""Benchmark of the KV-cache attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference] [--workload NAME]

One "step" is one pass of the hot path over one batch of synthetic input: append one new
K/V row per sequence, then single-token attention over the whole cache (one layer).  The
default workload is the decode microbenchmark (batch 64, 32 heads, head_dim 128, bf16,
per-sequence cache length uniform in [512, 8192] from seed 0); the cache (9 GB) is far
larger than L2, so no flush is needed between steps.  With N > 1 every rank (one per GPU,
launched by torchrun) owns its own batch of 64 sequences and there is no collective in the
step (weak scaling); time is the maximum over ranks.

Rank 0 prints ONE JSON line.  ``value`` is decode tokens/s with inputs resident in HBM;
``e2e`` is the same step through the public API with host buffers (pinned host -> device
copies of q / new K / new V and the device -> host read of the output inside the timed
region); ``roofline`` is the decode kernel's algorithmic HBM bytes over its CUDA-event time
against the measured copy bandwidth; ``cpu_baseline`` is the CPU oracle (a port of the
reference math, all host threads) on a bounded sample of the same workload.

``--impl reference`` times that CPU port alone: the reference itself has no CPU or CUDA
implementation of this path that can run here (its kernels are WGSL dispatched through
wgpu / Vulkan, and this machine has no graphics stack).
"""
from __future__ import annotations

import argparse
import json
import os
import pathlib
import sys
import threading
import time

import numpy as np

ROOT = pathlib.Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

WORKLOADS = {
    # name: (B, H, D, len_lo, len_hi, block_size, description)
    "decode": dict(B=64, H=32, D=128, lo=512, hi=8192, block_size=0,
                   desc="decode microbench: B=64 H=32 D=128 bf16, len~U[512,8192] seed 0, [B,H,T,D] cache"),
    "decode_small": dict(B=8, H=32, D=128, lo=512, hi=8192, block_size=0,
                         desc="decode microbench cut to 8 sequences (1.2 GB cache, for profiler captures)"),
    "paged": dict(B=64, H=32, D=128, lo=512, hi=8192, block_size=16,
                  desc="paged decode: same shapes, 16-token blocks placed by a seeded permutation of 65536 blocks"),
    "longctx": dict(B=4, H=64, D=128, lo=131072, hi=131072, block_size=0,
                    desc="long-context decode: B=4 H=64 D=128 bf16, len 131072, batch-resident on one GPU"),
    "longctx_headsplit": dict(B=4, H=64, D=128, lo=131072, hi=131072, block_size=0, head_split=True,
                              desc="long-context decode: B=4 H=64 D=128 bf16, len 131072, heads split over the "
                                   "GPUs, outputs all-gathered with NCCL"),
    "qkv_append": dict(B=64, H=32, D=128, T=256, layers=4, qkv=True,
                       desc="Q/K/V projection fused with the cache append: B=64 E=4096 (H=32 D=128) bf16, one layer per step"),
    "decode_layer": dict(B=64, H=32, D=128, lo=512, hi=8192, layers=2, layer_step=True,
                         desc="one decoder layer of a cached decode step (LN, QKV+append, attention, Wo, LN, MLP): "
                              "B=64 E=4096 (H=32 D=128) bf16, len~U[512,8192] seed 0"),
    "prefill_layer": dict(B=8, H=32, D=128, N=4096, layers=2, prompt_layer=True,
                          desc="one decoder layer over a whole prompt (LN, Q/K/V GEMMs, causal attention + cache write, Wo, "
                               "LN, MLP): B=8 N=4096 E=4096 (H=32 D=128) bf16"),
    "prefill_layer_small": dict(B=1, H=32, D=128, N=4096, layers=2, prompt_layer=True,
                                desc="the prompt-side layer cut to one sequence (for profiler captures)"),
    "prefill_small": dict(B=2, H=32, D=128, N=4096, prefill=True,
                          desc="causal prefill cut to 2 sequences (for profiler captures)"),
    "prefill": dict(B=8, H=32, D=128, N=4096, prefill=True,
                    desc="causal prefill: B=8 H=32 D=128 N=4096 bf16, fused with the K/V cache write"),
}
SLACK = 1024  # rows of head-room above the longest sequence for the appended tokens


def measured_hbm_peak():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        try:
            return float(json.loads(path.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons of one GPU through NVML while the timed region runs."""

    def __init__(self, index: int, period: float = 0.01):
        super().__init__(daemon=True)
        self.index, self.period = index, period
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop_evt = threading.Event()
        self.ok = False
        try:
            import pynvml

            pynvml.nvmlInit()
            self.nv = pynvml
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM))
            self.ok = True
        except Exception:
            self.ok = False

    def run(self):
        if not self.ok:
            return
        nv = self.nv
        names = {
            getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8): "hw_slowdown",
            getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40): "hw_thermal_slowdown",
            getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20): "sw_thermal_slowdown",
            getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4): "sw_power_cap",
        }
        while not self._stop_evt.is_set():
            try:
                self.samples.append(int(nv.nvmlDeviceGetClockInfo(self.handle, nv.NVML_CLOCK_SM)))
                try:
                    mask = int(nv.nvmlDeviceGetCurrentClocksEventReasons(self.handle))
                except Exception:
                    mask = int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.handle))
                for bit, name in names.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop_evt.wait(self.period)

    def finish(self):
        self._stop_evt.set()
        if self.is_alive():
            self.join(timeout=2)
        med = int(np.median(self.samples)) if self.samples else None
        return {"sm_mhz": med, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(self.samples)}


def physical_gpu_index(local_rank: int) -> int:
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        try:
            return int(vis.split(",")[local_rank])
        except Exception:
            return local_rank
    return local_rank


def make_lengths(w, seed):
    rng = np.random.default_rng(seed)
    if w["lo"] == w["hi"]:
        return np.full(w["B"], w["lo"], dtype=np.int64)
    return rng.integers(w["lo"], w["hi"] + 1, size=w["B"])


def algorithmic_bytes(lens_after, H, D, es, B, block_size):
    """Bytes the step must move: K and V rows of every attended token once, q, out, and the
    append (read new K, V; write the rows).  Split-K partials are overhead, not counted."""
    kv = int(np.sum(lens_after)) * H * D * 2 * es
    qo = 2 * B * H * D * es
    app = 4 * B * H * D * es
    table = 4 * int(np.sum((lens_after + block_size - 1) // block_size)) if block_size else 0
    return kv, kv + qo + app + table


# ------------------------------------------------------------------------------------------
# CPU arm: the oracle port on a bounded sample
# ------------------------------------------------------------------------------------------

def cpu_port_run(w, lens, steps, warmup, sample_seqs, log=None):
    """Times append + decode of the CPU oracle (C, OpenMP, all host threads) on the first
    `sample_seqs` sequences of the workload.  Returns (tokens_per_s, ms_per_step, threads)."""
    from oracle import c_oracle, kv_oracle

    Bs = min(sample_seqs, w["B"])
    H, D = w["H"], w["D"]
    sl = np.asarray(lens[:Bs], dtype=np.int32)
    T_max = int(sl.max()) + SLACK
    rng = np.random.default_rng(1234)
    # bf16 bit patterns of N(0,1) samples; one shared block of rows keeps set-up time bounded
    base_rows = kv_oracle.f32_to_bf16_bits(rng.standard_normal((4096, D)).astype(np.float32))
    reps = (T_max + 4095) // 4096
    one_head = np.tile(base_rows, (reps, 1))[:T_max]
    k_cache = np.ascontiguousarray(np.broadcast_to(one_head[None, None], (Bs, H, T_max, D)))
    v_cache = k_cache.copy()
    q = kv_oracle.f32_to_bf16_bits(rng.standard_normal((Bs, H * D)).astype(np.float32))
    nk = kv_oracle.f32_to_bf16_bits(rng.standard_normal((Bs, H * D)).astype(np.float32))
    nv = kv_oracle.f32_to_bf16_bits(rng.standard_normal((Bs, H * D)).astype(np.float32))
    strides = (H * T_max * D, D, T_max * D)
    # torchrun exports OMP_NUM_THREADS=1 to its workers; the CPU arm is meant to use every host core
    c_oracle.set_num_threads(len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else os.cpu_count())
    threads = c_oracle.num_threads()
    pos = sl.copy()

    def step():
        c_oracle.append(nk, nv, k_cache, v_cache, pos, Bs, H, D, strides)
        pos[:] += 1
        return c_oracle.decode(q, k_cache, v_cache, pos, Bs, H, D, strides)

    for _ in range(warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    dt = time.perf_counter() - t0
    ms = dt / steps * 1e3
    return Bs / (dt / steps), ms, threads, Bs


def run_reference(args, w, rank):
    if rank != 0:
        return
    if w.get("prefill") or w.get("qkv") or w.get("layer_step"):
        w = WORKLOADS["decode"]  # the CPU arm times the decode step, the headline workload
    lens = make_lengths(w, 0)
    steps = max(1, args.steps)
    warm = max(1, min(args.warmup, 3))
    sample = 8 if w["B"] >= 8 else 1
    # keep the whole run within a few minutes whatever K is
    steps = min(steps, 20)
    tps, ms, threads, Bs = cpu_port_run(w, lens, steps, warm, sample)
    line = {
        "impl": "reference",
        "metric": "decode tokens/s",
        "value": tps,
        "unit": "tokens/s",
        "n_gpus": args.gpus,
        "steps": steps,
        "warmup": warm,
        "ms_per_step": ms,
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "bf16 storage, f64 accumulate",
        "data": "synthetic",
        "config": {"workload": w["desc"], "sample": f"first {Bs} sequences of the batch per step"},
        "cpu_baseline": {"value": tps, "unit": "tokens/s", "cores": threads, "kind": "port",
                         "sample": f"append + decode of the first {Bs} of {w['B']} sequences, {steps} steps"},
        "e2e": {"value": tps, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "CPU port of the reference math (oracle/kv_oracle.c); the reference's own WGSL path "
                "needs wgpu/Vulkan: unavailable on this box",
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------
# GPU arm
# ------------------------------------------------------------------------------------------

def run_b200(args, w, rank, world):
    import torch
    import torch.distributed as dist

    import __graft_entry__

    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    pkg = __graft_entry__.import_package()
    gpu = pkg.gpu
    ctx = gpu.context_create(local_rank)

    B, H, D, bs = w["B"], w["H"], w["D"], w["block_size"]
    head_split = bool(w.get("head_split"))
    H_total = H
    if head_split:
        from llm_experiments_b200 import sharding

        h0, h1 = sharding.head_range(H, rank, world)  # this rank's heads of every sequence
        H = h1 - h0
    E = H * D
    dtype = torch.bfloat16
    # every rank holds its own batch (own K/V/q values) with the seed-0 lengths of the named configuration,
    # so that the work per GPU is the same at every N (weak scaling)
    lens0 = make_lengths(w, 0)
    # head-room for the rows appended by the longest timed loop (lengths are reset between loops)
    slack = max(SLACK, args.steps + max(3, args.warmup) + 64)
    T_max = int(lens0.max()) + slack
    n_blocks = 0
    if bs:
        max_blocks = (T_max + bs - 1) // bs
        n_blocks = max(65536, B * max_blocks)
    cache = gpu.kv_cache_create(ctx, gpu.KVCacheConfig(batch_size=B, max_seq_len=T_max, n_layers=1, n_heads=H,
                                                       head_dim=D, dtype=dtype, layout="bhtd", ragged=True,
                                                       block_size=bs, n_blocks=n_blocks))
    if bs:
        perm = np.random.default_rng(0).permutation(n_blocks)[: B * max_blocks].astype(np.int32)
        cache.block_table = torch.from_numpy(perm.reshape(B, max_blocks)).to(device)
    gen = torch.Generator(device=device).manual_seed(1000 + rank)
    layer = cache.layers[0]
    for buf in (layer.k_cache.buffer, layer.v_cache.buffer):
        # N(0,1) in bf16, drawn in slabs to bound the fp32 temporary
        flat = buf.view(-1)
        slab = 1 << 28
        for off in range(0, flat.numel(), slab):
            n = min(slab, flat.numel() - off)
            flat[off:off + n] = torch.randn(n, generator=gen, device=device, dtype=torch.float32).to(dtype)
    q_dev = torch.randn((B, E), generator=gen, device=device, dtype=torch.float32).to(dtype)
    nk_dev = torch.randn((B, E), generator=gen, device=device, dtype=torch.float32).to(dtype)
    nv_dev = torch.randn((B, E), generator=gen, device=device, dtype=torch.float32).to(dtype)
    out_dev = torch.empty((B, E), device=device, dtype=dtype)
    wrap = lambda t: gpu.GPUBuffer2D(buffer=t, shape=tuple(t.shape), size=t.numel())  # noqa: E731
    q_b, nk_b, nv_b, out_b = wrap(q_dev), wrap(nk_dev), wrap(nv_dev), wrap(out_dev)

    def reset_lengths():
        gpu.kv_cache_set_lengths(cache, lens0)

    fused = None
    if head_split and args.fused_gather:
        fused = sharding.FusedHeadGather(device, B, H_total, D, dtype)

    def step_device():
        gpu.batch_begin(ctx)
        gpu.kv_cache_update(ctx, cache, 0, nk_b, nv_b)
        if fused is not None:
            full = fused.decode(ctx, cache, 0, q_b)  # merge kernel stores into every rank's buffer
        else:
            gpu.attention_with_kv_cache(ctx, cache, 0, q_b, out_b)
            full = None
        gpu.batch_commit(ctx)
        if head_split and world > 1 and fused is None:
            full = sharding.gather_heads(out_dev)  # NCCL all-gather: [B, H_total*D] on every rank
        return full

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        """K steps between two events on the launching stream; returns ms (max over ranks)."""
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device=device, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        barrier()
        return ms

    steps, warm = args.steps, max(3, args.warmup)

    # ---- value: inputs resident in HBM -------------------------------------------------
    reset_lengths()
    for _ in range(warm):
        step_device()
    sampler = ClockSampler(physical_gpu_index(local_rank))  # runs across the three timed loops below
    sampler.start()
    ms_total = timed(step_device, steps)
    ms_step = ms_total / steps
    seqs_total = B if head_split else world * B  # head split: the same B sequences on every rank
    tokens_per_s = seqs_total / (ms_step * 1e-3)

    # ---- roofline: the decode call (split kernel + combine) alone, CUDA events ---------
    reset_lengths()
    cache.seq_lens.add_(1)  # the state the decode sees inside a step
    cache.current_len = int(lens0.max()) + 1

    def decode_only():
        gpu.batch_begin(ctx)
        gpu.attention_with_kv_cache(ctx, cache, 0, q_b, out_b)
        gpu.batch_commit(ctx)

    for _ in range(3):
        decode_only()
    ms_dec = timed(decode_only, steps) / steps
    kv_bytes, step_bytes = algorithmic_bytes(lens0 + 1, H, D, 2, B, bs)
    dec_bytes = kv_bytes + 2 * B * E * 2 + (4 * int(np.sum((lens0 + bs) // bs)) if bs else 0)
    peak, peak_kind = measured_hbm_peak()
    achieved = dec_bytes / (ms_dec * 1e-3) / 1e9

    # ---- e2e: host buffers through the public API --------------------------------------
    reset_lengths()
    q_host = q_dev.cpu().pin_memory()
    nk_host = nk_dev.cpu().pin_memory()
    nv_host = nv_dev.cpu().pin_memory()
    out_host = torch.empty((B, E), dtype=dtype).pin_memory()
    out_host_full = torch.empty((B, H_total * D), dtype=dtype).pin_memory()

    def step_e2e():
        gpu.gpu_buffer_2d_write(ctx, q_host, q_b)
        gpu.gpu_buffer_2d_write(ctx, nk_host, nk_b)
        gpu.gpu_buffer_2d_write(ctx, nv_host, nv_b)
        full = step_device()
        if head_split and (world > 1 or fused is not None):
            out_host_full.copy_(full, non_blocking=True)
            torch.cuda.current_stream().synchronize()
        else:
            gpu.gpu_buffer_2d_read(ctx, out_b, out_host)  # blocks until the result is on the host

    for _ in range(3):
        step_e2e()
    ms_e2e = timed(step_e2e, steps) / steps
    clocks = sampler.finish()
    e2e_tps = seqs_total / (ms_e2e * 1e-3)
    h2d = 3 * B * E * 2
    d2h = B * (H_total if head_split else H) * D * 2

    # ---- CPU baseline (rank 0, N=1 only) -----------------------------------------------
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        sample = 8 if B >= 8 else 1
        tps, ms_cpu, threads, Bs = cpu_port_run(w, lens0, steps=6, warmup=1, sample_seqs=sample)
        cpu = {"value": tps, "unit": "tokens/s", "cores": threads, "kind": "port",
               "sample": f"append + decode of the first {Bs} of {B} sequences, 6 steps, {ms_cpu:.1f} ms/step"}

    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if rank != 0:
        return
    line = {
        "metric": "decode tokens/s",
        "value": tokens_per_s,
        "unit": "tokens/s",
        "n_gpus": world,
        "steps": steps,
        "warmup": warm,
        "ms_per_step": ms_step,
        "higher_is_better": True,
        "scaling": "strong" if head_split else "weak",
        "vs_baseline": None,
        "dtype": "bf16 storage, fp32 arithmetic",
        "data": "synthetic",
        "config": {"workload": w["desc"], "batch_per_gpu": B, "global_batch": seqs_total,
                   "sum_len_rank0": int(np.sum(lens0)), "l2": "inputs (GBs of cache) far larger than L2, no flush",
                   "parallelism": (f"heads split x{world}, outputs gathered "
                                   + ("by peer stores fused into the merge kernel" if fused is not None
                                      else "with one NCCL all-gather per step") if head_split
                                   else f"batch-sharded x{world}, no collective in the step")},
        "e2e": {"value": e2e_tps, "unit": "tokens/s", "ms_per_step": ms_e2e, "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h},
        "gpu_launches": 3 * steps,
        "clocks": clocks,
        "roofline": {"bound": "hbm", "kernel": "decode_split_kernel + decode_combine_kernel (one b2kv_decode call)",
                     "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "frac_of_8000_nominal": achieved / 8000.0, "peak_kind": peak_kind, "ms_per_launch": ms_dec,
                     "algorithmic_bytes_per_launch": dec_bytes,
                     "traffic": int(DRAM_BYTES_PER_TOKEN_HEAD * float(np.sum(lens0 + 1)) * H) if not bs else None},
        "step_hbm_gbs": step_bytes / (ms_step * 1e-3) / 1e9,
        "cpu_baseline": cpu,
    }
    print(json.dumps(line), flush=True)


# dram__bytes_read.sum + dram__bytes_write.sum of prefill_tc_kernel per sequence at H=32, D=128, N=4096, from an
# ncu capture of the 2-sequence case (`--workload prefill_small`: 211.3 MB read + 156.5 MB written per launch;
# the algorithmic figure per sequence is Q + K + V + O + two cache copies = 6 x 33.5 MB).  Every sequence brings
# the same traffic, so a full launch is this figure times its sequences.
PREFILL_DRAM_BYTES_PER_SEQUENCE = int((211.3e6 + 156.5e6) / 2)


def measured_tensor_peak():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        try:
            d = json.loads(path.read_text())
            return float(d["bf16_tflops_sustained"]), float(d["bf16_tflops"]), "measured"
        except Exception:
            pass
    return 1400.0, 1590.0, "fallback"


def run_prefill(args, w, rank, world):
    """Causal prefill fused with the cache write; value = prompt tokens/s, roofline = tensor."""
    import torch
    import torch.distributed as dist

    import __graft_entry__

    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    pkg = __graft_entry__.import_package()
    gpu = pkg.gpu
    ctx = gpu.context_create(local_rank)
    B, H, D, N = w["B"], w["H"], w["D"], w["N"]
    E = H * D
    dtype = torch.bfloat16
    gen = torch.Generator(device=device).manual_seed(2000 + rank)
    mk = lambda: torch.randn((B * N, E), generator=gen, device=device, dtype=torch.float32).to(dtype)  # noqa: E731
    Q, K, V = mk(), mk(), mk()
    O = torch.empty_like(Q)
    cache = gpu.kv_cache_create(ctx, gpu.KVCacheConfig(batch_size=B, max_seq_len=N, n_layers=1, n_heads=H, head_dim=D,
                                                       dtype=dtype, layout="bhtd"))
    wrap = lambda t: gpu.GPUBuffer2D(buffer=t, shape=tuple(t.shape), size=t.numel())  # noqa: E731
    Qb, Kb, Vb, Ob = wrap(Q), wrap(K), wrap(V), wrap(O)

    def step_device():
        gpu.batch_begin(ctx)
        gpu.flash_attention(ctx, Qb, Kb, Vb, Ob, None, None, B, N, H, D, cache=cache, layer_idx=0)
        gpu.batch_commit(ctx)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device=device, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        barrier()
        return ms

    steps, warm = min(args.steps, 50), max(3, args.warmup)
    for _ in range(warm):
        step_device()
    sampler = ClockSampler(physical_gpu_index(local_rank))
    sampler.start()
    ms_step = timed(step_device, steps) / steps
    Qh, Kh, Vh = Q.cpu().pin_memory(), K.cpu().pin_memory(), V.cpu().pin_memory()
    Oh = torch.empty_like(Qh).pin_memory()

    def step_e2e():
        gpu.gpu_buffer_2d_write(ctx, Qh, Qb)
        gpu.gpu_buffer_2d_write(ctx, Kh, Kb)
        gpu.gpu_buffer_2d_write(ctx, Vh, Vb)
        step_device()
        gpu.gpu_buffer_2d_read(ctx, Ob, Oh)

    step_e2e()
    e2e_steps = max(2, min(steps, 5))
    ms_e2e = timed(step_e2e, e2e_steps) / e2e_steps
    clocks = sampler.finish()
    flops = 4.0 * B * H * D * N * (N + 1) / 2
    sustained, burst, kind = measured_tensor_peak()
    achieved = flops / (ms_step * 1e-3) / 1e12
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        from oracle import c_oracle

        hs = 4  # heads of one sequence timed on the CPU
        sl = lambda X: np.ascontiguousarray(  # noqa: E731
            X.reshape(B, N, H, D)[0, :, :hs, :].reshape(N, hs * D).cpu().view(torch.int16).numpy().view(np.uint16))
        t0 = time.perf_counter()
        c_oracle.prefill(sl(Q), sl(K), sl(V), 1, N, hs, D, want_stats=False)
        dt = time.perf_counter() - t0
        cpu = {"value": N * hs / H / dt, "unit": "tokens/s", "cores": c_oracle.num_threads(), "kind": "port",
               "sample": f"{hs} of {H} heads of one sequence ({dt:.2f} s); value counts {hs}/{H} of a token per row"}
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if rank != 0:
        return
    line = {
        "metric": "prefill tokens/s", "value": world * B * N / (ms_step * 1e-3), "unit": "tokens/s", "n_gpus": world,
        "steps": steps, "warmup": warm, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16 operands, fp32 accumulate", "data": "synthetic",
        "config": {"workload": w["desc"], "batch_per_gpu": B, "global_batch": world * B,
                   "l2": "Q/K/V/O/cache (1.6 GB per step) larger than L2, no flush",
                   "parallelism": f"batch-sharded x{world}, no collective"},
        "e2e": {"value": world * B * N / (ms_e2e * 1e-3), "unit": "tokens/s", "ms_per_step": ms_e2e,
                "h2d_bytes_per_step": 3 * B * N * E * 2, "d2h_bytes_per_step": B * N * E * 2},
        "gpu_launches": steps, "clocks": clocks,
        "roofline": {"bound": "tensor", "kernel": "prefill_tc_kernel", "achieved": achieved, "peak": sustained,
                     "unit": "TFLOP/s", "frac": achieved / sustained, "frac_of_burst": achieved / burst,
                     "peak_kind": kind + " (sustained cuBLAS bf16; kernel timed in a loop)",
                     "algorithmic_flops_per_launch": flops,
                     "traffic": B * PREFILL_DRAM_BYTES_PER_SEQUENCE if (H, D, N) == (32, 128, 4096) else None},
        "cpu_baseline": cpu,
    }
    print(json.dumps(line), flush=True)


def run_qkv_append(args, w, rank, world):
    """One decode step's Q/K/V projection fused with the cache append; value = tokens/s, roofline = HBM
    (the step streams 3*E*E weights).  The layers' weights (4 x 100 MB) are used in turn, so that a step's
    weights are not in L2 from the step before."""
    import torch
    import torch.distributed as dist

    import __graft_entry__

    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    pkg = __graft_entry__.import_package()
    gpu = pkg.gpu
    ctx = gpu.context_create(local_rank)
    B, H, D, T, n_layers = w["B"], w["H"], w["D"], w["T"], w["layers"]
    E = H * D
    dtype = torch.bfloat16
    gen = torch.Generator(device=device).manual_seed(3000 + rank)
    rnd = lambda shape, scale: (torch.randn(shape, generator=gen, device=device) * scale).to(dtype)  # noqa: E731
    wrap = lambda t: gpu.GPUBuffer2D(buffer=t, shape=tuple(t.shape), size=t.numel())  # noqa: E731
    weights = [[wrap(rnd((E, E), E ** -0.5)) for _ in range(3)] for _ in range(n_layers)]
    x, q = rnd((B, E), 1.0), torch.empty((B, E), dtype=dtype, device=device)
    xb, qb = wrap(x), wrap(q)
    cache = gpu.kv_cache_create(ctx, gpu.KVCacheConfig(batch_size=B, max_seq_len=T, n_layers=n_layers, n_heads=H,
                                                       head_dim=D, dtype=dtype, layout="bhtd", ragged=True))
    lens = np.random.default_rng(0).integers(0, T - 1, size=B).astype(np.int32)
    gpu.kv_cache_set_lengths(cache, lens)
    state = {"i": 0}

    def step_device():
        li = state["i"] % n_layers
        state["i"] += 1
        gpu.batch_begin(ctx)
        gpu.qkv_project_append(ctx, cache, li, xb, *weights[li], qb, advance=False)
        gpu.batch_commit(ctx)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device=device, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        barrier()
        return ms

    steps, warm = args.steps, max(3, args.warmup)
    for _ in range(warm):
        step_device()
    sampler = ClockSampler(physical_gpu_index(local_rank))
    sampler.start()
    ms_step = timed(step_device, steps) / steps
    xh, qh = x.cpu().pin_memory(), torch.empty_like(q, device="cpu").pin_memory()

    def step_e2e():
        gpu.gpu_buffer_2d_write(ctx, xh, xb)
        step_device()
        gpu.gpu_buffer_2d_read(ctx, qb, qh)

    step_e2e()
    ms_e2e = timed(step_e2e, steps) / steps
    clocks = sampler.finish()
    es = 2
    bytes_step = 3 * E * E * es + B * E * es + 3 * B * E * es
    peak, kind = measured_hbm_peak()
    achieved = bytes_step / (ms_step * 1e-3) / 1e9
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        from oracle import kv_oracle

        f32 = lambda t: t.float().cpu().numpy()  # noqa: E731
        xs, ws = f32(x), [f32(t.buffer) for t in weights[0]]
        reps = 3
        t0 = time.perf_counter()
        for _ in range(reps):
            kv_oracle.qkv_project(xs, *ws)
        dt = (time.perf_counter() - t0) / reps
        cpu = {"value": B / dt, "unit": "tokens/s", "cores": os.cpu_count(), "kind": "port",
               "sample": f"the three projections of one step in float64 numpy ({dt:.2f} s per step)"}
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if rank != 0:
        return
    line = {
        "metric": "projected tokens/s (one layer's Q/K/V projection + cache append per step)",
        "value": world * B / (ms_step * 1e-3), "unit": "tokens/s", "n_gpus": world, "steps": steps, "warmup": warm,
        "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16 operands, fp32 accumulate", "data": "synthetic",
        "config": {"workload": w["desc"], "batch_per_gpu": B, "global_batch": world * B,
                   "l2": f"{n_layers} layers' weights ({n_layers * 3 * E * E * es / 1e6:.0f} MB) used in turn, larger than L2",
                   "parallelism": f"batch-sharded x{world}, no collective"},
        "e2e": {"value": world * B / (ms_e2e * 1e-3), "unit": "tokens/s", "ms_per_step": ms_e2e,
                "h2d_bytes_per_step": B * E * es, "d2h_bytes_per_step": B * E * es},
        "gpu_launches": steps, "clocks": clocks,
        "roofline": {"bound": "hbm", "kernel": "qkv_append_kernel", "achieved": achieved, "peak": peak, "unit": "GB/s",
                     "frac": achieved / peak, "peak_kind": kind, "algorithmic_bytes_per_launch": bytes_step,
                     "traffic": None},
        "cpu_baseline": cpu,
    }
    print(json.dumps(line), flush=True)


def run_decode_layer(args, w, rank, world):
    """One whole decoder layer per step: layernorm, Q/K/V projection + append, cached attention, output
    projection + residual, layernorm, MLP.  value = tokens/s through one layer; roofline = HBM over the bytes
    the step must move (K/V rows attended + 12 E^2 weights + the small row buffers)."""
    import torch
    import torch.distributed as dist

    import __graft_entry__

    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    pkg = __graft_entry__.import_package()
    gpu = pkg.gpu
    from llm_experiments_b200 import decode_layer

    ctx = gpu.context_create(local_rank)
    B, H, D, n_layers = w["B"], w["H"], w["D"], w["layers"]
    E, T_max = H * D, w["hi"] + 8
    dtype = torch.bfloat16
    gen = torch.Generator(device=device).manual_seed(4000 + rank)
    rnd = lambda shape, scale=1.0: (torch.randn(shape, generator=gen, device=device) * scale).to(dtype)  # noqa: E731
    b2 = lambda t: gpu.GPUBuffer2D(buffer=t, shape=tuple(t.shape), size=t.numel())  # noqa: E731
    b1 = lambda t: gpu.GPUBuffer1D(buffer=t, shape=tuple(t.shape), size=t.numel())  # noqa: E731

    def make_weights():
        raw = dict(ln1_gamma=rnd((E,), 0.1) + 1, ln1_beta=rnd((E,), 0.1), wq=rnd((E, E), E ** -0.5), wk=rnd((E, E), E ** -0.5),
                   wv=rnd((E, E), E ** -0.5), wo=rnd((E, E), E ** -0.5), ln2_gamma=rnd((E,), 0.1) + 1, ln2_beta=rnd((E,), 0.1),
                   w1=rnd((E, 4 * E), E ** -0.5), b1=rnd((4 * E,), 0.1), w2=rnd((4 * E, E), (4 * E) ** -0.5), b2=rnd((E,), 0.1))
        return decode_layer.DecoderLayerWeights(**{k: (b1(v) if v.dim() == 1 else b2(v)) for k, v in raw.items()})

    weights = [make_weights() for _ in range(n_layers)]
    lens = make_lengths(w, 0)
    caches = []
    for _ in range(n_layers):
        c = gpu.kv_cache_create(ctx, gpu.KVCacheConfig(batch_size=B, max_seq_len=T_max, n_layers=1, n_heads=H, head_dim=D,
                                                       dtype=dtype, layout="bhtd", ragged=True))
        c.layers[0].k_cache.buffer.normal_(generator=gen)
        c.layers[0].v_cache.buffer.normal_(generator=gen)
        gpu.kv_cache_set_lengths(c, lens)
        caches.append(c)
    lens_dev, max_len = torch.from_numpy(lens.astype(np.int32)).to(device), int(lens.max())
    x, y = rnd((B, E)), torch.empty((B, E), dtype=dtype, device=device)
    xb, yb = b2(x), b2(y)
    scratch = decode_layer.decoder_layer_scratch(ctx, B, E)
    state = {"i": 0}

    def step_device():
        li = state["i"] % n_layers
        state["i"] += 1
        cache = caches[li]
        cache.seq_lens.copy_(lens_dev)  # every step starts from the same lengths (256 bytes, device to device)
        cache.current_len = max_len
        gpu.batch_begin(ctx)
        decode_layer.decoder_layer_step(ctx, cache, xb, weights[li], scratch, yb)
        gpu.batch_commit(ctx)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device=device, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        barrier()
        return ms

    steps, warm = args.steps, max(3, args.warmup)
    for _ in range(warm):
        step_device()
    sampler = ClockSampler(physical_gpu_index(local_rank))
    sampler.start()
    ms_step = timed(step_device, steps) / steps
    xh, yh = x.cpu().pin_memory(), torch.empty_like(y, device="cpu").pin_memory()

    def step_e2e():
        gpu.gpu_buffer_2d_write(ctx, xh, xb)
        step_device()
        gpu.gpu_buffer_2d_read(ctx, yb, yh)

    step_e2e()
    ms_e2e = timed(step_e2e, steps) / steps
    clocks = sampler.finish()
    es = 2
    kv_bytes = int((lens.astype(np.int64) + 1).sum()) * H * D * es * 2
    weight_bytes = 12 * E * E * es
    row_bytes = B * E * es * 14 + B * 4 * E * es * 2  # the [B, E] and [B, 4E] row buffers read / written between kernels
    bytes_step = kv_bytes + weight_bytes + row_bytes
    peak, kind = measured_hbm_peak()
    achieved = bytes_step / (ms_step * 1e-3) / 1e9
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if rank != 0:
        return
    line = {
        "metric": "tokens/s through one decoder layer (cached decode step)", "value": world * B / (ms_step * 1e-3),
        "unit": "tokens/s", "n_gpus": world, "steps": steps, "warmup": warm, "ms_per_step": ms_step,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16 storage, fp32 arithmetic",
        "data": "synthetic",
        "config": {"workload": w["desc"], "batch_per_gpu": B, "global_batch": world * B,
                   "l2": f"{n_layers} layers' caches and weights used in turn, far larger than L2",
                   "parallelism": f"batch-sharded x{world}, no collective"},
        "e2e": {"value": world * B / (ms_e2e * 1e-3), "unit": "tokens/s", "ms_per_step": ms_e2e,
                "h2d_bytes_per_step": B * E * es, "d2h_bytes_per_step": B * E * es},
        "gpu_launches": steps * 8, "clocks": clocks,
        "roofline": {"bound": "hbm", "kernel": "the layer's 8 kernels together", "achieved": achieved, "peak": peak,
                     "unit": "GB/s", "frac": achieved / peak, "peak_kind": kind,
                     "algorithmic_bytes_per_launch": bytes_step, "kv_bytes": kv_bytes, "weight_bytes": weight_bytes,
                     "traffic": None},
        "cpu_baseline": None,
    }
    print(json.dumps(line), flush=True)


def run_prompt_layer(args, w, rank, world):
    """One whole decoder layer over a prompt per step: layernorm, three projection GEMMs, causal attention
    fused with the cache write, output projection + residual, layernorm, MLP.  value = prompt tokens/s
    through one layer; roofline = tensor, over the layer's matmul and attention flops."""
    import torch
    import torch.distributed as dist

    import __graft_entry__

    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    pkg = __graft_entry__.import_package()
    gpu = pkg.gpu
    from llm_experiments_b200 import decode_layer

    ctx = gpu.context_create(local_rank)
    ctx.config.flash_attn_max_head_dim = 128
    B, H, D, N, n_layers = w["B"], w["H"], w["D"], w["N"], w["layers"]
    E, rows = H * D, B * N
    dtype = torch.bfloat16
    gen = torch.Generator(device=device).manual_seed(5000 + rank)
    rnd = lambda shape, scale=1.0: (torch.randn(shape, generator=gen, device=device) * scale).to(dtype)  # noqa: E731
    b2 = lambda t: gpu.GPUBuffer2D(buffer=t, shape=tuple(t.shape), size=t.numel())  # noqa: E731
    b1 = lambda t: gpu.GPUBuffer1D(buffer=t, shape=tuple(t.shape), size=t.numel())  # noqa: E731

    def make_weights():
        raw = dict(ln1_gamma=rnd((E,), 0.1) + 1, ln1_beta=rnd((E,), 0.1), wq=rnd((E, E), E ** -0.5), wk=rnd((E, E), E ** -0.5),
                   wv=rnd((E, E), E ** -0.5), wo=rnd((E, E), E ** -0.5), ln2_gamma=rnd((E,), 0.1) + 1, ln2_beta=rnd((E,), 0.1),
                   w1=rnd((E, 4 * E), E ** -0.5), b1=rnd((4 * E,), 0.1), w2=rnd((4 * E, E), (4 * E) ** -0.5), b2=rnd((E,), 0.1))
        return decode_layer.DecoderLayerWeights(**{k: (b1(v) if v.dim() == 1 else b2(v)) for k, v in raw.items()})

    weights = [make_weights() for _ in range(n_layers)]
    caches = [gpu.kv_cache_create(ctx, gpu.KVCacheConfig(batch_size=B, max_seq_len=N, n_layers=1, n_heads=H, head_dim=D,
                                                         dtype=dtype, layout="bhtd")) for _ in range(n_layers)]
    x, y = rnd((rows, E)), torch.empty((rows, E), dtype=dtype, device=device)
    xb, yb = b2(x), b2(y)
    scratch = decode_layer.prompt_layer_scratch(ctx, rows, E)
    state = {"i": 0}

    def step_device():
        li = state["i"] % n_layers
        state["i"] += 1
        gpu.batch_begin(ctx)
        decode_layer.prompt_layer_step(ctx, caches[li], xb, weights[li], scratch, yb, B, N)
        gpu.batch_commit(ctx)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device=device, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        barrier()
        return ms

    steps, warm = min(args.steps, 50), max(3, args.warmup)
    for _ in range(warm):
        step_device()
    sampler = ClockSampler(physical_gpu_index(local_rank))
    sampler.start()
    ms_step = timed(step_device, steps) / steps
    xh, yh = x.cpu().pin_memory(), torch.empty_like(y, device="cpu").pin_memory()

    def step_e2e():
        gpu.gpu_buffer_2d_write(ctx, xh, xb)
        step_device()
        gpu.gpu_buffer_2d_read(ctx, yb, yh)

    step_e2e()
    e2e_steps = max(2, min(steps, 5))
    ms_e2e = timed(step_e2e, e2e_steps) / e2e_steps
    clocks = sampler.finish()
    es = 2
    gemm_flops = 2.0 * rows * E * E * 12  # Q, K, V, Wo (4 E^2) + the MLP (8 E^2)
    attn_flops = 4.0 * B * H * D * N * (N + 1) / 2
    flops = gemm_flops + attn_flops
    sustained, burst, kind = measured_tensor_peak()
    achieved = flops / (ms_step * 1e-3) / 1e12
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if rank != 0:
        return
    line = {
        "metric": "prompt tokens/s through one decoder layer", "value": world * rows / (ms_step * 1e-3),
        "unit": "tokens/s", "n_gpus": world, "steps": steps, "warmup": warm, "ms_per_step": ms_step,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16 operands, fp32 accumulate",
        "data": "synthetic",
        "config": {"workload": w["desc"], "batch_per_gpu": B, "global_batch": world * B, "seq_len": N,
                   "l2": f"{n_layers} layers' weights used in turn; activations ({rows * E * es / 1e6:.0f} MB per buffer) "
                         "larger than L2",
                   "parallelism": f"batch-sharded x{world}, no collective"},
        "e2e": {"value": world * rows / (ms_e2e * 1e-3), "unit": "tokens/s", "ms_per_step": ms_e2e,
                "h2d_bytes_per_step": rows * E * es, "d2h_bytes_per_step": rows * E * es},
        "gpu_launches": steps * 9, "clocks": clocks,
        "roofline": {"bound": "tensor", "kernel": "the layer's 9 kernels together (6 gemm_tc_kernel, prefill_tc_kernel, "
                                                  "2 layernorm)",
                     "achieved": achieved, "peak": sustained, "unit": "TFLOP/s", "frac": achieved / sustained,
                     "frac_of_burst": achieved / burst,
                     "peak_kind": f"{kind} (sustained cuBLAS bf16; the layer is timed in a long loop)",
                     "algorithmic_flops_per_launch": flops, "gemm_flops": gemm_flops, "attention_flops": attn_flops,
                     "traffic": None},
        "cpu_baseline": None,
    }
    print(json.dumps(line), flush=True)


# dram__bytes_read.sum + dram__bytes_write.sum of the split kernel per attended (token, head), from
# an ncu capture of the 8-sequence case (`--workload decode_small`: 412.4 MB for
# 24908 tokens x 32 heads; the algorithmic figure is 512 B).  Traffic grows in proportion to the
# tokens attended, so a full launch is this figure times its tokens and heads.
DRAM_BYTES_PER_TOKEN_HEAD = 517.4


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="decode", choices=sorted(WORKLOADS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--fused-gather", action="store_true",
                    help="head-split workloads: gather the outputs with peer stores from the merge kernel instead of NCCL")
    ap.add_argument("--tune", action="append", default=[], metavar="NAME=VALUE",
                    help="set a kernel tuning knob of the library (b2kv_tune), e.g. prefill_variant=1")
    args = ap.parse_args()
    if args.tune and args.impl != "reference":
        import __graft_entry__

        native = __graft_entry__.import_package()._native
        for item in args.tune:
            name, _, value = item.partition("=")
            native.tune(name, int(value))
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    w = WORKLOADS[args.workload]
    w.setdefault("block_size", 0)
    if w.get("prefill") and args.impl != "reference":
        run_prefill(args, w, rank, world)
        return
    if w.get("qkv") and args.impl != "reference":
        run_qkv_append(args, w, rank, world)
        return
    if w.get("layer_step") and args.impl != "reference":
        run_decode_layer(args, w, rank, world)
        return
    if w.get("prompt_layer") and args.impl != "reference":
        run_prompt_layer(args, w, rank, world)
        return
    if args.impl == "reference":
        run_reference(args, w, rank)
        return
    if world != args.gpus:
        if args.gpus != 1 and world == 1:
            raise SystemExit("launch with torchrun for --gpus > 1")
    run_b200(args, w, rank, world)


if __name__ == "__main__":
    main()
