#!/usr/bin/env python3
"""Benchmark of the KV-cache attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--repeats R] [--impl b200|reference]
                    [--workload NAME] [--only]

One "step" is one pass of the hot path over one batch of synthetic input: append one new
K/V row per sequence, then single-token attention over the whole cache (one layer).  The
headline workload is the decode microbenchmark (batch 64, 32 heads, head_dim 128, bf16,
per-sequence cache length uniform in [512, 8192] from seed 0); the cache (9 GB) is far
larger than L2, so no flush is needed between steps.  With N > 1 every rank (one per GPU,
launched by torchrun) owns its own batch of 64 sequences and there is no collective in the
step (weak scaling); time is the maximum over ranks.

Rank 0 prints ONE JSON line.  ``value`` is decode tokens/s with inputs resident in HBM;
``e2e`` is the same step through the public API with host buffers (one pinned host -> device
copy of q, new K and new V and the device -> host read of the output inside the timed
region); ``roofline`` is the decode kernel's algorithmic HBM bytes over its CUDA-event time
against the measured copy bandwidth; ``cpu_baseline`` is the CPU oracle (a port of the
reference math, all host threads) on the same 64 sequences.  Every timed loop of K steps is
repeated R times; the figures are medians over the repeats, with the fastest and slowest beside
them.

With the default workload the same line carries, measured in the same process after the
headline loops (each cache is freed before the next is built):

* ``workloads.paged``, ``workloads.prefill``, ``workloads.longctx``: the other single-GPU
  configurations (paged decode through a block table, causal prefill on the tensor cores fused
  with the cache write, long-context decode), each with its own roofline and clocks;
* with N > 1: ``parity_multi`` (a small head-split decode gathered with NCCL and with the
  peer stores of the merge kernel, and a sequence-split decode, each checked on rank 0 against
  the CPU oracle outside every timed region), ``workloads.decode_strong`` (the 64 sequences cut
  into N sets of 64 / N, as contiguous slices and balanced by the tokens attended, no collective) and ``workloads.longctx_headsplit`` (the long
  context with its heads split over the GPUs, outputs gathered by NCCL and by the fused peer
  stores).

``--workload NAME --only`` times a single workload (used for profiler captures).

``--impl reference`` times the CPU port alone: the reference itself has no CPU or CUDA
implementation of this path that can run here (its kernels are WGSL dispatched through
wgpu / Vulkan, and this machine has no graphics stack).
"""
from __future__ import annotations

import argparse
import gc
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
    "decode": dict(kind="decode", B=64, H=32, D=128, lo=512, hi=8192, block_size=0,
                   desc="decode microbench: B=64 H=32 D=128 bf16, len~U[512,8192] seed 0, [B,H,T,D] cache"),
    "decode_small": dict(kind="decode", B=8, H=32, D=128, lo=512, hi=8192, block_size=0,
                         desc="decode microbench cut to 8 sequences (1.2 GB cache, for profiler captures)"),
    "decode_strong": dict(kind="decode", B=64, H=32, D=128, lo=512, hi=8192, block_size=0, strong=True,
                          desc="decode microbench, its 64 sequences cut into contiguous slices of 64 / N over the GPUs"),
    "paged": dict(kind="decode", B=64, H=32, D=128, lo=512, hi=8192, block_size=16,
                  desc="paged decode: same shapes, 16-token blocks placed by a seeded permutation of 65536 blocks"),
    "longctx": dict(kind="decode", B=4, H=64, D=128, lo=131072, hi=131072, block_size=0,
                    desc="long-context decode: B=4 H=64 D=128 bf16, len 131072, batch-resident on one GPU"),
    "longctx_headsplit": dict(kind="decode", B=4, H=64, D=128, lo=131072, hi=131072, block_size=0, head_split=True,
                              desc="long-context decode: B=4 H=64 D=128 bf16, len 131072, heads split over the "
                                   "GPUs, outputs all-gathered"),
    "qkv_append": dict(kind="qkv", B=64, H=32, D=128, T=256, layers=4,
                       desc="Q/K/V projection fused with the cache append: B=64 E=4096 (H=32 D=128) bf16, one layer per step"),
    "decode_layer": dict(kind="layer_step", B=64, H=32, D=128, lo=512, hi=8192, layers=2,
                         desc="one decoder layer of a cached decode step (LN, QKV+append, attention, Wo, LN, MLP): "
                              "B=64 E=4096 (H=32 D=128) bf16, len~U[512,8192] seed 0"),
    "prefill_layer": dict(kind="prompt_layer", B=8, H=32, D=128, N=4096, layers=2,
                          desc="one decoder layer over a whole prompt (LN, Q/K/V GEMMs, causal attention + cache write, Wo, "
                               "LN, MLP): B=8 N=4096 E=4096 (H=32 D=128) bf16"),
    "prefill_layer_small": dict(kind="prompt_layer", B=1, H=32, D=128, N=4096, layers=2,
                                desc="the prompt-side layer cut to one sequence (for profiler captures)"),
    "prefill_small": dict(kind="prefill", B=2, H=32, D=128, N=4096,
                          desc="causal prefill cut to 2 sequences (for profiler captures)"),
    "prefill": dict(kind="prefill", B=8, H=32, D=128, N=4096,
                    desc="causal prefill: B=8 H=32 D=128 N=4096 bf16, fused with the K/V cache write"),
    "prefill_f32": dict(kind="prefill", B=2, H=32, D=128, N=4096, f32=True,
                        desc="causal prefill of fp32 prompts (the reference's storage type) on the tensor cores, operands split "
                             "into bfloat16 halves: B=2 H=32 D=128 N=4096, fused with the K/V cache write"),
    "model_step": dict(kind="model_step", B=64, H=32, D=128, lo=512, hi=8192, layers=4, vocab=32768,
                       desc="one cached decode step of a 4-layer bf16 decoder (E=4096, H=32, vocab 32768): embedding, "
                            "4 decoder layers, final layernorm, logits, argmax; B=64, len~U[512,8192] seed 0"),
    "model_step_small": dict(kind="model_step", B=8, H=32, D=128, lo=128, hi=1024, layers=4, vocab=32768,
                             desc="the same 4-layer decoder at B=8 with short contexts, len~U[128,1024] seed 0: a step is "
                                  "bound by its 36 launches, so it is also timed as one replayed CUDA graph"),
}
SLACK = 1024  # rows of head-room above the longest sequence for the appended tokens

# DRAM traffic constants from ncu captures of small cases (dram__bytes_read.sum + dram__bytes_write.sum), scaled by
# the units a full launch processes.  They describe the DEFAULT kernel variants only and have to be captured again
# (small case, one kernel, --clock-control none) whenever a kernel or its launch order changes; a run with any
# --tune knob reports no traffic.
#   decode_split_kernel<bf16, 128, 64, 3, 8>: 412.6 MB for 24908 tokens x 32 heads of `--workload decode_small`
#   (profiles/decode_split_kernel_decode_small.md); the algorithmic figure is 512 B per attended (token, head).
DRAM_BYTES_PER_TOKEN_HEAD = 517.7
#   prefill_tc_kernel<128> with launch groups: 212.7 MB read + 155.1 MB written for the 2 sequences of
#   `--workload prefill_small` (profiles/prefill_tc_kernel_prefill_small.md); algorithmic: 6 x 33.5 MB per sequence.
PREFILL_DRAM_BYTES_PER_SEQUENCE = int((212.7e6 + 155.1e6) / 2)


def measured_peaks():
    """(HBM GB/s, bf16 TFLOP/s sustained, bf16 TFLOP/s burst, "measured" | "fallback")."""
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        try:
            d = json.loads(path.read_text())
            return float(d["hbm_gbs"]), float(d["bf16_tflops_sustained"]), float(d["bf16_tflops"]), "measured"
        except Exception:
            pass
    return 6650.0, 1400.0, 1590.0, "fallback"


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


def make_lengths(w, seed=0):
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


def headline_config(w, world):
    """`config` of the JSON line; the GPU arm and the CPU arm of the same workload print the same one."""
    return {"workload": w["desc"], "batch_per_gpu": w["B"], "global_batch": world * w["B"],
            "sum_len_rank0": int(np.sum(make_lengths(w))) if "lo" in w else None,
            "l2": "inputs (GBs of cache) far larger than L2, no flush",
            "parallelism": f"batch-sharded x{world}, no collective in the step"}


# ------------------------------------------------------------------------------------------
# harness shared by every GPU workload
# ------------------------------------------------------------------------------------------

class Harness:
    """Device, process group, library context and the timing rules: W >= 3 warm-up steps, then R repeats of
    exactly K steps between two CUDA events on the launching stream, a barrier and a device synchronisation on
    both sides of every repeat, the maximum over ranks per repeat, the median over the repeats."""

    def __init__(self, args):
        import torch
        import torch.distributed as dist

        import __graft_entry__

        self.torch, self.dist, self.args = torch, dist, args
        self.rank = int(os.environ.get("RANK", "0"))
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        torch.cuda.set_device(self.local_rank)
        self.device = torch.device("cuda", self.local_rank)
        if self.world > 1:
            # the fused gather's peers must not be bound to an NVLink multicast object; the collectives here
            # are a few KB, so in-switch reduction has nothing to offer them either
            os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
            dist.init_process_group("nccl", device_id=self.device)
        self.pkg = __graft_entry__.import_package()
        self.gpu = self.pkg.gpu
        self.ctx = self.gpu.context_create(self.local_rank)
        self.steps = max(1, args.steps)
        self.warmup = max(3, args.warmup)
        self.repeats = max(1, args.repeats)
        self.tuned = bool(args.tune)

    def wrap(self, t):
        return self.gpu.GPUBuffer2D(buffer=t, shape=tuple(t.shape), size=t.numel())

    def wrap1(self, t):
        return self.gpu.GPUBuffer1D(buffer=t, shape=tuple(t.shape), size=t.numel())

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
        self.torch.cuda.synchronize()

    def timed(self, fn, steps):
        """K steps between two events on the launching stream; returns ms (max over ranks)."""
        torch = self.torch
        self.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        if self.world > 1:
            t = torch.tensor([ms], device=self.device, dtype=torch.float64)
            self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
            ms = float(t.item())
        self.barrier()
        return ms

    def measure(self, fn, steps=None, warmup=None, repeats=None, before_repeat=None):
        """Warm-up, then `repeats` timed loops of `steps` steps.  Returns per-step milliseconds:
        {"ms": median, "min": ..., "max": ..., "repeats": R, "steps": K}."""
        steps = self.steps if steps is None else steps
        warmup = self.warmup if warmup is None else warmup
        repeats = self.repeats if repeats is None else repeats
        if before_repeat:
            before_repeat()
        for _ in range(warmup):
            fn()
        per_step = []
        for _ in range(repeats):
            if before_repeat:
                before_repeat()
            per_step.append(self.timed(fn, steps) / steps)
        return {"ms": float(np.median(per_step)), "min": float(min(per_step)), "max": float(max(per_step)),
                "repeats": repeats, "steps": steps}

    def sampler(self):
        s = ClockSampler(physical_gpu_index(self.local_rank))
        s.start()
        return s

    def release(self):
        gc.collect()
        self.torch.cuda.empty_cache()

    def finish(self):
        if self.world > 1:
            self.dist.barrier()
            self.dist.destroy_process_group()


def spread(m, prefix="ms_per_step"):
    return {prefix: m["ms"], prefix + "_min": m["min"], prefix + "_max": m["max"], "repeats": m["repeats"]}


def fill_normal(torch, buf, gen, dtype):
    """N(0,1) values in `dtype`, drawn in slabs to bound the fp32 temporary."""
    flat = buf.view(-1)
    slab = 1 << 28
    for off in range(0, flat.numel(), slab):
        n = min(slab, flat.numel() - off)
        flat[off:off + n] = torch.randn(n, generator=gen, device=buf.device, dtype=torch.float32).to(dtype)


# ------------------------------------------------------------------------------------------
# decode workloads (contiguous, paged, long context, batch-sharded, head-split)
# ------------------------------------------------------------------------------------------

def run_decode(h: Harness, w, *, gather="nccl", cpu_baseline=False, assign="contiguous"):
    """Append + decode over one layer's cache.  Returns the record of the workload (every rank computes it; the
    figures are maxima over ranks)."""
    torch, gpu, ctx = h.torch, h.gpu, h.ctx
    from llm_experiments_b200 import sharding

    rank, world, device = h.rank, h.world, h.device
    B_total, H_total, D, bs = w["B"], w["H"], w["D"], w["block_size"]
    head_split = bool(w.get("head_split")) and world > 1
    strong = bool(w.get("strong")) and world > 1
    lens_all = make_lengths(w)
    B, H, lens0 = B_total, H_total, lens_all
    if head_split:
        h0, h1 = sharding.head_range(H_total, rank, world)  # this rank's heads of every sequence
        H = h1 - h0
    if strong:
        if assign == "balanced":  # sequences dealt so that every rank attends about the same number of tokens
            mine = sharding.balanced_assignment(lens_all, world)[rank]
        else:  # this rank's contiguous slice of the sequences
            mine = list(range(*sharding.shard_range(B_total, rank, world)))
        B, lens0 = len(mine), lens_all[mine]
    E = H * D
    dtype = torch.bfloat16
    steps = h.steps
    # head-room for the rows appended by the longest timed loop (lengths are reset before every loop)
    slack = max(SLACK, steps + h.warmup + 64)
    T_max = int(lens_all.max()) + slack
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
        fill_normal(torch, buf, gen, dtype)
    # the step's inputs (q, new K row, new V row of every sequence) live in one buffer, so that the end-to-end
    # step uploads them with one host -> device copy
    qkv_dev = torch.randn((3 * B, E), generator=gen, device=device, dtype=torch.float32).to(dtype)
    q_dev, nk_dev, nv_dev = qkv_dev[:B], qkv_dev[B:2 * B], qkv_dev[2 * B:]
    out_dev = torch.empty((B, E), device=device, dtype=dtype)
    q_b, nk_b, nv_b, out_b, qkv_b = h.wrap(q_dev), h.wrap(nk_dev), h.wrap(nv_dev), h.wrap(out_dev), h.wrap(qkv_dev)

    def reset_lengths():
        gpu.kv_cache_set_lengths(cache, lens0)

    fused = sharding.FusedHeadGather(device, B, H_total, D, dtype) if (head_split and gather == "fused") else None

    def step_device():
        gpu.batch_begin(ctx)
        gpu.kv_cache_update(ctx, cache, 0, nk_b, nv_b)
        if fused is not None:
            full = fused.decode(ctx, cache, 0, q_b)  # the decode kernel stores into every rank's buffer
        else:
            gpu.attention_with_kv_cache(ctx, cache, 0, q_b, out_b)
            full = None
        gpu.batch_commit(ctx)
        if head_split and fused is None:
            full = sharding.gather_heads(out_dev)  # NCCL all-gather: [B, H_total*D] on every rank
        return full

    sampler = h.sampler()  # runs across the timed loops below
    # ---- value: inputs resident in HBM -------------------------------------------------
    m_step = h.measure(step_device, before_repeat=reset_lengths)
    seqs_total = B_total if (head_split or strong) else world * B_total
    tokens_per_s = seqs_total / (m_step["ms"] * 1e-3)

    # ---- roofline: the decode call (split kernel + combine) alone, CUDA events ---------
    def decode_state():
        reset_lengths()
        cache.seq_lens.add_(1)  # the state the decode sees inside a step
        cache.current_len = int(lens0.max()) + 1

    def decode_only():
        gpu.batch_begin(ctx)
        gpu.attention_with_kv_cache(ctx, cache, 0, q_b, out_b)
        gpu.batch_commit(ctx)

    decode_state()
    m_dec = h.measure(decode_only, warmup=3)
    kv_bytes, step_bytes = algorithmic_bytes(lens0 + 1, H, D, 2, B, bs)
    dec_bytes = kv_bytes + 2 * B * E * 2 + (4 * int(np.sum((lens0 + bs) // bs)) if bs else 0)
    hbm_peak, _, _, peak_kind = measured_peaks()
    achieved = dec_bytes / (m_dec["ms"] * 1e-3) / 1e9

    # ---- e2e: host buffers through the public API --------------------------------------
    qkv_host = qkv_dev.cpu().pin_memory()
    out_host = torch.empty((B, E), dtype=dtype).pin_memory()
    out_host_full = torch.empty((B, H_total * D), dtype=dtype).pin_memory()

    def step_e2e():
        gpu.gpu_buffer_2d_write(ctx, qkv_host, qkv_b)
        full = step_device()
        if head_split:
            out_host_full.copy_(full, non_blocking=True)
            torch.cuda.current_stream().synchronize()
        else:
            gpu.gpu_buffer_2d_read(ctx, out_b, out_host)  # blocks until the result is on the host

    m_e2e = h.measure(step_e2e, warmup=3, before_repeat=reset_lengths)
    clocks = sampler.finish()
    e2e_tps = seqs_total / (m_e2e["ms"] * 1e-3)
    status = int(ctx.dev_status.item()) if ctx.dev_status is not None else 0

    default_variant = (not h.tuned) and not bs and D == 128
    traffic = int(DRAM_BYTES_PER_TOKEN_HEAD * float(np.sum(lens0 + 1)) * H) if default_variant else None
    launches_per_step = 2 + (1 if fused is not None else 0)  # append, split (+ the flag wait of the fused gather)
    if head_split:
        par = (f"heads split x{world}, outputs gathered "
               + ("by peer stores fused into the decode kernel" if fused is not None
                  else "with one NCCL all-gather per step"))
    elif strong:
        par = (f"the batch cut into {world} sets of {B_total}/{world} sequences ("
               + ("balanced by tokens attended" if assign == "balanced" else "contiguous slices")
               + "), no collective in the step")
    else:
        par = f"batch-sharded x{world}, no collective in the step"
    rec = {
        "metric": "decode tokens/s", "value": tokens_per_s, "unit": "tokens/s",
        **spread(m_step),
        "scaling": "strong" if (head_split or strong) else "weak",
        "config": {"workload": w["desc"], "batch_per_gpu": B, "global_batch": seqs_total,
                   "sum_len_rank0": int(np.sum(lens0)), "l2": "inputs (GBs of cache) far larger than L2, no flush",
                   "parallelism": par},
        "e2e": {"value": e2e_tps, "unit": "tokens/s", **spread(m_e2e), "h2d_bytes_per_step": 3 * B * E * 2,
                "d2h_bytes_per_step": B * (H_total if head_split else H) * D * 2},
        "gpu_launches": launches_per_step * steps * h.repeats,
        "gpu_launches_per_step": launches_per_step,
        "clocks": clocks,
        "dev_status": status,
        "roofline": {"bound": "hbm", "kernel": "decode_split_kernel (one b2kv_decode call; the partials are merged inside it)",
                     "achieved": achieved, "peak": hbm_peak, "unit": "GB/s", "frac": achieved / hbm_peak,
                     "frac_of_8000_nominal": achieved / 8000.0, "peak_kind": peak_kind,
                     "ms_per_launch": m_dec["ms"], "ms_per_launch_min": m_dec["min"], "ms_per_launch_max": m_dec["max"],
                     "algorithmic_bytes_per_launch": dec_bytes, "traffic": traffic,
                     "traffic_source": ("ncu capture of the 8-sequence case of the default kernel variant, scaled by the "
                                        "(token, head) pairs attended" if traffic is not None else None)},
        "step_hbm_gbs": step_bytes / (m_step["ms"] * 1e-3) / 1e9,
    }
    if cpu_baseline and rank == 0 and world == 1 and not h.args.no_cpu_baseline:
        tps, ms_cpu, threads, Bs = cpu_port_run(w, lens_all, steps=6, warmup=1)
        rec["cpu_baseline"] = {"value": tps, "unit": "tokens/s", "cores": threads, "kind": "port",
                               "sample": f"append + decode of all {Bs} sequences of the batch, 6 steps, "
                                         f"{ms_cpu:.1f} ms/step"}
    del cache, layer, fused
    h.release()
    return rec


# ------------------------------------------------------------------------------------------
# multi-GPU parity: the communicating configurations against the CPU oracle, outside every timed region
# ------------------------------------------------------------------------------------------

def run_parity_multi(h: Harness):
    """A small head-split decode (NCCL gather and fused peer-store gather) and a sequence-split decode on the real
    GPUs of this launch; every rank holds the same seeded problem, rank 0 checks the gathered results against
    the CPU oracle.  Returns the record (rank 0's view; `ok` is reduced over the ranks)."""
    torch, gpu, ctx, dist = h.torch, h.gpu, h.ctx, h.dist
    from llm_experiments_b200 import sharding

    rank, world, device = h.rank, h.world, h.device
    B, D, T_max, dtype = 3, 128, 904, torch.bfloat16
    H = 8 if 8 % world == 0 else world
    Hl = H // world
    lens = [900, 17, 512]
    g = torch.Generator().manual_seed(7)  # drawn on the CPU so that every rank holds the same values
    k_log = torch.randn((B, T_max, H, D), generator=g).to(dtype)
    v_log = torch.randn((B, T_max, H, D), generator=g).to(dtype)
    qs = [torch.randn((B, H * D), generator=g).to(dtype) for _ in range(3)]
    h0, h1 = sharding.head_range(H, rank, world)
    cache = gpu.kv_cache_create(ctx, gpu.KVCacheConfig(batch_size=B, max_seq_len=T_max, n_layers=1, n_heads=Hl,
                                                       head_dim=D, dtype=dtype, layout="bhtd", ragged=True))
    to_bhtd = lambda x: x.permute(0, 2, 1, 3).contiguous().to(device)  # noqa: E731  [B, T, h, D] -> [B, h, T, D]
    cache.layers[0].k_cache.buffer.view(B, Hl, T_max, D).copy_(to_bhtd(k_log[:, :, h0:h1]))
    cache.layers[0].v_cache.buffer.view(B, Hl, T_max, D).copy_(to_bhtd(v_log[:, :, h0:h1]))
    gpu.kv_cache_set_lengths(cache, lens)
    fused = sharding.FusedHeadGather(device, B, H, D, dtype)
    results = {"nccl": [], "fused": []}
    for q in qs[:2]:
        q_local = sharding.slice_heads(q.to(device), H, D, rank, world)
        out_local = torch.empty_like(q_local)
        gpu.batch_begin(ctx)
        gpu.attention_with_kv_cache(ctx, cache, 0, h.wrap(q_local), h.wrap(out_local))
        gpu.batch_commit(ctx)
        results["nccl"].append(sharding.gather_heads(out_local).clone())
        gpu.batch_begin(ctx)
        via_fused = fused.decode(ctx, cache, 0, h.wrap(q_local))
        gpu.batch_commit(ctx)
        torch.cuda.synchronize()
        results["fused"].append(via_fused.clone())
        h.barrier()  # nobody starts the next step's peer stores before every rank has copied this result
    # sequence split: rank r caches tokens [r*per, (r+1)*per) of every sequence, all heads
    per = T_max // world
    lo = rank * per
    local_lens = [max(0, min(n, lo + per) - lo) for n in lens]
    seq_cache = gpu.kv_cache_create(ctx, gpu.KVCacheConfig(batch_size=B, max_seq_len=per, n_layers=1, n_heads=H,
                                                           head_dim=D, dtype=dtype, layout="bhtd", ragged=True))
    seq_cache.layers[0].k_cache.buffer.view(B, H, per, D).copy_(to_bhtd(k_log[:, lo:lo + per]))
    seq_cache.layers[0].v_cache.buffer.view(B, H, per, D).copy_(to_bhtd(v_log[:, lo:lo + per]))
    gpu.kv_cache_set_lengths(seq_cache, local_lens)
    seq_cache.current_len = max(1, seq_cache.current_len)
    gpu.batch_begin(ctx)
    via_seq = sharding.sequence_split_decode(ctx, seq_cache, 0, h.wrap(qs[2].to(device)))
    gpu.batch_commit(ctx)
    torch.cuda.synchronize()
    status = int(ctx.dev_status.item()) if ctx.dev_status is not None else 0

    rec = {"world": world, "case": f"B={B} H={H} D={D} bf16, lengths {lens}, {Hl} head(s) per rank; sequence split "
                                   f"in slices of {per} tokens", "tolerance_abs": 2e-2, "dev_status": status}
    ok = status == 0
    fused_equal = all(torch.equal(a.view(torch.uint8), b.view(torch.uint8))
                      for a, b in zip(results["nccl"], results["fused"]))
    ok = ok and fused_equal
    if rank == 0:
        # the CPU oracle as the checker (never timed here): logical [B, T, H, D] arrays, reference strides
        from oracle import c_oracle

        bits = lambda t: t.contiguous().cpu().view(torch.int16).numpy().view(np.uint16)  # noqa: E731
        lens_np = np.asarray(lens, dtype=np.int32)
        want = [c_oracle.decode(bits(q), bits(k_log), bits(v_log), lens_np, B, H, D, (T_max * H * D, H * D, D))
                for q in qs]
        err = lambda got, ref: float(np.max(np.abs(got.float().cpu().numpy() - ref)))  # noqa: E731
        rec["max_abs_err"] = {"headsplit_nccl": max(err(a, r) for a, r in zip(results["nccl"], want[:2])),
                              "headsplit_fused": max(err(a, r) for a, r in zip(results["fused"], want[:2])),
                              "sequence_split": err(via_seq, want[2])}
        ok = ok and all(v <= 2e-2 for v in rec["max_abs_err"].values())
    flag = torch.tensor([1 if ok else 0], device=device, dtype=torch.int32)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    rec["fused_bit_equal_nccl"] = bool(fused_equal)
    rec["ok"] = bool(int(flag.item()))
    del cache, seq_cache, fused
    h.release()
    return rec


# ------------------------------------------------------------------------------------------
# CPU arm: the oracle port on the same sequences
# ------------------------------------------------------------------------------------------

def cpu_port_run(w, lens, steps, warmup, sample_seqs=None, log=None):
    """Times append + decode of the CPU oracle (C, OpenMP, all host threads) on the first `sample_seqs`
    sequences of the workload (all of them by default).  Returns (tokens_per_s, ms_per_step, threads, sequences)."""
    from oracle import c_oracle, kv_oracle

    Bs = w["B"] if sample_seqs is None else min(sample_seqs, w["B"])
    H, D = w["H"], w["D"]
    sl = np.asarray(lens[:Bs], dtype=np.int32)
    T_max = int(sl.max()) + max(SLACK, steps + warmup + 8)
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


def run_reference(args, w, rank, world):
    if rank != 0:
        return
    if w["kind"] != "decode" or w.get("head_split") or w.get("strong"):
        w = WORKLOADS["decode"]  # the CPU arm times the decode step, the headline workload
    lens = make_lengths(w)
    steps = max(1, min(args.steps, 500))  # about 0.1 s per step: the whole run stays within minutes
    warm = max(0, args.warmup)
    tps, ms, threads, Bs = cpu_port_run(w, lens, steps, warm)
    sample = f"append + decode of all {Bs} sequences of the batch per step, {steps} steps"
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
        "config": headline_config(w, max(1, world)),
        "cpu_baseline": {"value": tps, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": tps, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "CPU port of the reference math (oracle/kv_oracle.c), ONE process on rank 0 working on one batch of "
                f"{Bs} sequences whatever N is; the reference's own WGSL path needs wgpu/Vulkan: unavailable on this box",
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------
# prefill
# ------------------------------------------------------------------------------------------

def run_prefill(h: Harness, w):
    """Causal prefill fused with the cache write; value = prompt tokens/s, roofline = tensor."""
    torch, gpu, ctx = h.torch, h.gpu, h.ctx
    rank, world, device = h.rank, h.world, h.device
    B, H, D, N = w["B"], w["H"], w["D"], w["N"]
    E = H * D
    f32 = bool(w.get("f32"))
    dtype = torch.float32 if f32 else torch.bfloat16
    es = 4 if f32 else 2
    gen = torch.Generator(device=device).manual_seed(2000 + rank)
    mk = lambda: torch.randn((B * N, E), generator=gen, device=device, dtype=torch.float32).to(dtype)  # noqa: E731
    Q, K, V = mk(), mk(), mk()
    O = torch.empty_like(Q)
    cache = gpu.kv_cache_create(ctx, gpu.KVCacheConfig(batch_size=B, max_seq_len=N, n_layers=1, n_heads=H, head_dim=D,
                                                       dtype=dtype, layout="bhtd"))
    Qb, Kb, Vb, Ob = h.wrap(Q), h.wrap(K), h.wrap(V), h.wrap(O)
    ctx.config.flash_attn_max_head_dim = max(D, ctx.config.flash_attn_max_head_dim)

    def step_device():
        gpu.batch_begin(ctx)
        gpu.flash_attention(ctx, Qb, Kb, Vb, Ob, None, None, B, N, H, D, cache=cache, layer_idx=0)
        gpu.batch_commit(ctx)

    steps = min(h.steps, 50)
    sampler = h.sampler()
    m_step = h.measure(step_device, steps=steps)
    Qh, Kh, Vh = Q.cpu().pin_memory(), K.cpu().pin_memory(), V.cpu().pin_memory()
    Oh = torch.empty_like(Qh).pin_memory()

    def step_e2e():
        gpu.gpu_buffer_2d_write(ctx, Qh, Qb)
        gpu.gpu_buffer_2d_write(ctx, Kh, Kb)
        gpu.gpu_buffer_2d_write(ctx, Vh, Vb)
        step_device()
        gpu.gpu_buffer_2d_read(ctx, Ob, Oh)

    m_e2e = h.measure(step_e2e, steps=max(2, min(steps, 5)), warmup=1, repeats=min(h.repeats, 3))
    clocks = sampler.finish()
    status = int(ctx.dev_status.item()) if ctx.dev_status is not None else 0
    flops = 4.0 * B * H * D * N * (N + 1) / 2
    _, sustained, burst, kind = measured_peaks()
    achieved = flops / (m_step["ms"] * 1e-3) / 1e12
    traffic = B * PREFILL_DRAM_BYTES_PER_SEQUENCE if ((H, D, N) == (32, 128, 4096) and not h.tuned and not f32) else None
    rec = {
        "metric": "prefill tokens/s", "value": world * B * N / (m_step["ms"] * 1e-3), "unit": "tokens/s",
        **spread(m_step), "steps": steps, "scaling": "weak",
        "dtype": ("fp32 storage, operands as two bf16 halves (three MMAs per product), fp32 accumulate" if f32
                  else "bf16 operands, fp32 accumulate"),
        "config": {"workload": w["desc"], "batch_per_gpu": B, "global_batch": world * B,
                   "l2": f"Q/K/V/O/cache ({6 * B * N * E * es / 1e9:.1f} GB per step) larger than L2, no flush",
                   "parallelism": f"batch-sharded x{world}, no collective"},
        "e2e": {"value": world * B * N / (m_e2e["ms"] * 1e-3), "unit": "tokens/s", **spread(m_e2e),
                "h2d_bytes_per_step": 3 * B * N * E * es, "d2h_bytes_per_step": B * N * E * es},
        "gpu_launches": steps * h.repeats * (5 if f32 else 1), "gpu_launches_per_step": 5 if f32 else 1, "clocks": clocks,
        "dev_status": status,
        "roofline": {"bound": "tensor",
                     "kernel": ("prefill_tc_f32_kernel (+ 3 split_kernel, append_rows_kernel); flops counted once per "
                                "fp32 product, the kernel issues three bf16 MMAs for each" if f32 else "prefill_tc_kernel"),
                     "achieved": achieved, "peak": sustained,
                     "unit": "TFLOP/s", "frac": achieved / sustained, "frac_of_burst": achieved / burst,
                     "peak_kind": kind + " (sustained cuBLAS bf16; kernel timed in a loop)",
                     "algorithmic_flops_per_launch": flops, "traffic": traffic,
                     "traffic_source": ("ncu capture of the 2-sequence case of the default kernel, scaled by the "
                                        "sequences" if traffic is not None else None)},
    }
    if rank == 0 and world == 1 and not h.args.no_cpu_baseline:
        from oracle import c_oracle

        hs = 4  # heads of one sequence timed on the CPU
        if f32:
            sl = lambda X: np.ascontiguousarray(X.reshape(B, N, H, D)[0, :, :hs, :].reshape(N, hs * D).cpu().numpy())  # noqa: E731
        else:
            sl = lambda X: np.ascontiguousarray(  # noqa: E731
                X.reshape(B, N, H, D)[0, :, :hs, :].reshape(N, hs * D).cpu().view(torch.int16).numpy().view(np.uint16))
        t0 = time.perf_counter()
        c_oracle.prefill(sl(Q), sl(K), sl(V), 1, N, hs, D, want_stats=False)
        dt = time.perf_counter() - t0
        rec["cpu_baseline"] = {"value": N * hs / H / dt, "unit": "tokens/s", "cores": c_oracle.num_threads(),
                               "kind": "port",
                               "sample": f"{hs} of {H} heads of one sequence ({dt:.2f} s); value counts {hs}/{H} of a "
                                         "token per row"}
    del cache, Q, K, V, O, Qh, Kh, Vh, Oh
    h.release()
    return rec


# ------------------------------------------------------------------------------------------
# the callers either side of the attention call
# ------------------------------------------------------------------------------------------

def layer_weights(h: Harness, gen, E, decode_layer):
    torch = h.torch
    rnd = lambda shape, scale=1.0: (torch.randn(shape, generator=gen, device=h.device) * scale).to(torch.bfloat16)  # noqa: E731
    raw = dict(ln1_gamma=rnd((E,), 0.1) + 1, ln1_beta=rnd((E,), 0.1), wq=rnd((E, E), E ** -0.5), wk=rnd((E, E), E ** -0.5),
               wv=rnd((E, E), E ** -0.5), wo=rnd((E, E), E ** -0.5), ln2_gamma=rnd((E,), 0.1) + 1, ln2_beta=rnd((E,), 0.1),
               w1=rnd((E, 4 * E), E ** -0.5), b1=rnd((4 * E,), 0.1), w2=rnd((4 * E, E), (4 * E) ** -0.5), b2=rnd((E,), 0.1))
    return decode_layer.DecoderLayerWeights(**{k: (h.wrap1(v) if v.dim() == 1 else h.wrap(v)) for k, v in raw.items()})


def run_qkv_append(h: Harness, w):
    """One decode step's Q/K/V projection fused with the cache append; value = tokens/s, roofline = HBM
    (the step streams 3*E*E weights).  The layers' weights (4 x 100 MB) are used in turn, so that a step's
    weights are not in L2 from the step before."""
    torch, gpu, ctx = h.torch, h.gpu, h.ctx
    rank, world, device = h.rank, h.world, h.device
    B, H, D, T, n_layers = w["B"], w["H"], w["D"], w["T"], w["layers"]
    E = H * D
    dtype = torch.bfloat16
    gen = torch.Generator(device=device).manual_seed(3000 + rank)
    rnd = lambda shape, scale: (torch.randn(shape, generator=gen, device=device) * scale).to(dtype)  # noqa: E731
    weights = [[h.wrap(rnd((E, E), E ** -0.5)) for _ in range(3)] for _ in range(n_layers)]
    x, q = rnd((B, E), 1.0), torch.empty((B, E), dtype=dtype, device=device)
    xb, qb = h.wrap(x), h.wrap(q)
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

    sampler = h.sampler()
    m_step = h.measure(step_device)
    xh, qh = x.cpu().pin_memory(), torch.empty_like(q, device="cpu").pin_memory()

    def step_e2e():
        gpu.gpu_buffer_2d_write(ctx, xh, xb)
        step_device()
        gpu.gpu_buffer_2d_read(ctx, qb, qh)

    m_e2e = h.measure(step_e2e, warmup=1)
    clocks = sampler.finish()
    es = 2
    bytes_step = 3 * E * E * es + B * E * es + 3 * B * E * es
    peak, _, _, kind = measured_peaks()
    achieved = bytes_step / (m_step["ms"] * 1e-3) / 1e9
    rec = {
        "metric": "projected tokens/s (one layer's Q/K/V projection + cache append per step)",
        "value": world * B / (m_step["ms"] * 1e-3), "unit": "tokens/s", **spread(m_step), "scaling": "weak",
        "dtype": "bf16 operands, fp32 accumulate",
        "config": {"workload": w["desc"], "batch_per_gpu": B, "global_batch": world * B,
                   "l2": f"{n_layers} layers' weights ({n_layers * 3 * E * E * es / 1e6:.0f} MB) used in turn, larger than L2",
                   "parallelism": f"batch-sharded x{world}, no collective"},
        "e2e": {"value": world * B / (m_e2e["ms"] * 1e-3), "unit": "tokens/s", **spread(m_e2e),
                "h2d_bytes_per_step": B * E * es, "d2h_bytes_per_step": B * E * es},
        "gpu_launches": h.steps * h.repeats, "gpu_launches_per_step": 1, "clocks": clocks,
        "roofline": {"bound": "hbm", "kernel": "qkv_append_kernel", "achieved": achieved, "peak": peak, "unit": "GB/s",
                     "frac": achieved / peak, "peak_kind": kind, "algorithmic_bytes_per_launch": bytes_step,
                     "traffic": None},
    }
    if rank == 0 and world == 1 and not h.args.no_cpu_baseline:
        from oracle import kv_oracle

        f32 = lambda t: t.float().cpu().numpy()  # noqa: E731
        xs, ws = f32(x), [f32(t.buffer) for t in weights[0]]
        reps = 3
        t0 = time.perf_counter()
        for _ in range(reps):
            kv_oracle.qkv_project(xs, *ws)
        dt = (time.perf_counter() - t0) / reps
        rec["cpu_baseline"] = {"value": B / dt, "unit": "tokens/s", "cores": os.cpu_count(), "kind": "port",
                               "sample": f"the three projections of one step in float64 numpy ({dt:.2f} s per step)"}
    return rec


def run_decode_layer(h: Harness, w):
    """One whole decoder layer per step: layernorm, Q/K/V projection + append, cached attention, output
    projection + residual, layernorm, MLP.  value = tokens/s through one layer; roofline = HBM over the bytes
    the step must move (K/V rows attended + 12 E^2 weights + the small row buffers)."""
    torch, gpu, ctx = h.torch, h.gpu, h.ctx
    from llm_experiments_b200 import decode_layer

    rank, world, device = h.rank, h.world, h.device
    B, H, D, n_layers = w["B"], w["H"], w["D"], w["layers"]
    E, T_max = H * D, w["hi"] + 8
    dtype = torch.bfloat16
    gen = torch.Generator(device=device).manual_seed(4000 + rank)
    weights = [layer_weights(h, gen, E, decode_layer) for _ in range(n_layers)]
    lens = make_lengths(w)
    caches = []
    for _ in range(n_layers):
        c = gpu.kv_cache_create(ctx, gpu.KVCacheConfig(batch_size=B, max_seq_len=T_max, n_layers=1, n_heads=H, head_dim=D,
                                                       dtype=dtype, layout="bhtd", ragged=True))
        c.layers[0].k_cache.buffer.normal_(generator=gen)
        c.layers[0].v_cache.buffer.normal_(generator=gen)
        gpu.kv_cache_set_lengths(c, lens)
        caches.append(c)
    lens_dev, max_len = torch.from_numpy(lens.astype(np.int32)).to(device), int(lens.max())
    x = torch.randn((B, E), generator=gen, device=device).to(dtype)
    y = torch.empty((B, E), dtype=dtype, device=device)
    xb, yb = h.wrap(x), h.wrap(y)
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

    sampler = h.sampler()
    m_step = h.measure(step_device)
    xh, yh = x.cpu().pin_memory(), torch.empty_like(y, device="cpu").pin_memory()

    def step_e2e():
        gpu.gpu_buffer_2d_write(ctx, xh, xb)
        step_device()
        gpu.gpu_buffer_2d_read(ctx, yb, yh)

    m_e2e = h.measure(step_e2e, warmup=1)
    clocks = sampler.finish()
    es = 2
    kv_bytes = int((lens.astype(np.int64) + 1).sum()) * H * D * es * 2
    weight_bytes = 12 * E * E * es
    row_bytes = B * E * es * 14 + B * 4 * E * es * 2  # the [B, E] and [B, 4E] row buffers read / written between kernels
    bytes_step = kv_bytes + weight_bytes + row_bytes
    peak, _, _, kind = measured_peaks()
    achieved = bytes_step / (m_step["ms"] * 1e-3) / 1e9
    return {
        "metric": "tokens/s through one decoder layer (cached decode step)", "value": world * B / (m_step["ms"] * 1e-3),
        "unit": "tokens/s", **spread(m_step), "scaling": "weak", "dtype": "bf16 storage, fp32 arithmetic",
        "config": {"workload": w["desc"], "batch_per_gpu": B, "global_batch": world * B,
                   "l2": f"{n_layers} layers' caches and weights used in turn, far larger than L2",
                   "parallelism": f"batch-sharded x{world}, no collective"},
        "e2e": {"value": world * B / (m_e2e["ms"] * 1e-3), "unit": "tokens/s", **spread(m_e2e),
                "h2d_bytes_per_step": B * E * es, "d2h_bytes_per_step": B * E * es},
        "gpu_launches": h.steps * h.repeats * 8, "gpu_launches_per_step": 8, "clocks": clocks,
        "roofline": {"bound": "hbm", "kernel": "the layer's 8 kernels together", "achieved": achieved, "peak": peak,
                     "unit": "GB/s", "frac": achieved / peak, "peak_kind": kind,
                     "algorithmic_bytes_per_launch": bytes_step, "kv_bytes": kv_bytes, "weight_bytes": weight_bytes,
                     "traffic": None},
    }


def run_prompt_layer(h: Harness, w):
    """One whole decoder layer over a prompt per step: layernorm, three projection GEMMs, causal attention
    fused with the cache write, output projection + residual, layernorm, MLP.  value = prompt tokens/s
    through one layer; roofline = tensor, over the layer's matmul and attention flops."""
    torch, gpu, ctx = h.torch, h.gpu, h.ctx
    from llm_experiments_b200 import decode_layer

    rank, world, device = h.rank, h.world, h.device
    ctx.config.flash_attn_max_head_dim = 128
    B, H, D, N, n_layers = w["B"], w["H"], w["D"], w["N"], w["layers"]
    E, rows = H * D, B * N
    dtype = torch.bfloat16
    gen = torch.Generator(device=device).manual_seed(5000 + rank)
    weights = [layer_weights(h, gen, E, decode_layer) for _ in range(n_layers)]
    caches = [gpu.kv_cache_create(ctx, gpu.KVCacheConfig(batch_size=B, max_seq_len=N, n_layers=1, n_heads=H, head_dim=D,
                                                         dtype=dtype, layout="bhtd")) for _ in range(n_layers)]
    x = torch.randn((rows, E), generator=gen, device=device).to(dtype)
    y = torch.empty((rows, E), dtype=dtype, device=device)
    xb, yb = h.wrap(x), h.wrap(y)
    scratch = decode_layer.prompt_layer_scratch(ctx, rows, E)
    state = {"i": 0}

    def step_device():
        li = state["i"] % n_layers
        state["i"] += 1
        gpu.batch_begin(ctx)
        decode_layer.prompt_layer_step(ctx, caches[li], xb, weights[li], scratch, yb, B, N)
        gpu.batch_commit(ctx)

    steps = min(h.steps, 50)
    sampler = h.sampler()
    m_step = h.measure(step_device, steps=steps)
    xh, yh = x.cpu().pin_memory(), torch.empty_like(y, device="cpu").pin_memory()

    def step_e2e():
        gpu.gpu_buffer_2d_write(ctx, xh, xb)
        step_device()
        gpu.gpu_buffer_2d_read(ctx, yb, yh)

    m_e2e = h.measure(step_e2e, steps=max(2, min(steps, 5)), warmup=1, repeats=min(h.repeats, 3))
    clocks = sampler.finish()
    es = 2
    gemm_flops = 2.0 * rows * E * E * 12  # Q, K, V, Wo (4 E^2) + the MLP (8 E^2)
    attn_flops = 4.0 * B * H * D * N * (N + 1) / 2
    flops = gemm_flops + attn_flops
    _, sustained, burst, kind = measured_peaks()
    achieved = flops / (m_step["ms"] * 1e-3) / 1e12
    return {
        "metric": "prompt tokens/s through one decoder layer", "value": world * rows / (m_step["ms"] * 1e-3),
        "unit": "tokens/s", **spread(m_step), "steps": steps, "scaling": "weak",
        "dtype": "bf16 operands, fp32 accumulate",
        "config": {"workload": w["desc"], "batch_per_gpu": B, "global_batch": world * B, "seq_len": N,
                   "l2": f"{n_layers} layers' weights used in turn; activations ({rows * E * es / 1e6:.0f} MB per buffer) "
                         "larger than L2",
                   "parallelism": f"batch-sharded x{world}, no collective"},
        "e2e": {"value": world * rows / (m_e2e["ms"] * 1e-3), "unit": "tokens/s", **spread(m_e2e),
                "h2d_bytes_per_step": rows * E * es, "d2h_bytes_per_step": rows * E * es},
        "gpu_launches": steps * h.repeats * 9, "gpu_launches_per_step": 9, "clocks": clocks,
        "roofline": {"bound": "tensor", "kernel": "the layer's 9 kernels together (6 GEMM launches, the prefill kernel, "
                                                  "2 layernorm)",
                     "achieved": achieved, "peak": sustained, "unit": "TFLOP/s", "frac": achieved / sustained,
                     "frac_of_burst": achieved / burst,
                     "peak_kind": f"{kind} (sustained cuBLAS bf16; the layer is timed in a long loop)",
                     "algorithmic_flops_per_launch": flops, "gemm_flops": gemm_flops, "attention_flops": attn_flops,
                     "traffic": None},
    }


def run_model_step(h: Harness, w):
    """One cached decode step of a whole bf16 decoder on the library's kernels: embedding gather, L decoder
    layers, final layernorm, logits projection, argmax.  value = generated tokens/s; roofline = HBM over the
    K/V rows attended plus every weight once."""
    torch, gpu, ctx = h.torch, h.gpu, h.ctx
    from llm_experiments_b200 import model

    rank, world, device = h.rank, h.world, h.device
    B, H, D, L, vocab = w["B"], w["H"], w["D"], w["layers"], w["vocab"]
    E, T_max = H * D, w["hi"] + 8
    cfg = model.DecoderConfig(vocab_size=vocab, context_size=T_max, embedding_dim=E, n_heads=H, n_layers=L)
    weights = model.random_weights(ctx, cfg, seed=6000 + rank)
    state = model.decoder_state_create(ctx, cfg, weights, batch_size=B, max_seq_len=T_max, ragged=True)
    lens = make_lengths(w)
    gen = torch.Generator(device=device).manual_seed(6100 + rank)
    for c in state.caches:
        c.layers[0].k_cache.buffer.normal_(generator=gen)
        c.layers[0].v_cache.buffer.normal_(generator=gen)
    lens_dev, max_len = torch.from_numpy(lens.astype(np.int32)).to(device), int(lens.max())
    tokens = torch.randint(0, vocab, (B,), generator=gen, device=device, dtype=torch.int32)
    tok_b = h.wrap1(tokens)
    next_b = h.wrap1(torch.empty(B, dtype=torch.int32, device=device))

    def step_device():
        for c in state.caches:
            c.seq_lens.copy_(lens_dev)  # every step starts from the same lengths
            c.current_len = max_len
        gpu.batch_begin(ctx)
        model.decode_step(ctx, state, tok_b, next_b)
        gpu.batch_commit(ctx)

    sampler = h.sampler()
    m_step = h.measure(step_device)
    tok_h = tokens.cpu().pin_memory()
    next_h = torch.empty(B, dtype=torch.int32).pin_memory()

    def step_e2e():
        gpu.gpu_buffer_1d_write(ctx, tok_h, tok_b)
        step_device()
        gpu.gpu_buffer_1d_read(ctx, next_b, next_h)

    m_e2e = h.measure(step_e2e, warmup=1)

    # the same step as one replayed CUDA graph (what a launch-bound step gains from it)
    for c in state.caches:
        gpu.kv_cache_set_lengths(c, lens)
    graphed = model.GraphedDecodeStep(ctx, state)
    graphed.token_ids.buffer.copy_(tokens)
    graphed.capture()

    def step_graph():
        for c in state.caches:
            c.seq_lens.copy_(lens_dev)
            c.current_len = max_len
        graphed.step()

    m_graph = h.measure(step_graph)
    clocks = sampler.finish()
    status = int(ctx.dev_status.item()) if ctx.dev_status is not None else 0
    es = 2
    kv_bytes = L * int((lens.astype(np.int64) + 1).sum()) * H * D * es * 2
    weight_bytes = L * 12 * E * E * es + E * vocab * es
    bytes_step = kv_bytes + weight_bytes
    peak, _, _, kind = measured_peaks()
    achieved = bytes_step / (m_step["ms"] * 1e-3) / 1e9
    launches = model.launches_per_decode_step(cfg)
    return {
        "metric": "generated tokens/s (whole cached decode step of the model)", "value": world * B / (m_step["ms"] * 1e-3),
        "unit": "tokens/s", **spread(m_step), "scaling": "weak", "dtype": "bf16 storage, fp32 arithmetic",
        "config": {"workload": w["desc"], "batch_per_gpu": B, "global_batch": world * B,
                   "l2": "caches (38 GB) and weights (1.9 GB) far larger than L2, no flush",
                   "parallelism": f"batch-sharded x{world}, no collective"},
        "e2e": {"value": world * B / (m_e2e["ms"] * 1e-3), "unit": "tokens/s", **spread(m_e2e),
                "h2d_bytes_per_step": B * 4, "d2h_bytes_per_step": B * 4},
        "gpu_launches": h.steps * h.repeats * launches, "gpu_launches_per_step": launches, "clocks": clocks,
        "dev_status": status,
        "cuda_graph": {"value": world * B / (m_graph["ms"] * 1e-3), "unit": "tokens/s", **spread(m_graph),
                       "what": "the same step captured once and replayed (one graph launch per step)"},
        "roofline": {"bound": "hbm", "kernel": f"the step's {launches} kernels together", "achieved": achieved,
                     "peak": peak, "unit": "GB/s", "frac": achieved / peak, "peak_kind": kind,
                     "algorithmic_bytes_per_launch": bytes_step, "kv_bytes": kv_bytes, "weight_bytes": weight_bytes,
                     "traffic": None},
    }


RUNNERS = {"prefill": run_prefill, "qkv": run_qkv_append, "layer_step": run_decode_layer,
           "prompt_layer": run_prompt_layer, "model_step": run_model_step}


def run_one(h: Harness, name, **kw):
    w = dict(WORKLOADS[name])
    w.setdefault("block_size", 0)
    if w["kind"] == "decode":
        return run_decode(h, w, **kw)
    return RUNNERS[w["kind"]](h, w)


def sub_record(fn, *a, **kw):
    """A sub-workload must not take the headline down with it: its failure is recorded in its place."""
    try:
        return fn(*a, **kw)
    except Exception as e:  # noqa: BLE001
        return {"error": f"{type(e).__name__}: {e}"}


def run_b200(args):
    h = Harness(args)
    name = args.workload
    w = WORKLOADS[name]
    rank, world = h.rank, h.world
    extra = {}
    if name == "decode" and not args.only:
        # the communicating configurations are checked for parity before anything is timed
        if world > 1:
            extra["parity_multi"] = sub_record(run_parity_multi, h)
    if w["kind"] == "decode":
        head = run_one(h, name, cpu_baseline=True, gather="fused" if args.fused_gather else "nccl")
    else:
        head = run_one(h, name)
    if name == "decode" and not args.only:
        subs = {}
        for sub in ("paged", "prefill", "longctx"):
            subs[sub] = sub_record(run_one, h, sub)
        if world > 1:
            subs["decode_strong"] = {}
            for assign in ("contiguous", "balanced"):
                strong = sub_record(run_one, h, "decode_strong", assign=assign)
                if "ms_per_step" in strong:
                    strong["speedup_vs_one_gpu"] = head["ms_per_step"] / strong["ms_per_step"]
                    strong["efficiency"] = strong["speedup_vs_one_gpu"] / world
                subs["decode_strong"][assign] = strong
            hs = {}
            for how in ("nccl", "fused"):
                r = sub_record(run_one, h, "longctx_headsplit", gather=how)
                if "ms_per_step" in r and "ms_per_step" in subs["longctx"]:
                    r["speedup_vs_one_gpu"] = subs["longctx"]["ms_per_step"] / r["ms_per_step"]
                    r["efficiency"] = r["speedup_vs_one_gpu"] / world
                hs[how] = r
            subs["longctx_headsplit"] = hs
        extra["workloads"] = subs
    h.finish()
    if rank != 0:
        return
    line = {
        "metric": head["metric"], "value": head["value"], "unit": head["unit"], "n_gpus": world,
        "steps": head.get("steps", h.steps), "warmup": h.warmup, "ms_per_step": head["ms_per_step"],
        "ms_per_step_min": head["ms_per_step_min"], "ms_per_step_max": head["ms_per_step_max"],
        "repeats": head["repeats"], "higher_is_better": True, "scaling": head.get("scaling", "weak"),
        "vs_baseline": None, "dtype": head.get("dtype", "bf16 storage, fp32 arithmetic"), "data": "synthetic",
        "config": head["config"], "e2e": head["e2e"], "gpu_launches": head["gpu_launches"],
        "gpu_launches_per_step": head.get("gpu_launches_per_step"), "clocks": head["clocks"],
        "roofline": head["roofline"], "cpu_baseline": head.get("cpu_baseline"),
    }
    for k in ("step_hbm_gbs", "dev_status", "cuda_graph"):
        if k in head:
            line[k] = head[k]
    line.update(extra)
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--repeats", type=int, default=10, help="timed loops of --steps steps each; medians are reported")
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="decode", choices=sorted(WORKLOADS))
    ap.add_argument("--only", action="store_true", help="time the named workload alone, without the sub-records")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--fused-gather", action="store_true",
                    help="head-split workloads: gather the outputs with peer stores from the merge kernel instead of NCCL")
    ap.add_argument("--tune", action="append", default=[], metavar="NAME=VALUE",
                    help="set a kernel tuning knob of the library (b2kv_tune), e.g. prefill_variant=2")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        run_reference(args, WORKLOADS[args.workload], rank, world)
        return
    if args.tune:
        import __graft_entry__

        native = __graft_entry__.import_package()._native
        for item in args.tune:
            name, _, value = item.partition("=")
            native.tune(name, int(value))
    if world != args.gpus and args.gpus != 1 and world == 1:
        raise SystemExit("launch with torchrun for --gpus > 1")
    run_b200(args)


if __name__ == "__main__":
    main()
