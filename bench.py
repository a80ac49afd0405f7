#!/usr/bin/env python
"""Throughput benchmark of the NTC decode path.

    python bench.py --gpus N --steps K --warmup W            # this library
    python bench.py --impl reference --gpus N --steps K ...  # the unmodified reference decoder

A step is one full decode (every mip, one kernel launch) of the 4096x4096, 12-channel PBR texture
set of the benchmark definition: 12 latent features at grid scale 4, FP8 hidden layers with an int8
output layer, full 13-level mip chain, seeded synthetic latents and weights.  With N > 1 (launched
through torch.distributed.run, one rank per GPU) every rank decodes its own texture set of that
shape: the path has no exchange step, so the ranks share nothing (weak scaling).

The JSON line reports
  value     decoded Gtexel/s with the compressed set resident in HBM, timed with CUDA events around
            each launch (L2 is flushed between steps), max over ranks;
  e2e       the same metric through the texture-set level of the C ABI with HOST buffers: every step
            uploads the compressed set from pinned memory, decodes and reads every mip back to
            pinned host memory (wall clock);
  roofline  algorithmic bytes of one launch / its mean duration against the measured HBM copy peak;
  cpu_baseline  the scalar CPU restatement of the same arithmetic on this machine's cores.

The reference arm runs the reference's own CUDA decoder (LibNTC has no CPU decoder) through its
public API on the same GPU and reports the end-to-end figure as its value, so that the two arms'
`e2e` values compare like with like; its kernel-only figure is given beside it.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402

import __graft_entry__ as entry  # noqa: E402

METRIC = "decoded Gtexel/s (full mip chain)"
UNIT = "Gtexel/s"
L2_FLUSH_BYTES = 256 << 20
WORKLOAD = ("PBR texture set 4096x4096, 12 channels, 13 mips, latent shape {gridSizeScale 4, 12 features}, "
            "FP8 e4m3 hidden layers + int8 output layer")

# DRAM bytes per launch of the decode kernel on this workload (dram__bytes_read.sum +
# dram__bytes_write.sum from the ncu capture summarised in profiles/).
MEASURED_TRAFFIC_BYTES = 492.5e6  # profiles/decode_kernel_fp8_4096sq_launch_list.md


def measured_peak_gbs():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.process = None

    def start(self):
        try:
            self.process = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.gpu_index), "--query-gpu=" + self.QUERY, "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.process = None

    def stop(self):
        if self.process is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.process.terminate()
        try:
            out, _ = self.process.communicate(timeout=5)
        except Exception:
            self.process.kill()
            out = ""
        clocks, max_clocks, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.splitlines():
            fields = [f.strip() for f in line.split(",")]
            if len(fields) < 9:
                continue
            try:
                clocks.append(float(fields[1]))
                max_clocks.append(float(fields[2]))
            except ValueError:
                continue
            for name, value in zip(names, fields[5:9]):
                if value.lower().startswith("active"):
                    reasons.add(name)
        if not clocks:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        return {"sm_mhz": statistics.median(clocks), "sm_max_mhz": max(max_clocks), "reasons": sorted(reasons),
                "samples": len(clocks)}


def dist_setup(n_gpus: int):
    import torch

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world > 1:
        import torch.distributed as dist

        torch.cuda.set_device(local_rank)
        dist.init_process_group(backend="nccl", device_id=torch.device("cuda", local_rank))
        return rank, local_rank, world, dist
    return 0, 0, 1, None


def barrier_sync(dist, torch):
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()


def reduce_max(dist, torch, value: float, device) -> float:
    if dist is None:
        return value
    t = torch.tensor([value], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def reduce_sum(dist, torch, value: float, device) -> float:
    if dist is None:
        return value
    t = torch.tensor([value], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return float(t.item())


def cpu_baseline(synthetic_set) -> dict:
    """The CPU restatement (exact-accumulation numerics, the kernel's arithmetic contract) on all
    host cores, on a bounded sample: the top rows of mip 0."""
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import oracle_py

    oracle_py.build_oracle()
    checker = oracle_py.OracleSet.from_synthetic(synthetic_set)
    cores = os.cpu_count() or 1
    rows = 64
    start = time.perf_counter()
    checker.decode_mip(0, synthetic_set.use_int8, oracle_py.NUMERICS_SPEC, y0=0, y1=rows)
    probe = time.perf_counter() - start
    width = synthetic_set.geometry.color_mips[0].width
    # aim at roughly 15 s of CPU work
    rows = int(min(synthetic_set.geometry.color_mips[0].height, max(rows, rows * 15.0 / max(probe, 1e-3))))
    rows -= rows % 4
    start = time.perf_counter()
    checker.decode_mip(0, synthetic_set.use_int8, oracle_py.NUMERICS_SPEC, y0=0, y1=rows)
    elapsed = time.perf_counter() - start
    texels = rows * width
    return {"value": texels / elapsed / 1e9, "unit": UNIT, "cores": cores, "kind": "port",
            "sample": "rows 0..%d of mip 0 (%d texels, %.1f s)" % (rows - 1, texels, elapsed)}


def run_ours(args) -> dict:
    import torch

    entry.load_package()
    from rtxntc_library_b200 import binding, synthetic

    rank, local_rank, world, dist = dist_setup(args.gpus)
    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)

    spec = synthetic.config_spec(1)
    spec.seed = 1 + 1000 * rank  # every rank decodes its own texture set
    data = synthetic.make_texture_set(spec)
    geo = data.geometry
    texels = geo.total_texels
    use_int8 = data.use_int8

    # ---- device-resident throughput -------------------------------------------------------
    resident = binding.ResidentTextureSet.from_synthetic(data, device=str(device))
    params = resident.params(use_int8)
    flush = torch.empty(L2_FLUSH_BYTES, dtype=torch.uint8, device=device)
    for _ in range(args.warmup):
        resident.launch(params)
    torch.cuda.synchronize()
    resident.check_status()

    sampler = ClockSampler(local_rank)
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    stops = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    launches_before = binding.lib().ntcb_launch_count()
    barrier_sync(dist, torch)
    if rank == 0:
        sampler.start()
    wall_start = time.perf_counter()
    for step in range(args.steps):
        flush.fill_(step & 0xFF)  # evict L2 between steps (not inside the per-step events)
        starts[step].record()
        resident.launch(params)
        stops[step].record()
    barrier_sync(dist, torch)
    wall = time.perf_counter() - wall_start
    clocks = sampler.stop() if rank == 0 else None
    launches = binding.lib().ntcb_launch_count() - launches_before
    resident.check_status()
    step_ms = [s.elapsed_time(e) for s, e in zip(starts, stops)]
    device_seconds = reduce_max(dist, torch, sum(step_ms) / 1e3, device)
    total_launches = int(reduce_sum(dist, torch, float(launches), device))
    value = world * texels * args.steps / device_seconds / 1e9

    # ---- end to end through the texture-set API with host buffers ---------------------------
    del resident, flush
    torch.cuda.empty_cache()
    context = binding.Context(local_rank)
    texture_set = context.create_texture_set(data.container)
    host_out = torch.empty(texels * geo.channels, dtype=torch.float16).pin_memory()
    base = host_out.data_ptr()

    def e2e_step():
        texture_set.decompress(use_int8)
        for mip, cm in enumerate(geo.color_mips):
            texture_set.read_channels_into(mip, base + cm.texel_offset * geo.channels * 2)

    for _ in range(max(1, min(args.warmup, 3))):
        e2e_step()
    barrier_sync(dist, torch)
    e2e_start = time.perf_counter()
    for _ in range(args.steps):
        e2e_step()
    texture_set.synchronize()
    e2e_seconds = reduce_max(dist, torch, time.perf_counter() - e2e_start, device)
    barrier_sync(dist, torch)
    e2e_value = world * texels * args.steps / e2e_seconds / 1e9
    h2d = geo.encoded_latent_bytes + 2 * binding.STAGED_NETWORK_BYTES
    d2h = texels * geo.channels * 2
    texture_set.close()
    context.close()

    # ---- roofline of the decode kernel -----------------------------------------------------
    peak, peak_kind = measured_peak_gbs()
    algorithmic_bytes = texels * geo.channels * 2 + geo.encoded_latent_bytes + binding.STAGED_NETWORK_BYTES
    launch_seconds = statistics.mean(step_ms) / 1e3
    achieved = algorithmic_bytes / launch_seconds / 1e9
    roofline = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                "traffic": MEASURED_TRAFFIC_BYTES, "peak_source": "%s copy bandwidth" % peak_kind,
                "algorithmic_bytes_per_launch": algorithmic_bytes}

    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": device_seconds * 1e3 / args.steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "fp8_e4m3 x fp8_e4m3 -> f32 (layers 0-2), s8 x s8 -> s32 (layer 3), f16 activations",
        "data": "synthetic (seeded latents and weights of the configuration's shape)",
        "config": {"workload": WORKLOAD, "texels_per_step_per_gpu": texels, "texture_sets": world,
                   "parallelism": "one texture set per GPU, no collective", "launches_per_step": 1,
                   "l2": "256 MiB written between steps, outside the per-step events; the 537 MB output also exceeds L2"},
        "clocks": clocks, "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": total_launches, "roofline": roofline, "wall_seconds_timed_region": wall,
    }
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline(data)
    if dist is not None:
        dist.destroy_process_group()
    return line if rank == 0 else None


def run_reference(args) -> dict:
    """The unmodified reference library (oracle/_ref) through its own public API."""
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if rank != 0:
        return None
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import oracle_py

    if not oracle_py.reference_available():
        return {"impl": "reference", "unavailable": "oracle/_ref/libntc_ref.so is not built (oracle/build_ref.sh needs the reference sources)"}
    import torch

    entry.load_package()
    from rtxntc_library_b200 import synthetic

    data = synthetic.make_texture_set(synthetic.config_spec(1))
    geo = data.geometry
    texels = geo.total_texels
    decoder = oracle_py.ReferenceDecoder(data.container, geo.channels, device=0)
    host_out = torch.empty(texels * geo.channels, dtype=torch.float16).pin_memory()
    base = host_out.data_ptr()

    kernel_ms = []

    def step():
        kernel_ms.append(decoder.decompress(data.use_int8))
        for mip, cm in enumerate(geo.color_mips):
            decoder.read_mip_into(mip, cm.width, cm.height, base + cm.texel_offset * geo.channels * 2, False)

    for _ in range(args.warmup):
        step()
    kernel_ms.clear()
    sampler = ClockSampler(0)
    torch.cuda.synchronize()
    sampler.start()
    start = time.perf_counter()
    for _ in range(args.steps):
        step()
    torch.cuda.synchronize()
    seconds = time.perf_counter() - start
    clocks = sampler.stop()
    decoder.close()
    value = texels * args.steps / seconds / 1e9
    kernel_value = texels / (statistics.mean(kernel_ms) / 1e3) / 1e9
    return {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": seconds * 1e3 / args.steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f16 x f16 -> f16 (wmma), as the reference's CUDA decoder computes",
        "data": "synthetic (seeded latents and weights of the configuration's shape)",
        "config": {"workload": WORKLOAD, "texels_per_step_per_gpu": texels,
                   "path": "CreateCompressedTextureSetFromMemory once; per step Decompress + ReadChannels(FLOAT16, Host) of every mip",
                   "note": "the reference has no CPU decoder and no multi-GPU path: one rank runs its CUDA decoder on GPU 0"
                           + ("; the other %d ranks idle" % (world - 1) if world > 1 else "")},
        "clocks": clocks,
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "kernel_only": {"value": kernel_value, "unit": UNIT, "ms": statistics.mean(kernel_ms),
                        "source": "DecompressionStats::gpuTimeMilliseconds (mip loop only; upload, unpack and weight conversion excluded)"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": 0, "kind": "reference",
                         "sample": "whole workload; the reference's only decoder is its CUDA kernel, run on the GPU of this box"},
    }


def main() -> int:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=20)
    parser.add_argument("--warmup", type=int, default=3)
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--no-cpu-baseline", action="store_true")
    args = parser.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else max(args.warmup, 1)
    line = run_reference(args) if args.impl == "reference" else run_ours(args)
    if line is not None:
        print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
