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

  e2e_unorm8  the end-to-end job with UNORM8 pixels as the client's format: the decode kernel's
            converting epilogue writes them, so the read-back is half as large (informational; the
            reference arm reports Decompress + ReadChannels(UNORM8) beside it).

`--config 0|2|3|4` time the other benchmark configurations on their own (1024^2 single mip; 64 sets
of 2048^2 sharded by set; 8192^2 sharded by tile rows; 16.7 M inference-on-sample queries split
over the ranks - the last three split a fixed job over the ranks, strong scaling); they report the
device-resident figure only.  The default run carries them as `other_configs` sub-records.

The reference arm runs the reference's own CUDA decoder (LibNTC has no CPU decoder) through its
public API on the same GPU.  Like this library's arm, its `value` is the device figure (the
reference's own DecompressionStats::gpuTimeMilliseconds, which brackets its mip loop) and its `e2e`
the wall clock of Decompress + ReadChannels(FLOAT16, Host) of every mip, with the bytes it copies.
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

# DRAM bytes per launch of the decode kernel on the benchmark workload come from the ncu capture
# summarised in this file (its line "traffic_bytes_per_launch: N").
TRAFFIC_CAPTURE = "profiles/decode_kernel_fp8_4096sq_launch_list.md"
# Thread instructions per texel of the decode kernel (smsp__inst_executed.sum x 32 / texels) come from
# this capture (its line "thread_instructions_per_texel: N"): the third bound, SIMT instruction issue.
INSTRUCTION_CAPTURE = "profiles/decode_kernel_ref_fp8_2048sq_ncu_full.md"


def captured_figure(path: str, key: str):
    """A `key: number` line of a capture summary under profiles/, or None."""
    try:
        with open(os.path.join(ROOT, path)) as f:
            for line in f:
                if line.strip().startswith(key + ":"):
                    return float(line.split(":", 1)[1].split()[0])
    except Exception:
        pass
    return None


def measured_tensor_peak_tflops():
    """Dense 8-bit tensor peak used for the MMA bound: no 8-bit GEMM peak is measured on this pool,
    so twice the measured bf16 burst figure stands in (8-bit operands run at twice the 16-bit rate)."""
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return 2.0 * float(json.load(f)["bf16_tflops"]), "2 x measured bf16 burst (no 8-bit peak is measured)"
    except Exception:
        return 2.0 * 1590.0, "2 x fallback bf16 burst"


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
                 "-lms", "50"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
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


WORKLOADS = {
    0: "single texture set 1024x1024, 4 channels, mip 0 only, latent shape {2, 8 features}, int8 weights",
    1: WORKLOAD,
    2: "64 texture sets 2048x2048, 8 channels, 12 mips each, latent shape {4, 8 features}, int8 weights, sharded by set",
    3: "texture set 8192x8192, 16 channels, 14 mips, latent shape {4, 16 features}, int8 weights, sharded by tile rows",
    4: "inference on sample: 16,777,216 random (u, v, lod) queries on the 4096x4096 12-channel FP8 set (latents re-laid pixel-major once per set), split over the ranks",
}
SAMPLE_QUERIES = 1 << 24


def config_block(config: int, numerics_name: str, job_texels: int, rank_texels: int) -> dict:
    """The `config` object of the JSON line; both arms print the same keys and, for the same workload
    and rank count, the same values."""
    return {"workload": WORKLOADS[config], "numerics": numerics_name,
            "texels_per_step": job_texels, "texels_per_step_this_rank": rank_texels,
            "parallelism": "sharded by texture set / tile rows, no collective",
            "l2": "256 MiB written between steps, outside the per-step events; each step's output also exceeds L2"}


def build_launches(config: int, rank: int, world: int, device, binding, synthetic, sharding, numerics: int):
    """The decode launches one rank issues per step: [(resident set, params)], the texels they
    produce on this rank, the texels of the whole job, algorithmic bytes of this rank's step and
    the synthetic set used for the CPU baseline."""
    launches, texels, alg_bytes = [], 0, 0
    if config in (0, 1):
        spec = synthetic.config_spec(config)
        spec.seed += 1000 * rank  # every rank decodes its own texture set (weak scaling)
        data = synthetic.make_texture_set(spec)
        resident = binding.ResidentTextureSet.from_synthetic(data, device=str(device), numerics=numerics)
        launches.append((resident, resident.params(data.use_int8)))
        texels = data.geometry.total_texels
        alg_bytes = texels * data.geometry.channels * 2 + data.geometry.encoded_latent_bytes + binding.STAGED_NETWORK_BYTES
        return launches, texels, texels * world, alg_bytes, data, "weak"
    if config == 2:
        specs = [synthetic.config_spec(2, i) for i in range(64)]
        geometries = [spec.geometry() for spec in specs]
        plan = sharding.plan_batch(geometries, world)[rank]
        by_set = {}
        for unit in plan:
            by_set.setdefault(unit.set_index, set()).update(unit.mips)
        first = None
        for index, mips in sorted(by_set.items()):
            data = synthetic.make_texture_set(specs[index])
            first = first or data
            resident = binding.ResidentTextureSet.from_synthetic(data, device=str(device), numerics=numerics)
            launches.append((resident, resident.params(True, mips=sorted(mips))))
            done = sum(data.geometry.color_mips[m].width * data.geometry.color_mips[m].height for m in mips)
            texels += done
            alg_bytes += done * data.geometry.channels * 2 + data.geometry.encoded_latent_bytes + binding.STAGED_NETWORK_BYTES
        return launches, texels, sum(g.total_texels for g in geometries), alg_bytes, first, "strong"
    if config == 3:
        data = synthetic.make_texture_set(synthetic.config_spec(3))
        geo = data.geometry
        ranges = sharding.plan_rows(geo, world)[rank]
        resident = binding.ResidentTextureSet.from_synthetic(data, device=str(device), numerics=numerics)
        mips = [m for m, (b, e) in enumerate(ranges) if e > b]
        launches.append((resident, resident.params(True, mips=mips, row_ranges={m: ranges[m] for m in mips})))
        texels = sharding.texels_of_rows(geo, ranges)
        alg_bytes = texels * geo.channels * 2 + geo.encoded_latent_bytes + binding.STAGED_NETWORK_BYTES
        return launches, texels, geo.total_texels, alg_bytes, data, "strong"
    raise ValueError("unknown configuration")


class SampleJob:
    """Configuration 4 on one rank: this rank's slice of the query array against its resident copy
    of the 4096x4096 FP8 set (the set is replicated, the queries are split)."""

    def __init__(self, rank: int, world: int, device, binding, synthetic, numerics: int, interleaved: bool = True):
        import torch

        # interleaved: the queries read the pixel-major copy of the latents (ntcb_interleave_latents: one launch of
        # about 0.1 ms per texture set, made here, before the timed region - like staging the network)
        self.interleaved = interleaved
        self.data = synthetic.make_texture_set(synthetic.config_spec(4))
        self.resident = binding.ResidentTextureSet.from_synthetic(self.data, device=str(device), numerics=numerics,
                                                                  allocate_output=False)
        begin, end = SAMPLE_QUERIES * rank // world, SAMPLE_QUERIES * (rank + 1) // world
        queries = synthetic.make_queries(SAMPLE_QUERIES, max_lod=12.0, seed=9)[begin:end]
        self.queries = torch.from_numpy(np.ascontiguousarray(queries)).to(device)
        self.count = end - begin
        geo = self.data.geometry
        # per query: 12 B in, 2 B x channels out, plus the set once
        self.algorithmic_bytes = self.count * (12 + 2 * geo.channels) + geo.encoded_latent_bytes + binding.STAGED_NETWORK_BYTES

        if interleaved:
            self.resident.interleave_latents()

    def step(self):
        self.out = self.resident.sample(self.queries, False, interleaved=self.interleaved)

    def check_status(self):
        self.resident.check_status()


def time_steps(torch, dist, device, step, checks, steps: int, warmup: int, flush):
    """W untimed steps, then K steps each bracketed by CUDA events on the launching stream (the L2
    flush sits between the events of consecutive steps), barrier + synchronize on both sides.
    Returns (seconds summed over the K steps, max over ranks; per-step milliseconds of this rank;
    wall seconds of the timed region)."""
    for _ in range(warmup):
        step()
    torch.cuda.synchronize()
    for check in checks:
        check()
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
    stops = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
    barrier_sync(dist, torch)
    wall_start = time.perf_counter()
    for index in range(steps):
        flush.fill_(index & 0xFF)  # evict L2 between steps (not inside the per-step events)
        starts[index].record()
        step()
        stops[index].record()
    barrier_sync(dist, torch)
    wall = time.perf_counter() - wall_start
    for check in checks:
        check()
    step_ms = [s.elapsed_time(e) for s, e in zip(starts, stops)]
    return reduce_max(dist, torch, sum(step_ms) / 1e3, device), step_ms, wall


def measure_other_config(config: int, rank: int, world: int, dist, device, binding, synthetic, sharding, numerics: int,
                         steps: int, flush) -> dict:
    """Device-resident throughput of one of the other benchmark configurations at this launch's rank
    count (a sub-record of the default line; the same figure `--config N` reports on its own)."""
    import torch

    if config == 4:
        job = SampleJob(rank, world, device, binding, synthetic, numerics)
        seconds, step_ms, _ = time_steps(torch, dist, device, job.step, [job.check_status], steps, 3, flush)
        record = {"workload": WORKLOADS[4], "value": SAMPLE_QUERIES * steps / seconds / 1e9, "unit": "Gquery/s",
                  "ms_per_step": seconds * 1e3 / steps, "scaling": "strong", "queries_this_rank": job.count,
                  "latents": "pixel-major copy made once per set by ntcb_interleave_latents (outside the timed region)"}
        # the same queries against the latents in the file's order
        job.interleaved = False
        seconds, _, _ = time_steps(torch, dist, device, job.step, [job.check_status], steps, 3, flush)
        record["value_with_latents_in_file_order"] = SAMPLE_QUERIES * steps / seconds / 1e9
        del job
    else:
        launches, texels, job_texels, _, _, scaling = build_launches(config, rank, world, device, binding, synthetic,
                                                                     sharding, numerics)

        def step():
            for resident, params in launches:
                resident.launch(params)

        seconds, step_ms, _ = time_steps(torch, dist, device, step, [r.check_status for r, _ in launches], steps, 3, flush)
        record = {"workload": WORKLOADS[config], "value": job_texels * steps / seconds / 1e9, "unit": UNIT,
                  "ms_per_step": seconds * 1e3 / steps, "scaling": scaling, "texels_per_step": job_texels,
                  "texels_per_step_this_rank": texels, "launches_per_step_this_rank": len(launches)}
        launches.clear()
    record["steps"] = steps
    torch.cuda.empty_cache()
    return record


def run_ours(args) -> dict:
    import torch

    entry.load_package()
    from rtxntc_library_b200 import binding, sharding, synthetic

    rank, local_rank, world, dist = dist_setup(args.gpus)
    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)

    numerics = binding.NUMERICS_EXACT if args.numerics == "exact" else binding.NUMERICS_REFERENCE
    numerics_name = "reference" if numerics == binding.NUMERICS_REFERENCE else "exact"
    flush = torch.empty(L2_FLUSH_BYTES, dtype=torch.uint8, device=device)

    if args.config == 4:
        job = SampleJob(rank, world, device, binding, synthetic, numerics)
        launches, texels, job_texels, algorithmic_bytes, data, scaling = [], job.count, SAMPLE_QUERIES, job.algorithmic_bytes, job.data, "strong"
        step, checks = job.step, [job.check_status]
    else:
        launches, texels, job_texels, algorithmic_bytes, data, scaling = build_launches(
            args.config, rank, world, device, binding, synthetic, sharding, numerics)

        def step():
            for resident, params in launches:
                resident.launch(params)

        checks = [resident.check_status for resident, _ in launches]
    geo = data.geometry
    use_int8 = data.use_int8

    # ---- device-resident throughput -------------------------------------------------------
    # nvidia-smi needs a moment before its first sample: start it ahead of the warm-up so that the
    # (short) timed region is covered
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.5)
    launches_before = binding.lib().ntcb_launch_count()
    device_seconds, step_ms, wall = time_steps(torch, dist, device, step, checks, args.steps, args.warmup, flush)
    clocks = sampler.stop() if rank == 0 else None
    # launches inside the timed region (the warm-up steps are the same launches, untimed)
    launch_count = (binding.lib().ntcb_launch_count() - launches_before) * args.steps // (args.steps + args.warmup)
    total_launches = int(reduce_sum(dist, torch, float(launch_count), device))
    value = job_texels * args.steps / device_seconds / 1e9

    # ---- the other configurations, device-resident, at this rank count ------------------------
    other_configs = None
    if args.config == 1 and not args.no_other_configs:
        launches.clear()
        torch.cuda.empty_cache()
        other_steps = max(3, min(args.steps, 10))
        other_configs = {}
        for other in (0, 2, 3, 4):
            record = measure_other_config(other, rank, world, dist, device, binding, synthetic, sharding, numerics,
                                          other_steps, flush)
            other_configs["config_%d" % other] = record

    # ---- end to end through the texture-set API with host buffers ---------------------------
    e2e = None
    e2e_unorm8 = None
    e2e_ceiling = None
    if args.config in (0, 1):
        launches.clear()
        del flush
        torch.cuda.empty_cache()
        context = binding.Context(local_rank)
        texture_set = context.create_texture_set(data.container, numerics=numerics)
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
        e2e = {"value": world * texels * args.steps / e2e_seconds / 1e9, "unit": UNIT,
               "h2d_bytes_per_step": geo.encoded_latent_bytes + 2 * binding.STAGED_NETWORK_BYTES,
               "d2h_bytes_per_step": texels * geo.channels * 2}

        # The ceiling of that job on this machine: the same device-to-host bytes as one plain
        # cudaMemcpyAsync per step into the same pinned buffer, every rank at once, no decode.
        device_texels = torch.empty(texels * geo.channels, dtype=torch.float16, device=device)
        for _ in range(2):
            host_out.copy_(device_texels, non_blocking=True)
        barrier_sync(dist, torch)
        copy_start = time.perf_counter()
        for _ in range(args.steps):
            host_out.copy_(device_texels, non_blocking=True)
        torch.cuda.synchronize()
        copy_seconds = reduce_max(dist, torch, time.perf_counter() - copy_start, device)
        barrier_sync(dist, torch)
        del device_texels
        ceiling = world * texels * args.steps / copy_seconds / 1e9
        e2e_ceiling = {"value": ceiling, "unit": UNIT, "gb_per_s": world * texels * geo.channels * 2 * args.steps / copy_seconds / 1e9,
                       "e2e_fraction_of_ceiling": e2e["value"] / ceiling,
                       "what": "plain device-to-host copies of one step's texels into pinned host memory on all %d ranks at "
                               "once (no decode, no upload): what the host link sustains" % world}

        if args.config == 1:
            # the same job with UNORM8 pixels as the client's format: one fused launch writes them, the
            # read-back is half the size (the reference arm runs Decompress + ReadChannels(UNORM8))
            conversion = binding.make_conversion(binding.CHANNEL_FORMAT_UNORM8, geo.channels)
            host_bytes = torch.empty(texels * geo.channels, dtype=torch.uint8).pin_memory()

            def unorm8_step():
                binding.check(binding.lib().ntcb_texture_set_decompress_converted(
                    texture_set.handle, None, 1 if use_int8 else 0, ctypes.byref(conversion), binding.ADDRESS_SPACE_HOST,
                    host_bytes.data_ptr(), host_bytes.numel()))

            for _ in range(2):
                unorm8_step()
            barrier_sync(dist, torch)
            unorm8_start = time.perf_counter()
            for _ in range(args.steps):
                unorm8_step()
            unorm8_seconds = reduce_max(dist, torch, time.perf_counter() - unorm8_start, device)
            barrier_sync(dist, torch)
            e2e_unorm8 = {"value": world * texels * args.steps / unorm8_seconds / 1e9, "unit": UNIT,
                          "h2d_bytes_per_step": e2e["h2d_bytes_per_step"], "d2h_bytes_per_step": texels * geo.channels,
                          "path": "ntcb_texture_set_decompress_converted(UNORM8, all channels, Linear) to pinned host memory"}
        texture_set.close()
        context.close()

    # ---- roofline of the decode kernel (this rank's launches of one step) ---------------------
    peak, peak_kind = measured_peak_gbs()
    step_seconds = statistics.mean(step_ms) / 1e3
    achieved = algorithmic_bytes / step_seconds / 1e9
    traffic = captured_figure(TRAFFIC_CAPTURE, "traffic_bytes_per_launch") if args.config == 1 else None
    roofline = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                "traffic": traffic, "traffic_source": TRAFFIC_CAPTURE if traffic is not None else None,
                "peak_source": "%s copy bandwidth" % peak_kind, "algorithmic_bytes_per_step": algorithmic_bytes,
                "launches_per_step": launch_count // max(1, args.steps)}
    if args.config != 4:
        # the other two bounds of a tile: the matrix products at the 8-bit tensor peak, and SIMT
        # instruction issue (every SM sub-partition issues one warp instruction per clock)
        tensor_peak, tensor_source = measured_tensor_peak_tflops()
        flops = 16384.0 * texels
        roofline["mma"] = {"achieved": flops / step_seconds / 1e12, "peak": tensor_peak, "unit": "TFLOP/s",
                           "frac": flops / step_seconds / 1e12 / tensor_peak, "flops_per_texel": 16384, "peak_source": tensor_source}
        t_hbm, t_mma = algorithmic_bytes / (peak * 1e9), flops / (tensor_peak * 1e12)
        roofline["tile"] = {"t_hbm_ms": t_hbm * 1e3, "t_mma_ms": t_mma * 1e3, "frac": max(t_hbm, t_mma) / step_seconds,
                            "what": "the slower of the bytes at the HBM peak and the matrix products at the 8-bit tensor peak, over the measured time"}
        instructions = captured_figure(INSTRUCTION_CAPTURE, "thread_instructions_per_texel") if args.config == 1 else None
        if instructions:
            properties = torch.cuda.get_device_properties(device)
            sm_hz = (clocks or {}).get("sm_mhz") or 1965.0
            issue_peak = properties.multi_processor_count * 4 * 32 * sm_hz * 1e6 / instructions / 1e9
            roofline["simt"] = {"thread_instructions_per_texel": instructions, "source": INSTRUCTION_CAPTURE,
                                "peak": issue_peak, "unit": UNIT, "frac": (texels / step_seconds / 1e9) / issue_peak,
                                "what": "SMs x 4 sub-partitions x 32 lanes x SM clock / thread instructions per texel"}
    if numerics == binding.NUMERICS_REFERENCE:
        dtype = ("f16 x f16 -> f16 (tcgen05 kind::f16, binary16 accumulators rounded per 16 products: the reference's own "
                 "arithmetic on int8 weights, reproduced bit for bit)" if use_int8 else
                 "e4m3 x e4m3 -> f16 (tcgen05 kind::f8f6f4, binary16 accumulators, 16 non-zero products per rounding; last layer "
                 "f16 x f16 -> f16): the reference's own arithmetic, reproduced bit for bit")
    else:
        dtype = ("fp8_e4m3 x fp8_e4m3 -> f32 (layers 0-2), s8 x s8 -> s32 (layer 3), f16 activations" if not use_int8
                 else "s8 x s8 -> s32 (all layers), f16 activations")
    line = {
        "metric": METRIC if args.config != 4 else "inference-on-sample Gquery/s", "value": value,
        "unit": UNIT if args.config != 4 else "Gquery/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": device_seconds * 1e3 / args.steps, "higher_is_better": True, "scaling": scaling,
        "vs_baseline": None, "dtype": dtype,
        "data": "synthetic (seeded latents and weights of the configuration's shape)",
        "config": config_block(args.config, numerics_name, job_texels, texels),
        "clocks": clocks, "e2e": e2e, "gpu_launches": total_launches, "roofline": roofline,
        "wall_seconds_timed_region": wall,
    }
    if e2e_ceiling is not None:
        line["e2e_ceiling"] = e2e_ceiling
    if e2e_unorm8 is not None:
        line["e2e_unorm8"] = e2e_unorm8
    if other_configs is not None:
        line["other_configs"] = other_configs
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
    flush = torch.empty(L2_FLUSH_BYTES, dtype=torch.uint8, device="cuda:0")

    # ---- device figure: the reference's own timing of its mip loop, L2 flushed between steps ----
    for _ in range(args.warmup):
        decoder.decompress(data.use_int8)
    sampler = ClockSampler(0)
    torch.cuda.synchronize()
    sampler.start()
    time.sleep(0.5)
    kernel_ms = []
    for index in range(args.steps):
        flush.fill_(index & 0xFF)
        torch.cuda.synchronize()
        kernel_ms.append(decoder.decompress(data.use_int8))
    clocks = sampler.stop()
    kernel_seconds = sum(kernel_ms) / 1e3
    value = texels * args.steps / kernel_seconds / 1e9

    # ---- end to end: Decompress + ReadChannels(FLOAT16, Host) of every mip, wall clock ----------
    def step():
        decoder.decompress(data.use_int8)
        for mip, cm in enumerate(geo.color_mips):
            decoder.read_mip_into(mip, cm.width, cm.height, base + cm.texel_offset * geo.channels * 2, False)

    for _ in range(max(1, min(args.warmup, 3))):
        step()
    torch.cuda.synchronize()
    start = time.perf_counter()
    for _ in range(args.steps):
        step()
    torch.cuda.synchronize()
    seconds = time.perf_counter() - start

    # the same job with UNORM8 pixels as the client's format
    host_bytes = torch.empty(texels * geo.channels, dtype=torch.uint8).pin_memory()

    def unorm8_step():
        decoder.decompress(data.use_int8)
        for mip, cm in enumerate(geo.color_mips):
            decoder.read_channels_into(mip, cm.width, cm.height, 1, geo.channels,
                                       host_bytes.data_ptr() + cm.texel_offset * geo.channels)

    unorm8_step()
    torch.cuda.synchronize()
    unorm8_start = time.perf_counter()
    for _ in range(args.steps):
        unorm8_step()
    torch.cuda.synchronize()
    unorm8_seconds = time.perf_counter() - unorm8_start
    decoder.close()
    e2e_value = texels * args.steps / seconds / 1e9

    # The same calls on the same reference build with ONE translation unit changed: TextureSet::Decompress
    # routed to libntcb200.so (oracle/_ref/libntc_ref_ntcb.so).  What an application linked against
    # ntc.h gets from the integration, measured through ntc.h.
    via_ntc_h = None
    if oracle_py.reference_ntcb_available():
        routed = oracle_py.ReferenceDecoder(data.container, geo.channels, device=0, library=oracle_py.REF_NTCB_LIB)

        def routed_step():
            routed.decompress(data.use_int8)
            for mip, cm in enumerate(geo.color_mips):
                routed.read_mip_into(mip, cm.width, cm.height, base + cm.texel_offset * geo.channels * 2, False)

        for _ in range(max(1, min(args.warmup, 3))):
            routed_step()
        routed_ms = []
        for index in range(args.steps):
            flush.fill_(index & 0xFF)
            torch.cuda.synchronize()
            routed_ms.append(routed.decompress(data.use_int8))
        torch.cuda.synchronize()
        routed_start = time.perf_counter()
        for _ in range(args.steps):
            routed_step()
        torch.cuda.synchronize()
        routed_seconds = time.perf_counter() - routed_start
        routed.close()
        via_ntc_h = {"value": texels * args.steps / (sum(routed_ms) / 1e3) / 1e9, "unit": UNIT,
                     "e2e": texels * args.steps / routed_seconds / 1e9,
                     "what": "the reference library with TextureSet::Decompress routed to libntcb200.so, driven through "
                             "ntc::CreateContext / ITextureSet::Decompress / ITextureSet::ReadChannels like the stock arm: "
                             "value from DecompressionStats::gpuTimeMilliseconds, e2e wall clock with ReadChannels(FLOAT16, Host)"}
    # every Decompress of a set loaded from a file uploads the encoded latents and both weight blobs
    # again (src/TextureSet.cpp:1695-1719); ReadChannels(Host) copies every mip back
    h2d = geo.encoded_latent_bytes + 9472 + 8608
    return {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "gpus_used": 1,
        "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": kernel_seconds * 1e3 / args.steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f16 x f16 -> f16 (wmma), as the reference's CUDA decoder computes",
        "data": "synthetic (seeded latents and weights of the configuration's shape)",
        "config": config_block(1, "reference", texels * world, texels),
        "reference_path": "CreateCompressedTextureSetFromMemory once; value: DecompressionStats::gpuTimeMilliseconds of "
                          "Decompress (its mip loop; upload, latent unpacking and weight conversion excluded); e2e: wall clock "
                          "of Decompress + ReadChannels(FLOAT16, Host) of every mip.  The reference has no CPU decoder and no "
                          "multi-GPU path: one rank runs its CUDA decoder on GPU 0"
                          + ("; the other %d ranks idle" % (world - 1) if world > 1 else ""),
        "clocks": clocks,
        "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": texels * geo.channels * 2,
                "ms_per_step": seconds * 1e3 / args.steps},
        "e2e_unorm8": {"value": texels * args.steps / unorm8_seconds / 1e9, "unit": UNIT,
                       "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": texels * geo.channels,
                       "path": "per step Decompress + ReadChannels(UNORM8, Host) of every mip"},
        "e2e_via_ntc_h": via_ntc_h,
        "gpu_launches": args.steps * geo.mips,  # the reference launches its kernel once per mip
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": 0, "kind": "reference",
                         "sample": "whole workload; the reference's only decoder is its CUDA kernel, run on the GPU of this box"},
    }


def run_profile_case(case: str) -> int:
    """A few bare launches of the decode kernel on a small square set, for a profiler to capture.

    `case` is SIZE:MODE:LAUNCHES[:NUMERICS], e.g. 2048:fp8:2: a SIZE x SIZE 12-channel set with a full mip chain
    (output larger than L2 from 2048 up, a few hundred MB on the device), MODE fp8 or int8, NUMERICS reference
    (default) or exact.  Prints a plain line, not the benchmark's JSON line: a figure taken under a
    profiler is not a benchmark value.
    """
    import torch

    fields = case.split(":")
    size, mode, launches = fields[:3]
    numerics = fields[3] if len(fields) > 3 else "reference"
    entry.load_package()
    from rtxntc_library_b200 import binding, synthetic

    spec = synthetic.TextureSetSpec(int(size), int(size), 12, 0, 4, 12, seed=1, weights=mode, latent_alphabet="2bit-even")
    data = synthetic.make_texture_set(spec)
    resident = binding.ResidentTextureSet.from_synthetic(
        data, numerics=binding.NUMERICS_EXACT if numerics == "exact" else binding.NUMERICS_REFERENCE)
    params = resident.params(mode == "int8")
    events = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(int(launches))]
    for start, stop in events:
        start.record()
        resident.launch(params)
        stop.record()
    torch.cuda.synchronize()
    resident.check_status()
    times = sorted(start.elapsed_time(stop) for start, stop in events[1:] or events)
    print("profile case %s (%s): %d texels, launches after the first: median %.4f ms, fastest %.4f ms"
          % (case, os.path.basename(binding.LIBRARY_PATH), data.geometry.total_texels, times[len(times) // 2], times[0]))
    return 0


def run_producers_case(side: int) -> int:
    """Times the two encoder-side producers on their own: latent packing on a SIDE x SIDE grid of four
    layers (algorithmic bytes per latent word: 8 read + 2 written; the arrays are larger than L2 from
    SIDE = 4096 up) against the HBM copy peak, and one network quantisation (a single CTA: latency).
    With the reference library present, its own kernels are timed beside them through the harness's
    host-to-host calls (copies included, so only an upper bound on their kernel time).  Prints a
    plain line per producer, not the benchmark's JSON line."""
    import numpy as np
    import torch

    entry.load_package()
    from rtxntc_library_b200 import binding

    layers, texels = 4, side * side
    stride = texels * 2
    latents = (torch.randint(0, 16, (layers * stride * 2,), device="cuda", dtype=torch.int32).to(torch.float16) / 15.0).contiguous()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    times = []
    for _ in range(13):
        start.record()
        packed = binding.pack_latents(latents, side, side, layers, stride)
        stop.record()
        torch.cuda.synchronize()
        times.append(start.elapsed_time(stop))
    ms = float(np.median(times[3:]))
    peak, source = measured_peak_gbs()
    gbs = 10.0 * texels * layers / ms / 1e6
    print("pack latents %dx%dx%d: %.3f ms, %.0f GB/s algorithmic = %.2f of %s HBM peak %.0f GB/s (%d words)"
          % (side, side, layers, ms, gbs, gbs / peak, source, peak, packed.numel()))

    rng = np.random.default_rng(1)
    weights = torch.from_numpy(rng.normal(0, 0.3, binding.NETWORK_WEIGHT_COUNT).astype(np.float16)).cuda()
    biases = torch.from_numpy(rng.normal(0, 0.5, binding.NETWORK_COLUMN_COUNT).astype(np.float16)).cuda()
    for mode, name in ((binding.WEIGHTS_INT8, "int8"), (binding.WEIGHTS_FP8, "fp8")):
        times = []
        for _ in range(13):
            start.record()
            binding.quantize_network(weights, biases, mode)
            stop.record()
            torch.cuda.synchronize()
            times.append(start.elapsed_time(stop))
        print("quantize network %s: %.1f us per call (blob allocation included)" % (name, 1000 * float(np.median(times[3:]))))
    return 0


def run_block_compress_case(side: int) -> int:
    """Times BC4, BC5, BC1, BC2 and BC3 encoding of a SIDE x SIDE mip of 12 interleaved fp16 channels (random texels
    with smooth and noisy regions; larger than L2 from SIDE = 4096 up).  Prints a plain line per
    format, not the benchmark's JSON line."""
    import numpy as np
    import torch

    entry.load_package()
    from rtxntc_library_b200 import binding

    generator = torch.Generator(device="cuda").manual_seed(3)
    base = torch.rand((side // 16, side // 16, 12), device="cuda", generator=generator)
    texels = torch.nn.functional.interpolate(base.permute(2, 0, 1)[None], size=(side, side), mode="bilinear")[0].permute(1, 2, 0)
    texels = (texels + 0.05 * torch.rand((side, side, 12), device="cuda", generator=generator)).clamp(0, 1).to(torch.float16).contiguous()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    peak, source = measured_peak_gbs()
    for block_format, name, channels in ((binding.BLOCK_FORMAT_BC4, "BC4", 1), (binding.BLOCK_FORMAT_BC5, "BC5", 2),
                                         (binding.BLOCK_FORMAT_BC1, "BC1", 3), (binding.BLOCK_FORMAT_BC2, "BC2", 4),
                                         (binding.BLOCK_FORMAT_BC3, "BC3", 4)):
        times = []
        for _ in range(13):
            start.record()
            binding.block_compress(texels, block_format, 2)
            stop.record()
            torch.cuda.synchronize()
            times.append(start.elapsed_time(stop))
        ms = float(np.median(times[3:]))
        touched = side * side * (24 + (0.5 if block_format in (1, 4) else 1.0))  # every 32-byte sector of the interleaved mip is read
        print("%s of %dx%d (12 interleaved channels): %.3f ms, %.1f Gtexel/s, %.0f GB/s of sectors touched = %.2f of %s HBM peak"
              % (name, side, side, ms, side * side / ms / 1e6, touched / ms / 1e6, touched / ms / 1e6 / peak, source))
    # BC7: the full search once (it is the offline path), then with the mode buffer made from its own blocks
    timings = {}
    blocks = None
    for name, repeats in (("BC7, full search", 4), ("BC7, mode buffer", 13)):
        modes = None
        if blocks is not None:
            modes = torch.from_numpy(binding.make_bc7_mode_buffer(blocks.cpu().numpy())).cuda()
        times = []
        for _ in range(repeats):
            start.record()
            result = binding.block_compress(texels, binding.BLOCK_FORMAT_BC7, 2, mode_buffer=modes)
            stop.record()
            torch.cuda.synchronize()
            times.append(start.elapsed_time(stop))
        if blocks is None:
            blocks = result
        else:
            timings["same"] = bool(torch.equal(result, blocks))
        ms = float(np.median(times[1:]))
        print("%s of %dx%d (12 interleaved channels): %.3f ms, %.2f Gtexel/s" % (name, side, side, ms, side * side / ms / 1e6))
    print("the mode-buffer path reproduces the full search's blocks: %s" % timings.get("same"))
    return 0


def run_batch_case(count: int) -> int:
    """Times ntcb_batch_decoder_run and ntcb_decode_batch - ONE process, every visible GPU - on `count` texture sets of the batch
    configuration's shape (2048 x 2048, 8 channels, 12 mips, Int8 weights) gathered in pinned host memory,
    and beside it what plain device-to-host copies of the same bytes sustain on the same GPUs at once (the
    ceiling of any job with host destinations).  Prints plain lines, not the benchmark's JSON line."""
    import torch

    entry.load_package()
    from rtxntc_library_b200 import binding, synthetic

    devices = list(range(torch.cuda.device_count()))
    spec = synthetic.config_spec(2, 0)
    sets = [synthetic.make_texture_set(synthetic.config_spec(2, index % 4)) for index in range(min(count, 4))]
    containers = [sets[index % len(sets)].container for index in range(count)]
    geometry = sets[0].geometry
    values = geometry.total_texels * geometry.channels
    images = [torch.empty(values, dtype=torch.float16).pin_memory() for _ in range(count)]
    times = []
    with binding.BatchDecoder(devices) as decoder:
        for _ in range(5):
            begin = time.perf_counter()
            code, statuses, units = decoder.run(containers, True, images)
            times.append(time.perf_counter() - begin)
            if code != 0 or any(statuses):
                print("ntcb_batch_decoder_run failed: %d %s" % (code, binding.lib().ntcb_last_error()))
                return 1
    begin = time.perf_counter()
    code, statuses, units = binding.decode_batch(containers, devices, True, images)
    one_shot = time.perf_counter() - begin
    seconds = min(times[1:])
    texels = geometry.total_texels * count
    per_device = {}
    for unit in units:
        per_device[unit.device] = per_device.get(unit.device, 0) + unit.texels
    # the ceiling: every device copies its share of the bytes to pinned host memory, all at once
    share = values * 2 * count // len(devices)
    sources = []
    for device in devices:
        with torch.cuda.device(device):
            sources.append(torch.empty(share, dtype=torch.uint8, device="cuda:%d" % device))
    targets = [torch.empty(share, dtype=torch.uint8).pin_memory() for _ in devices]
    copy_times = []
    for _ in range(4):
        for device in devices:
            torch.cuda.synchronize(device)
        begin = time.perf_counter()
        for device, source, target in zip(devices, sources, targets):
            with torch.cuda.device(device):
                target.copy_(source, non_blocking=True)
        for device in devices:
            torch.cuda.synchronize(device)
        copy_times.append(time.perf_counter() - begin)
    ceiling_seconds = min(copy_times[1:])
    print("ntcb_batch_decoder_run: %d sets of %dx%d x %d channels on %d GPU(s), %d work units: %.1f ms = %.2f Gtexel/s end to end "
          "(containers parsed, uploaded, decoded, %.0f MB gathered in pinned host memory); the decoder's first run %.1f ms; "
          "ntcb_decode_batch (create + run + destroy) %.1f ms"
          % (count, spec.width, spec.height, geometry.channels, len(devices), len(units), seconds * 1e3, texels / seconds / 1e9,
             values * 2 * count / 1e6, times[0] * 1e3, one_shot * 1e3))
    print("texels per device: %s" % ", ".join("%d: %.1f M" % (d, t / 1e6) for d, t in sorted(per_device.items())))
    print("plain D2H copies of the same bytes from %d GPU(s) at once: %.1f ms = %.1f GB/s = %.2f Gtexel/s; the batch call is at %.2f of it"
          % (len(devices), ceiling_seconds * 1e3, values * 2 * count / ceiling_seconds / 1e9, texels / ceiling_seconds / 1e9,
             ceiling_seconds / seconds))
    return 0


def main() -> int:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=100)
    parser.add_argument("--warmup", type=int, default=3)
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--no-cpu-baseline", action="store_true")
    parser.add_argument("--no-other-configs", action="store_true",
                        help="skip the sub-records of configurations 0, 2, 3 and 4 in the default line")
    parser.add_argument("--config", type=int, default=1, choices=[0, 1, 2, 3, 4],
                        help="benchmark configuration; 1 (the default) is the one the metric is quoted on")
    parser.add_argument("--numerics", default="reference", choices=["reference", "exact"],
                        help="reference (default): binary16 accumulation, the reference decoder's bits; exact: exact accumulation")
    parser.add_argument("--profile-case", metavar="SIZE:MODE:LAUNCHES[:NUMERICS]",
                        help="only launch the decode kernel LAUNCHES times on a small SIZE^2 set (fp8 or int8) and exit")
    parser.add_argument("--producers-case", metavar="SIDE", type=int,
                        help="only time latent packing on a SIDE x SIDE x 4 grid and one network quantisation, and exit")
    parser.add_argument("--block-compress-case", metavar="SIDE", type=int,
                        help="only time BC1 - BC5 and BC7 encoding of a SIDE x SIDE 12-channel mip, and exit")
    parser.add_argument("--batch-case", metavar="SETS", type=int,
                        help="only time ntcb_decode_batch (one process, every visible GPU) on SETS texture sets, and exit")
    args = parser.parse_args()
    if args.batch_case:
        return run_batch_case(args.batch_case)
    if args.profile_case:
        return run_profile_case(args.profile_case)
    if args.producers_case:
        return run_producers_case(args.producers_case)
    if args.block_compress_case:
        return run_block_compress_case(args.block_compress_case)
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else max(args.warmup, 1)
    line = run_reference(args) if args.impl == "reference" else run_ours(args)
    if line is not None:
        print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
