"""Benchmark of the hot path: `scaled_mm` bf16 activations x prepacked fp8-e5m2 weights at the
diffusion-transformer MLP-up shape (M=4096 tokens, K=3072, N=12288), bf16 output, fp32 accumulation.

    python bench.py [--gpus N] [--steps K] [--warmup W]            # this library on N GPUs (torchrun for N > 1)
    python bench.py --impl reference [--steps K] [--warmup W]      # the reference's CPU path on the host cores

One step = one pass of the operator over one batch of synthetic activations. With N GPUs every rank owns
its own 4096-token shard of a 4096*N-token batch against replicated weights (the token dimension is the
data-parallel one), so there is no collective on the data path and scaling is weak. Rank 0 prints one JSON
line. `value` is the whole-job TFLOP/s with inputs resident in HBM; `e2e` is the same metric through the
public Python API with the activations in pinned host memory and the result read back to the host every
step (the weights stay resident: they are model state, not step input).
"""

import argparse
import datetime
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

import torch

M, K, N = 4096, 3072, 12288
FLOP_PER_STEP = 2 * M * K * N
# A (bf16) + prepacked B (fp8) + C (bf16): the bytes one launch has to move at least once
ALGORITHMIC_BYTES = M * K * 2 + K * N + M * N * 2
ROTATING_SETS = 4  # distinct input/output sets cycled between steps: 4 x 164 MB > the 126 MB L2
# dram__bytes_read.sum + dram__bytes_write.sum of one launch at this shape, from the ncu capture summarized
# in profiles/scaled_mm_pair_4096x12288x3072_ncu.md (64.24 MB read + 62.41 MB written; less than the algorithmic
# bytes because part of the output is still in L2 when the kernel ends)
NCU_DRAM_BYTES_PER_LAUNCH = 126_650_000
METRIC = "scaled_mm TFLOP/s (bf16@fp8e5m2, 4096x3072x12288)"
CPU_SAMPLE_ROWS = 1024


def measured_peak():
    """`(burst, sustained, source)`: the driver-measured cuBLAS bf16 rates of this pool (best single launch, and a
    seconds-long loop under the power cap), or the stated fallback."""
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            peaks = json.load(f)
        return float(peaks["bf16_tflops"]), float(peaks.get("bf16_tflops_sustained", 0.0)) or None, "measured (cuBLAS bf16 burst, MEASURED_PEAKS.json)"
    except (OSError, KeyError, ValueError):
        return 1590.0, 1400.0, "fallback (earlier pool measurement, cuBLAS bf16 burst)"


def make_inputs(seed):
    """Benchmark distribution: A ~ N(0, 1) bf16; W ~ N(0, 0.02) quantized to e5m2 with scale = absmax / 57344."""
    from feather_ops_b200.scaled_mm import prepack_b_for_scaled_mm

    gen = torch.Generator().manual_seed(seed)
    a = torch.randn((M, K), generator=gen, dtype=torch.float32).to(torch.bfloat16)
    w = torch.randn((K, N), generator=gen, dtype=torch.float32) * 0.02
    scale = (w.abs().max() / 57344.0).to(torch.float32)
    b = (w / scale).to(torch.float8_e5m2)
    return a, prepack_b_for_scaled_mm(b), scale


class ClockSampler:
    """nvidia-smi clock and throttle-reason samples of one GPU, every 20 ms, each with its wall-clock time. It is
    started before the warm-up, so it is already running when the timed region begins; `stop(window)` keeps the
    samples whose time stamps fall inside the window (the timed region)."""

    QUERY = "timestamp,index,clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap,clocks_event_reasons.active,power.draw"

    def __init__(self, gpu_index):
        self.gpu_index = gpu_index
        self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "20"],
                                         stdout=self.file, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self, window=None):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        self.file.flush()
        self.file.seek(0)
        clocks, max_clock, reasons, mask, watts = [], None, set(), 0, []
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in self.file.read().splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) != 10 or not parts[1].isdigit() or int(parts[1]) != self.gpu_index:
                continue
            if window is not None:
                try:
                    stamp = datetime.datetime.strptime(parts[0], "%Y/%m/%d %H:%M:%S.%f")
                except ValueError:
                    continue
                if not (window[0] <= stamp <= window[1]):
                    continue
            try:
                clocks.append(float(parts[2]))
                max_clock = float(parts[3])
            except ValueError:
                continue
            for name, flag in zip(names, parts[4:]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
            try:
                mask |= int(parts[8], 16)   # every event reason the driver reports, as its bit mask
                watts.append(float(parts[9]))
            except ValueError:
                pass
        self.file.close()
        os.unlink(self.file.name)
        if not clocks:
            return {"sm_mhz": None, "sm_max_mhz": max_clock, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(clocks), "sm_max_mhz": max_clock, "reasons": sorted(reasons), "samples": len(clocks),
                "reasons_mask": hex(mask), "power_w": statistics.median(watts) if watts else None}


def use_all_host_threads():
    """torchrun exports OMP_NUM_THREADS=1: the CPU legs take every core this process may run on."""
    try:
        cores = len(os.sched_getaffinity(0))
    except AttributeError:
        cores = os.cpu_count() or 1
    torch.set_num_threads(max(1, cores))


def cpu_baseline(threads=None):
    """The reference's CPU path (`scaled_mm_naive`, restated in oracle/scaled_mm.py) on a bounded sample:
    the first CPU_SAMPLE_ROWS token rows of the benchmark batch against the full weight."""
    from oracle import scaled_mm as osm

    if threads:
        torch.set_num_threads(threads)
    else:
        use_all_host_threads()
    a, packed, scale = make_inputs(0)
    a = a[:CPU_SAMPLE_ROWS].contiguous()
    osm.scaled_mm_naive(a, packed, scale, None, torch.bfloat16, b_prepacked=True)  # warm-up
    best = float("inf")
    for _ in range(3):
        t0 = time.perf_counter()
        osm.scaled_mm_naive(a, packed, scale, None, torch.bfloat16, b_prepacked=True)
        best = min(best, time.perf_counter() - t0)
    flop = 2 * CPU_SAMPLE_ROWS * K * N
    return {
        "value": flop / best / 1e12,
        "unit": "TFLOP/s",
        "cores": torch.get_num_threads(),
        "kind": "port",
        "sample": f"first {CPU_SAMPLE_ROWS} of {M} token rows x full {K}x{N} weight, best of 3, torch CPU fp16 matmul as in the reference's naive path",
    }


def run_reference(args):
    """`--impl reference`: the reference's own CPU implementation of the path (no GPU, rank 0 only)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import scaled_mm as osm

    use_all_host_threads()
    a, packed, scale = make_inputs(0)
    a = a[:CPU_SAMPLE_ROWS].contiguous()
    for _ in range(max(1, min(args.warmup, 2))):
        osm.scaled_mm_naive(a, packed, scale, None, torch.bfloat16, b_prepacked=True)
    steps = max(1, args.steps)
    t0 = time.perf_counter()
    for _ in range(steps):
        osm.scaled_mm_naive(a, packed, scale, None, torch.bfloat16, b_prepacked=True)
    elapsed = time.perf_counter() - t0
    flop = 2 * CPU_SAMPLE_ROWS * K * N
    value = flop * steps / elapsed / 1e12
    sample = f"each step = first {CPU_SAMPLE_ROWS} of {M} token rows x full weight on the host cores (oracle port of feather_ops/naive.py)"
    line = {
        "impl": "reference",
        "metric": METRIC,
        "value": value,
        "unit": "TFLOP/s",
        "n_gpus": args.gpus,
        "steps": steps,
        "warmup": args.warmup,
        "ms_per_step": elapsed / steps * 1e3,
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "fp16 (CPU matmul of the reference's naive path)",
        "data": "synthetic",
        "config": {"workload": f"scaled_mm bf16@fp8e5m2 M={M} K={K} N={N}, bf16 out", "sample_rows": CPU_SAMPLE_ROWS},
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def run_library(args):
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the kernels have no CPU fallback")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    distributed = world > 1
    if distributed:
        import torch.distributed as dist

        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=device)

    import feather_ops_b200 as fo
    from feather_ops_b200.scaled_mm import select_scaled_mm_config

    # every rank owns its own token shard (seeded by rank) against replicated weights
    sets = []
    a_host, packed_host, scale_host = make_inputs(rank)
    packed = packed_host.to(device)
    scale = scale_host.to(device)
    for i in range(ROTATING_SETS):
        a = a_host.roll(i, 0).to(device)
        sets.append((a, packed.clone() if i else packed))
    outs = [torch.empty((M, N), device=device, dtype=torch.bfloat16) for _ in range(ROTATING_SETS)]
    tile = select_scaled_mm_config(M, N, K)

    def step(i):
        a, b = sets[i % ROTATING_SETS]
        torch.ops.feather_ops.scaled_mm.default(a, b, scale, None, outs[i % ROTATING_SETS], *tile[:5], bool(tile[5]))

    def barrier():
        if distributed:
            dist.barrier()
        torch.cuda.synchronize()

    # the clock sampler is started before the warm-up so that it is already producing samples when the timed region
    # begins; only the samples time-stamped inside the timed region are kept
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    for i in range(max(3, args.warmup)):
        step(i)
    barrier()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    region_begin = datetime.datetime.now()
    start.record()
    for i in range(args.steps):
        step(i)
    stop.record()
    barrier()
    region_end = datetime.datetime.now()
    elapsed_ms = start.elapsed_time(stop)
    clocks = sampler.stop((region_begin, region_end)) if rank == 0 else None
    if clocks is not None and clocks["samples"] >= 2:
        clocks["note"] = "nvidia-smi samples every 20 ms, time-stamped inside the timed region"
    if distributed:
        t = torch.tensor([elapsed_ms], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        elapsed_ms = float(t.item())
    ms_per_step = elapsed_ms / args.steps
    value = FLOP_PER_STEP * world / (ms_per_step * 1e-3) / 1e12

    # a short sampled run may not have covered the timed region: sample clocks again under a sustained loop
    if rank == 0 and (clocks is None or clocks["samples"] < 2):
        sampler = ClockSampler(local_rank)
        sampler.start()
        t_end = time.perf_counter() + 0.8
        i = 0
        while time.perf_counter() < t_end:
            step(i)
            i += 1
            if i % 64 == 0:
                torch.cuda.synchronize()
        torch.cuda.synchronize()
        clocks = sampler.stop()
        clocks["note"] = "sampled over a 0.8 s loop of the same launches right after the timed region (the timed region was shorter than the sampling period)"

    # ------------------------------------------------------------------ end to end: host buffers, public API
    e2e_steps = max(4, min(args.steps, 20))
    a_pinned = [a_host.roll(i, 0).pin_memory() for i in range(2)]
    c_pinned = [torch.empty((M, N), dtype=torch.bfloat16).pin_memory() for _ in range(2)]
    a_dev = [torch.empty((M, K), device=device, dtype=torch.bfloat16) for _ in range(2)]
    copy_in, copy_out = torch.cuda.Stream(device), torch.cuda.Stream(device)
    compute = torch.cuda.current_stream(device)
    in_done = [torch.cuda.Event() for _ in range(2)]
    mm_done = [torch.cuda.Event() for _ in range(2)]
    out_done = [torch.cuda.Event() for _ in range(2)]
    c_dev = [None, None]

    def e2e_pass(count):
        for i in range(count):
            s = i % 2
            with torch.cuda.stream(copy_in):
                copy_in.wait_event(mm_done[s])  # the previous user of this activation buffer has run
                a_dev[s].copy_(a_pinned[s], non_blocking=True)
                in_done[s].record(copy_in)
            compute.wait_event(in_done[s])
            compute.wait_event(out_done[s])  # the previous result in this slot has left the device
            c_dev[s] = fo.scaled_mm_hip(a_dev[s], packed, scale, None, torch.bfloat16)
            mm_done[s].record(compute)
            with torch.cuda.stream(copy_out):
                copy_out.wait_event(mm_done[s])
                c_pinned[s].copy_(c_dev[s], non_blocking=True)
                out_done[s].record(copy_out)
        copy_out.synchronize()

    e2e_pass(3)
    barrier()
    t0 = time.perf_counter()
    e2e_pass(e2e_steps)
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    if distributed:
        t = torch.tensor([e2e_s], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s = float(t.item())
    e2e_value = FLOP_PER_STEP * world * e2e_steps / e2e_s / 1e12

    if rank == 0:
        peak, peak_sustained, peak_source = measured_peak()
        achieved = FLOP_PER_STEP / (ms_per_step * 1e-3) / 1e12
        line = {
            "metric": METRIC,
            "value": value,
            "unit": "TFLOP/s",
            "n_gpus": world,
            "steps": args.steps,
            "warmup": max(3, args.warmup),
            "ms_per_step": ms_per_step,
            "higher_is_better": True,
            "scaling": "weak",
            "vs_baseline": None,
            "dtype": "bf16 x fp8e5m2 -> fp32 accumulate -> bf16",
            "data": "synthetic",
            "config": {
                "workload": f"scaled_mm bf16@fp8e5m2 M={M} (per GPU) K={K} N={N}, bf16 out, per-tensor scale, no bias",
                "parallelism": f"token shards over {world} GPU(s), replicated prepacked weight, no collective",
                "tile": list(tile),
                "l2": f"{ROTATING_SETS} rotating activation/weight/output sets ({ROTATING_SETS * ALGORITHMIC_BYTES / 1e6:.0f} MB) cycled between steps, larger than the 126 MB L2",
                "value_per_gpu": value / world,
            },
            "roofline": {
                "bound": "tensor",
                "achieved": achieved,
                "peak": peak,
                "unit": "TFLOP/s",
                "frac": achieved / peak,
                "traffic": NCU_DRAM_BYTES_PER_LAUNCH,
                "peak_source": peak_source,
                "kernel": "feather::smm::scaled_mm_pair_kernel<e5m2, bf16 operands, bf16 out> (CTA pairs, 256x256 tiles)",
                "frac_of_nominal_2250": achieved / 2250.0,
                # the timed region is K back-to-back launches: a long one sits between the two measured references
                "timed_region_ms": elapsed_ms,
                "peak_sustained": peak_sustained,
                "frac_of_sustained": None if not peak_sustained else achieved / peak_sustained,
                "algorithmic_bytes": ALGORITHMIC_BYTES,
            },
            "clocks": clocks,
            "e2e": {
                "value": e2e_value,
                "unit": "TFLOP/s",
                "h2d_bytes_per_step": M * K * 2,
                "d2h_bytes_per_step": M * N * 2,
                "steps": e2e_steps,
                "how": "feather_ops_b200.scaled_mm_hip per step; activations copied from pinned host memory and the bf16 result copied back to pinned host memory every step, on copy streams double-buffered against the compute stream; wall clock, max over ranks",
            },
            "gpu_launches": args.steps * world,
        }
        if world == 1:
            line["cpu_baseline"] = cpu_baseline()
        print(json.dumps(line), flush=True)
    if distributed:
        dist.barrier()
        dist.destroy_process_group()


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=500)
    parser.add_argument("--warmup", type=int, default=5)
    parser.add_argument("--impl", choices=("library", "reference"), default="library")
    args = parser.parse_args()
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    if args.impl == "reference":
        run_reference(args)
    else:
        run_library(args)


if __name__ == "__main__":
    main()
