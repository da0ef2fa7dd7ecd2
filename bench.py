"""Benchmark of the hot path: `scaled_mm` bf16 activations x prepacked fp8-e5m2 weights at the
diffusion-transformer MLP-up shape (M=4096 tokens, K=3072, N=12288), bf16 output, fp32 accumulation.

    python bench.py [--gpus N] [--steps K] [--warmup W]            # this library on N GPUs (torchrun for N > 1)
    python bench.py --impl reference [--steps K] [--warmup W]      # the reference's CPU path on the host cores

One step = one pass of the operator over LAUNCHES_PER_STEP token batches of 4096 rows (one launch each), so that
the timed region is long enough for clock samples whatever `--steps` is. With N GPUs every rank owns its own
token shard against replicated weights (the token dimension is the data-parallel one), so there is no collective
on the data path and scaling is weak. Rank 0 prints one JSON line. `value` is the whole-job TFLOP/s with inputs
resident in HBM; `e2e` is the same metric through the public Python API with the activations in pinned host memory
and the result read back to the host every batch (the weights stay resident: they are model state, not step input).

Beside the headline the line carries:
  kernels          (1 GPU) every other benchmark configuration - the CPU-runnable fp16 case, the three transformer
                   shapes, the int8 ConvRot quantizer / GEMM / linear, the three VAE convolutions in both dtypes, the
                   M sweep cold and warm - each with its time (median of rounds of about 50 ms), achieved rate, peak,
                   fraction, vendor-library comparator where one exists, and the reference's CPU callable timed beside it
  strong_m65536    (N GPUs) M = 65536 rows split over the ranks, device-timed and end to end
  n_sharded        (N > 1) the weight split by columns, the output all-gathered with NCCL: blocking, pipelined in row
                   chunks, and in the slab layout without any copy
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
FLOP_PER_LAUNCH = 2 * M * K * N
# A (bf16) + prepacked B (fp8) + C (bf16): the bytes one launch has to move at least once
ALGORITHMIC_BYTES = M * K * 2 + K * N + M * N * 2
ROTATING_SETS = 4  # distinct input/output sets cycled between launches: 4 x 164 MB > the 126 MB L2
NCU_DRAM_BYTES_PER_LAUNCH = 134_200_000
LAUNCHES_PER_STEP = 32
METRIC = "scaled_mm TFLOP/s (bf16@fp8e5m2, 4096x3072x12288)"
WORKLOAD = f"scaled_mm bf16@fp8e5m2 M={M} K={K} N={N}, bf16 out, per-tensor scale, no bias"
STRONG_M = 65536
ROOT = os.path.dirname(os.path.abspath(__file__))


def shared_config(world: int) -> dict:
    """The workload description, identical in the library arm and the reference arm."""
    return {
        "workload": WORKLOAD,
        "batch": f"{M} token rows per launch; a library step is {LAUNCHES_PER_STEP} such batches, a reference (CPU) step is one",
        "parallelism": f"token shards over {world} GPU(s), replicated prepacked weight, no collective on the data path",
        "l2": f"library arm: {ROTATING_SETS} rotating activation/weight/output sets ({ROTATING_SETS * ALGORITHMIC_BYTES / 1e6:.0f} MB > 126 MB L2) cycled between launches; CPU arm: host memory",
    }


def measured_peaks() -> dict:
    """The measured peaks of the device (`MEASURED_PEAKS.json` beside this file: copy bandwidth, cuBLAS bf16 burst and sustained), or the stated fallback."""
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            peaks = json.load(f)
        return {"bf16_tflops": float(peaks["bf16_tflops"]), "bf16_tflops_sustained": float(peaks.get("bf16_tflops_sustained", 0.0)) or None,
                "hbm_gbs": float(peaks["hbm_gbs"]), "source": "measured (MEASURED_PEAKS.json: cuBLAS bf16 burst / sustained, copy bandwidth)"}
    except (OSError, KeyError, ValueError):
        return {"bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "hbm_gbs": 6650.0, "source": "fallback (no MEASURED_PEAKS.json)"}


def make_inputs(seed, m=M, k=K, n=N):
    """Benchmark distribution: A ~ N(0, 1) bf16; W ~ N(0, 0.02) quantized to e5m2 with scale = absmax / 57344, in the
    reference's prepacked layout. Built with the oracle's prepack so that neither arm needs the library for it."""
    from oracle.scaled_mm import prepack_b

    gen = torch.Generator().manual_seed(seed)
    a = torch.randn((m, k), generator=gen, dtype=torch.float32).to(torch.bfloat16)
    w = torch.randn((k, n), generator=gen, dtype=torch.float32) * 0.02
    scale = (w.abs().max() / 57344.0).to(torch.float32)
    b = (w / scale).to(torch.float8_e5m2)
    return a, prepack_b(b), scale


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
                "reasons_mask": hex(mask), "power_w": statistics.median(watts) if watts else None,
                "sm_mhz_samples": clocks[:32], "power_w_samples": watts[:32]}


try:
    ORIGINAL_AFFINITY = os.sched_getaffinity(0)
except AttributeError:
    ORIGINAL_AFFINITY = None


def host_threads() -> int:
    """torchrun exports OMP_NUM_THREADS=1, and the library arm may have moved this rank next to its GPU: the CPU legs
    take every core this process was started on, with the default memory policy."""
    cores = os.cpu_count() or 1
    if ORIGINAL_AFFINITY is not None:
        try:
            os.sched_setaffinity(0, ORIGINAL_AFFINITY)
            import ctypes
            import platform

            if platform.machine() == "x86_64":
                ctypes.CDLL(None, use_errno=True).syscall(238, 0, None, 0)   # set_mempolicy(MPOL_DEFAULT)
        except OSError:
            pass
        cores = len(os.sched_getaffinity(0))
    torch.set_num_threads(max(1, cores))
    return torch.get_num_threads()


def _best_of(fn, repeats=3, budget_s=8.0):
    """Best wall-clock seconds of `fn()` over up to `repeats` runs after one warm-up, stopping early when the budget is spent."""
    fn()
    best, spent = float("inf"), 0.0
    for _ in range(repeats):
        t0 = time.perf_counter()
        fn()
        dt = time.perf_counter() - t0
        best, spent = min(best, dt), spent + dt
        if spent > budget_s:
            break
    return best


# ---------------------------------------------------------------------------------------------------------------
# CPU baselines: the reference's CPU-runnable callables (restated in oracle/), timed on the host cores
# ---------------------------------------------------------------------------------------------------------------
def cpu_baseline_headline() -> dict:
    """The reference's naive path (`feather_ops/naive.py`, restated in oracle/scaled_mm.py) on the whole benchmark batch."""
    from oracle import scaled_mm as osm

    cores = host_threads()
    a, packed, scale = make_inputs(0)
    best = _best_of(lambda: osm.scaled_mm_naive(a, packed, scale, None, torch.bfloat16, b_prepacked=True))
    return {"value": FLOP_PER_LAUNCH / best / 1e12, "unit": "TFLOP/s", "cores": cores, "kind": "port",
            "sample": f"all {M} token rows x full {K}x{N} weight, best of 3, torch CPU fp16 matmul as in the reference's naive path", "ms": best * 1e3}


def cpu_baselines_for_cases() -> dict:
    """`{case key prefix: cpu_baseline object}` for every entry of the `kernels` list: the callable the reference's
    own tests and CPU path use for that configuration, on bounded samples where the full problem would take too long."""
    import torch.nn.functional as F

    from oracle import int8_convrot as o8
    from oracle import scaled_mm as osm

    cores = host_threads()
    out = {}

    def naive(m, n, k, dtype, rows=None):
        gen = torch.Generator().manual_seed(m + n + k)
        sample = m if rows is None else min(m, rows)
        a = torch.randn((sample, k), generator=gen).to(dtype)
        b = osm.prepack_b((torch.randn((k, n), generator=gen) * 8).to(torch.float8_e5m2))
        scale = torch.tensor(0.01)
        best = _best_of(lambda: osm.scaled_mm_naive(a, b, scale, None, dtype, b_prepacked=True))
        return {"value": 2.0 * sample * n * k / best / 1e12, "unit": "TFLOP/s", "ms": best * 1e3, "cores": cores, "kind": "port",
                "sample": ("all" if sample == m else f"first {sample} of") + f" {m} rows, scaled_mm_naive (feather_ops/naive.py:4-41), best of 3"}

    out["cfg1 scaled_mm"] = naive(256, 4096, 4096, torch.float16)
    for n, k in ((12288, 3072), (3072, 12288), (9216, 3072)):
        out[f"cfg2 scaled_mm bf16 4096x{n}x{k}"] = naive(4096, n, k, torch.bfloat16)
    for m in (1, 16, 128, 1024, 8192):
        out[f"cfg5 scaled_mm M-sweep M={m} "] = naive(m, 12288, 3072, torch.bfloat16)
    out["cfg5 scaled_mm M-sweep M=65536"] = naive(65536, 12288, 3072, torch.bfloat16, rows=8192)

    # cfg3: the matmul-rotation + row-wise int8 recipe, then a float matmul of the codes with both scales
    m, k, n = 4096, 3072, 3072
    x = o8.make_activation(m, k, torch.bfloat16)
    w = o8.make_weight(n, k, torch.bfloat16)
    wq, ws = o8.quantize_convrot_weight(w)
    hadamard = o8.build_hadamard(256)
    best_q = _best_of(lambda: o8.quantize_rowwise_int8(o8.rotate(x, hadamard)))
    q, s = o8.quantize_rowwise_int8(o8.rotate(x, hadamard))
    out["cfg3 convrot_quantize"] = {"value": (m * k * 3 + m * 4) / best_q / 1e9, "unit": "GB/s", "ms": best_q * 1e3, "cores": cores, "kind": "port",
                                    "sample": "all 4096 rows: rotate (bf16 matmul with the 256x256 Hadamard) + quantize_rowwise_int8 (feather_ops/int8_convrot.py:255-282)"}
    wq_f = wq.float()

    def gemm_stand_in():
        return ((q.float() @ wq_f.T) * s[:, None] * ws[None, :]).to(torch.bfloat16)

    best_g = _best_of(gemm_stand_in)
    stand_in = {"value": 2.0 * m * n * k / best_g / 1e12, "unit": "TOP/s", "ms": best_g * 1e3, "cores": cores, "kind": "port",
                "sample": "all 4096 rows: fp32 matmul of the int8 codes with both scales (the dequantized product of tests/test_int8_convrot.py:52-57)"}
    out["cfg3 int8_scaled_mm"] = stand_in
    out["cfg3 convrot_int8_linear"] = {**stand_in, "value": 2.0 * m * n * k / (best_g + best_q) / 1e12, "ms": (best_g + best_q) * 1e3,
                                       "sample": "recipe quantizer + fp32 matmul of the codes, all 4096 rows"}
    out["int8_scaled_mm 8192x8192x8192"] = {**stand_in, "sample": "rate of the 4096x3072x3072 stand-in (the 8192^3 product is not run on the host)"}
    out["int8_scaled_mm_plain 8192x8192x8192"] = out["int8_scaled_mm 8192x8192x8192"]

    for channels, size in ((512, 128), (256, 256), (128, 512)):
        for dtype in (torch.bfloat16, torch.float16):
            gen = torch.Generator().manual_seed(channels)
            xc = torch.randn((1, channels, size, size), generator=gen).to(dtype)
            wc = (torch.randn((channels, channels, 3, 3), generator=gen) / (9 * channels) ** 0.5).to(dtype)
            bc = (torch.randn(channels, generator=gen) * 0.01).to(dtype)
            with torch.no_grad():
                best = _best_of(lambda: F.conv2d(xc, wc, bc, 1, 1), repeats=3, budget_s=6.0)
            out[f"cfg4 conv3x3 {channels}->{channels} @{size}x{size} {str(dtype).replace('torch.', '')}"] = {
                "value": 2.0 * channels * channels * 9 * size * size / best / 1e12, "unit": "TFLOP/s", "ms": best * 1e3, "cores": cores, "kind": "port",
                "sample": "the whole image, torch.nn.functional.conv2d in the tensor dtype on the host cores"}
    return out


def attach_cpu_baselines(records: list, baselines: dict) -> None:
    for record in records:
        for prefix, baseline in baselines.items():
            if record["case"].startswith(prefix):
                record["cpu_baseline"] = baseline
                break


# ---------------------------------------------------------------------------------------------------------------
# reference arm
# ---------------------------------------------------------------------------------------------------------------
def run_reference(args):
    """`--impl reference`: the reference's own CPU implementation of the path (no GPU, rank 0 only). Nothing of the
    library is imported here: the inputs are built with the oracle's prepack."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import scaled_mm as osm

    cores = host_threads()
    a, packed, scale = make_inputs(0)
    for _ in range(max(1, min(args.warmup, 2))):
        osm.scaled_mm_naive(a, packed, scale, None, torch.bfloat16, b_prepacked=True)
    steps = max(1, args.steps)
    t0 = time.perf_counter()
    for _ in range(steps):
        osm.scaled_mm_naive(a, packed, scale, None, torch.bfloat16, b_prepacked=True)
    elapsed = time.perf_counter() - t0
    value = FLOP_PER_LAUNCH * steps / elapsed / 1e12
    sample = f"each step = one whole batch (all {M} token rows x full weight) on the host cores: the oracle port of feather_ops/naive.py (torch CPU fp16 matmul)"
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
        "config": shared_config(args.gpus),
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------------------------
# library arm
# ---------------------------------------------------------------------------------------------------------------
def numa_local_setup(device_index: int) -> dict:
    """Before any pinned memory is allocated: run this rank on the CPUs next to its GPU (where the process is allowed
    to) and prefer that NUMA node for its pages, so that the pinned staging buffers of eight ranks do not all land on
    one memory controller. Returns what was found and done, for the JSON line."""
    info = {"numa_node": None, "cpus_local": None, "affinity_set": False, "mempolicy_set": False}
    try:
        props = torch.cuda.get_device_properties(device_index)
        bdf = f"{props.pci_domain_id:04x}:{props.pci_bus_id:02x}:{props.pci_device_id:02x}.0"
        base = f"/sys/bus/pci/devices/{bdf}"
        with open(f"{base}/numa_node") as f:
            node = int(f.read().strip())
        with open(f"{base}/local_cpulist") as f:
            text = f.read().strip()
        info["numa_node"], info["cpus_local"] = node, text
        local = set()
        for part in text.split(","):
            if "-" in part:
                lo, hi = part.split("-")
                local.update(range(int(lo), int(hi) + 1))
            elif part:
                local.add(int(part))
        allowed = os.sched_getaffinity(0)
        pick = allowed & local
        if pick and pick != allowed:
            os.sched_setaffinity(0, pick)
            info["affinity_set"] = True
        info["cpus_allowed"] = len(allowed)
        import platform

        if node >= 0 and platform.machine() == "x86_64":   # the system-call number below is the x86-64 one
            import ctypes

            libc = ctypes.CDLL(None, use_errno=True)
            mask = ctypes.c_ulong(1 << node)
            # set_mempolicy(MPOL_PREFERRED = 1, nodemask, maxnode): pages of later allocations come from the GPU's node when it has room
            if libc.syscall(238, 1, ctypes.byref(mask), 64) == 0:
                info["mempolicy_set"] = True
    except Exception as exc:  # noqa: BLE001 - a container may hide sysfs or forbid the calls: the bench goes on without
        info["error"] = f"{type(exc).__name__}: {exc}"[:120]
    return info


def copy_bandwidth(device, m, n, k, iters=6) -> dict:
    """GB/s of this rank's host <-> device copies alone (pinned buffers of the step's sizes): H2D of the activations, D2H of
    the result, and both at once on two streams. Wall clock around stream synchronization."""
    a_host = torch.empty((m, k), dtype=torch.bfloat16).pin_memory()
    c_host = torch.empty((m, n), dtype=torch.bfloat16).pin_memory()
    a_dev = torch.empty((m, k), device=device, dtype=torch.bfloat16)
    c_dev = torch.empty((m, n), device=device, dtype=torch.bfloat16)
    s_in, s_out = torch.cuda.Stream(device), torch.cuda.Stream(device)

    def h2d():
        with torch.cuda.stream(s_in):
            a_dev.copy_(a_host, non_blocking=True)

    def d2h():
        with torch.cuda.stream(s_out):
            c_host.copy_(c_dev, non_blocking=True)

    def timed(fns, nbytes):
        for fn in fns:
            fn()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(iters):
            for fn in fns:
                fn()
        torch.cuda.synchronize()
        return nbytes * iters / (time.perf_counter() - t0) / 1e9

    return {"h2d": timed([h2d], a_host.numel() * 2), "d2h": timed([d2h], c_host.numel() * 2), "both": timed([h2d, d2h], (a_host.numel() + c_host.numel()) * 2)}


def run_library(args):
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the kernels have no CPU fallback")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    numa = numa_local_setup(local_rank)
    distributed = world > 1
    dist = None
    if distributed:
        import torch.distributed as dist

        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=device)

    import feather_ops_b200 as fo
    from feather_ops_b200 import benchmarks, shard
    from feather_ops_b200.scaled_mm import _scaled_mm_auto, select_scaled_mm_config

    def barrier():
        if distributed:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(value: float) -> float:
        if not distributed:
            return value
        t = torch.tensor([value], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def gather_over_ranks(value: float) -> list:
        if not distributed:
            return [value]
        t = torch.tensor([value], device=device, dtype=torch.float64)
        every = [torch.empty_like(t) for _ in range(world)]
        dist.all_gather(every, t)
        return [float(x.item()) for x in every]

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

    def launch(i):
        a, b = sets[i % ROTATING_SETS]
        torch.ops.feather_ops.scaled_mm.default(a, b, scale, None, outs[i % ROTATING_SETS], *tile[:5], bool(tile[5]))

    def step():
        for i in range(LAUNCHES_PER_STEP):
            launch(i)

    # the clock sampler is started before the warm-up so that it is already producing samples when the timed region
    # begins; only the samples time-stamped inside the timed region are kept
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    warmup = max(3, args.warmup)
    for _ in range(warmup):
        step()
    barrier()
    marks = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps + 1)]
    barrier()
    region_begin = datetime.datetime.now()
    marks[0].record()
    for s in range(args.steps):
        step()
        marks[s + 1].record()
    barrier()
    region_end = datetime.datetime.now()
    elapsed_ms = marks[0].elapsed_time(marks[-1])
    step_ms = [marks[s].elapsed_time(marks[s + 1]) for s in range(args.steps)]
    clocks = sampler.stop((region_begin, region_end)) if rank == 0 else None
    if clocks is not None:
        clocks["note"] = "nvidia-smi samples every 20 ms, time-stamped inside the timed region"
    elapsed_ms = max_over_ranks(elapsed_ms)
    ms_per_step = elapsed_ms / args.steps
    value = FLOP_PER_LAUNCH * LAUNCHES_PER_STEP * world / (ms_per_step * 1e-3) / 1e12
    fastest_step_ms = max_over_ranks(min(step_ms))

    # ------------------------------------------------------------------ end to end: host buffers, public API
    # every rank with all ranks copying at once (what the end-to-end loop meets), then every rank in turn with the others idle
    # (what one GPU's link gives): the gap between the two is the share of the host side (root complex, memory) in the limit
    barrier()
    copy_gbs = copy_bandwidth(device, M, N, K)
    copy_gbs_per_rank = {key: [round(v, 1) for v in gather_over_ranks(val)] for key, val in copy_gbs.items()}
    copy_gbs_alone = copy_gbs
    if distributed:
        for turn in range(world):
            barrier()
            if turn == rank:
                copy_gbs_alone = copy_bandwidth(device, M, N, K)
        barrier()
    copy_gbs_per_rank_alone = {key: [round(v, 1) for v in gather_over_ranks(val)] for key, val in copy_gbs_alone.items()}

    def e2e_run(m_rows, batches, a_rows_host):
        """`batches` passes of `fo.scaled_mm_hip` over `m_rows` host rows each: H2D of the activations, the product,
        D2H of the result, double-buffered on copy streams. Returns wall seconds (max over ranks)."""
        a_pinned = [a_rows_host.roll(i, 0).pin_memory() for i in range(2)]
        c_pinned = [torch.empty((m_rows, N), dtype=torch.bfloat16).pin_memory() for _ in range(2)]
        a_dev = [torch.empty((m_rows, K), device=device, dtype=torch.bfloat16) for _ in range(2)]
        copy_in, copy_out = torch.cuda.Stream(device), torch.cuda.Stream(device)
        compute = torch.cuda.current_stream(device)
        in_done = [torch.cuda.Event() for _ in range(2)]
        mm_done = [torch.cuda.Event() for _ in range(2)]
        out_done = [torch.cuda.Event() for _ in range(2)]
        c_dev = [None, None]

        def run(count):
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

        run(2)
        barrier()
        t0 = time.perf_counter()
        run(batches)
        torch.cuda.synchronize()
        return max_over_ranks(time.perf_counter() - t0)

    e2e_batches = max(4, min(args.steps * LAUNCHES_PER_STEP, 24))
    e2e_s = e2e_run(M, e2e_batches, a_host)
    e2e_value = FLOP_PER_LAUNCH * world * e2e_batches / e2e_s / 1e12
    # a batch moves its activations in and its result out; `both` is the rate with the two directions in flight together
    d2h_floor_ms = (M * K * 2 + M * N * 2) / (min(copy_gbs_per_rank["both"]) * 1e9) * 1e3 if min(copy_gbs_per_rank["both"]) > 0 else None

    # ------------------------------------------------------------------ strong scaling: M = 65536 split over the ranks
    start_row, stop_row = shard.token_shard(STRONG_M, rank, world)
    rows = stop_row - start_row
    gen = torch.Generator(device=device).manual_seed(1000 + rank)
    a_strong = torch.randn((rows, K), device=device, generator=gen).to(torch.bfloat16)
    c_strong = torch.empty((rows, N), device=device, dtype=torch.bfloat16)
    strong_iters = 6
    for _ in range(2):
        _scaled_mm_auto(a_strong, packed, scale, None, c_strong)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(strong_iters):
        _scaled_mm_auto(a_strong, packed, scale, None, c_strong)
    e1.record()
    barrier()
    strong_ms = max_over_ranks(e0.elapsed_time(e1) / strong_iters)
    strong = {
        "workload": f"scaled_mm bf16@fp8e5m2 M={STRONG_M} rows in total, split with shard.token_shard ({rows} rows on rank 0), K={K} N={N}, replicated weight",
        "scaling": "strong",
        "ms": strong_ms,
        "tflops": 2.0 * STRONG_M * N * K / (strong_ms * 1e-3) / 1e12,
        "timing": f"CUDA events around {strong_iters} back-to-back launches after 2 warm-up launches, max over ranks; activations ({rows * K * 2 / 1e6:.0f} MB) + output ({rows * N * 2 / 1e6:.0f} MB) per rank exceed the L2",
    }
    del c_strong
    strong_e2e_s = e2e_run(rows, 3, a_strong.cpu())
    strong["e2e_tflops"] = 2.0 * STRONG_M * N * K * 3 / strong_e2e_s / 1e12
    strong["e2e_ms"] = strong_e2e_s / 3 * 1e3
    strong["e2e_how"] = "3 passes over this rank's rows through feather_ops_b200.scaled_mm_hip with pinned host activations and the result copied back, wall clock, max over ranks"
    del a_strong

    # ------------------------------------------------------------------ N-sharded variant with the NCCL all-gather
    n_sharded = None
    if distributed and N % world == 0 and (N // world) % 16 == 0:
        n_sharded = bench_n_sharded(device, dist, shard, packed, scale, rank, world, max_over_ranks, barrier)

    if rank == 0:
        peaks = measured_peaks()
        achieved = FLOP_PER_LAUNCH * LAUNCHES_PER_STEP / (ms_per_step * 1e-3) / 1e12
        burst = FLOP_PER_LAUNCH * LAUNCHES_PER_STEP / (fastest_step_ms * 1e-3) / 1e12
        line = {
            "metric": METRIC,
            "value": value,
            "unit": "TFLOP/s",
            "n_gpus": world,
            "steps": args.steps,
            "warmup": warmup,
            "ms_per_step": ms_per_step,
            "higher_is_better": True,
            "scaling": "weak",
            "vs_baseline": None,
            "dtype": "bf16 x fp8e5m2 -> fp32 accumulate -> bf16",
            "data": "synthetic",
            "config": shared_config(world),
            "launches_per_step": LAUNCHES_PER_STEP,
            "us_per_launch": ms_per_step * 1e3 / LAUNCHES_PER_STEP,
            "value_per_gpu": value / world,
            "tile": list(tile),
            "roofline": {
                "bound": "tensor",
                "achieved": achieved,
                "peak": peaks["bf16_tflops"],
                "unit": "TFLOP/s",
                "frac": achieved / peaks["bf16_tflops"],
                # dram__bytes_read.sum + dram__bytes_write.sum per launch from an ncu capture of this kernel at this shape (launches
                # 3 and 4 of a loop over the same four rotating buffer sets: 64.24 MB read + 61.07 / 63.67 MB written). Reads are the algorithmic A + B; the writes fall short of the
                # 100.7 MB of C because the profiler flushes the L2 before the captured launch and part of C is still dirty
                # in L2 when it ends. In the back-to-back timed region those lines are written back during the next launch, so
                # the steady-state traffic is at least the algorithmic bytes.
                "traffic": NCU_DRAM_BYTES_PER_LAUNCH,
                "traffic_note": "ncu capture with the bench's buffer rotation; the L2 is flushed before and part of C still dirty in L2 after the captured launch, steady state >= algorithmic_bytes",
                "peak_source": peaks["source"],
                "kernel": "feather::smm::scaled_mm_pair_kernel<e5m2, bf16 operands, bf16 out> (CTA pairs, 256x256 tiles)",
                "frac_of_nominal_2250": achieved / 2250.0,
                "timed_region_ms": elapsed_ms,
                "fastest_step_tflops": burst,
                "fastest_step_frac": burst / peaks["bf16_tflops"],
                "peak_sustained": peaks["bf16_tflops_sustained"],
                "frac_of_sustained": None if not peaks["bf16_tflops_sustained"] else achieved / peaks["bf16_tflops_sustained"],
                "algorithmic_bytes": ALGORITHMIC_BYTES,
                "algorithmic_gbs": ALGORITHMIC_BYTES * LAUNCHES_PER_STEP / (ms_per_step * 1e-3) / 1e9,
            },
            "clocks": clocks,
            "e2e": {
                "value": e2e_value,
                "unit": "TFLOP/s",
                "h2d_bytes_per_step": M * K * 2 * LAUNCHES_PER_STEP,
                "d2h_bytes_per_step": M * N * 2 * LAUNCHES_PER_STEP,
                "batches_timed": e2e_batches,
                "ms_per_batch": e2e_s / e2e_batches * 1e3,
                "copy_gbs_per_rank": copy_gbs_per_rank,
                "copy_gbs_per_rank_alone": copy_gbs_per_rank_alone,
                "copy_gbs_all_ranks_together": round(sum(copy_gbs_per_rank["both"]), 1),
                "copy_floor_ms_per_batch": d2h_floor_ms,
                "limiter": "the device -> host copy of the 100.7 MB result per batch: ms_per_batch follows the copy floor (both directions in flight, all ranks copying at once: copy_gbs_per_rank; copy_gbs_per_rank_alone is each rank with the others idle), the product itself takes us_per_launch",
                "numa": numa,
                "how": "feather_ops_b200.scaled_mm_hip per batch; activations copied from pinned host memory and the bf16 result copied back to pinned host memory every batch, on copy streams double-buffered against the compute stream; wall clock, max over ranks",
            },
            "strong_m65536": strong,
            "n_sharded": n_sharded,
            "gpu_launches": args.steps * LAUNCHES_PER_STEP * world,
        }
        if world == 1:
            line["cpu_baseline"] = cpu_baseline_headline()
            if not args.skip_kernels:
                bench_peaks = {"bf16_tflops": peaks["bf16_tflops"], "hbm_gbs": peaks["hbm_gbs"]}
                benchmarks.set_device_limits(device)
                records = benchmarks.bench_scaled_mm(device, bench_peaks)
                records += benchmarks.bench_msweep(device, bench_peaks, include_65536=False)   # M = 65536 is the strong_m65536 object
                records += benchmarks.bench_int8(device, bench_peaks)
                records += benchmarks.bench_conv(device, bench_peaks)
                torch.cuda.empty_cache()
                attach_cpu_baselines(records, cpu_baselines_for_cases())
                line["kernels"] = records
                line["kernels_protocol"] = "each case: warm-up, then 5 rounds of back-to-back launches (CUDA-graph replays) sized to about 50 ms inside one CUDA-event pair; us = median of the rounds; cold = rotating buffer sets larger than twice the L2"
        print(json.dumps(line), flush=True)
    if distributed:
        dist.barrier()
        dist.destroy_process_group()


def bench_n_sharded(device, dist, shard, packed, scale, rank, world, max_over_ranks, barrier) -> dict:
    """M = 65536 rows on every rank against this rank's column slab of the weight, the output all-gathered with NCCL.
    Times the parts alone (product, all-gather, permute copy) and the variants of `shard.scaled_mm_n_sharded`."""
    m = STRONG_M
    slab, _ = shard.weight_column_shard(packed, rank, world)
    width = slab.shape[1]
    gen = torch.Generator(device=device).manual_seed(7)   # the same activations on every rank
    a = torch.randn((m, K), device=device, generator=gen).to(torch.bfloat16)
    iters = 3

    def timed(fn):
        fn()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        barrier()
        return max_over_ranks(e0.elapsed_time(e1) / iters)

    local = torch.empty((m, width), device=device, dtype=torch.bfloat16)
    gathered = torch.empty((world * m, width), device=device, dtype=torch.bfloat16)
    row_major = torch.empty((m, world * width), device=device, dtype=torch.bfloat16)
    product_ms = timed(lambda: shard._kernel_into(a, slab, scale, None, local))
    gather_ms = timed(lambda: dist.all_gather_into_tensor(gathered, local))
    permute_ms = timed(lambda: shard._interleave(gathered.view(world, m, width), row_major))
    del local, gathered, row_major
    torch.cuda.empty_cache()
    variants = {}
    cases = [("blocking_row_major", {}), ("slabs_in_place", {"layout": "slabs"})]
    for chunks in (4, 8, 16):
        for margin in (0, 16, 32, 48):
            cases.append((f"pipelined_row_major_{chunks}_chunks_sm_margin_{margin}", {"chunks": chunks, "sm_margin": margin}))
    for margin in (0, 32):
        cases.append((f"slabs_pipelined_8_chunks_sm_margin_{margin}", {"layout": "slabs", "chunks": 8, "sm_margin": margin}))
    for name, kwargs in cases:
        variants[name] = timed(lambda kw=kwargs: shard.scaled_mm_n_sharded(a, slab, scale, None, torch.bfloat16, **kw))
        torch.cuda.empty_cache()
    received = (world - 1) * m * width * 2
    serial = product_ms + gather_ms + permute_ms
    best_name = min((name for name in variants if name.startswith("pipelined_row_major")), key=variants.get)
    best_row_major = variants[best_name]
    hideable = product_ms + permute_ms
    return {
        "workload": f"scaled_mm bf16@fp8e5m2 M={m} on every rank, K={K}, N={N} split into {world} column slabs of {width}; output all-gathered with NCCL",
        "product_ms": product_ms,
        "all_gather_ms": gather_ms,
        "permute_copy_ms": permute_ms,
        "all_gather_received_gb_per_gpu": received / 1e9,
        "all_gather_bus_gbs": received / (gather_ms * 1e-3) / 1e9,
        "variants_ms": variants,
        "serial_sum_ms": serial,
        "best_pipelined_row_major": best_name,
        "overlap_fraction_row_major": None if hideable <= 0 else max(0.0, min(1.0, (serial - best_row_major) / hideable)),
        "overlap_fraction_is": "(product + all-gather + interleave copy, each timed alone, minus the best pipelined time) / (product + interleave copy): the share of the non-collective work hidden behind the all-gather",
        "limiter": "the all-gather: every GPU receives (world - 1) / world of the output over NVLink, several times longer than its share of the product; the pipeline hides the product and the copies behind it",
        "timing": f"CUDA events around {iters} calls after one warm-up call, max over ranks",
    }


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=20)
    parser.add_argument("--warmup", type=int, default=5)
    parser.add_argument("--impl", choices=("library", "reference"), default="library")
    parser.add_argument("--skip-kernels", action="store_true", help="leave the per-configuration `kernels` list out (1 GPU only)")
    args = parser.parse_args()
    if ROOT not in sys.path:
        sys.path.insert(0, ROOT)
    if args.impl == "reference":
        run_reference(args)
    else:
        run_library(args)


if __name__ == "__main__":
    main()
