"""Per-operator measurements: every operator of the library at its benchmark shapes, with vendor-library comparators.

    python -m feather_ops_b200.benchmarks [scaled_mm] [msweep] [int8] [conv] [grid] [cells] [--profile] [--peaks FILE]

`--peaks FILE` names a JSON file with the measured peaks of the device (`hbm_gbs`, `bf16_tflops`); without it only
the fractions of the nominal peaks are reported. `--profile` is for runs under a profiler: every case makes three
plain launches (no CUDA graph, no timing), so a capture of one kernel stays a handful of launches.

Protocol (after the reference's bench/protocol.py:86-175): warm-up, then at least five rounds of back-to-back
launches inside one CUDA-event pair, each round sized to about 50 ms, median and p20 / p80 over the rounds. The
launches of a round are replayed from a CUDA graph so that kernels of a few microseconds are not timed as Python
call overhead. Inputs rotate over enough distinct buffer sets to exceed the L2 ("cold") unless a case says warm.
Every case is a dict; `main` prints one JSON object per case, `bench.py` collects them into its `kernels` list.
"""

import json
import statistics
import sys

import torch

L2_BYTES = 126 * 1024 * 1024   # replaced by the device's own figure in `main` / `set_device_limits`
NOMINAL = {"bf16_tflops": 2250.0, "int8_tops": 4500.0, "hbm_gbs": 8000.0}   # B200 dense peaks
ROUND_MS = 50.0
ROUNDS = 5
GRAPH_LAUNCHES_MAX = 256

PROFILE_MODE = False


def _percentile(samples, q):
    ordered = sorted(samples)
    pos = q * (len(ordered) - 1)
    lo = int(pos)
    hi = min(lo + 1, len(ordered) - 1)
    return ordered[lo] + (ordered[hi] - ordered[lo]) * (pos - lo)


def wait_records() -> dict:
    """The records of the kernels' bounded waits that are not `(0, 0)`: `{}` in a healthy run. A wait that ran out costs
    seconds, so a time measured over it is not a kernel time; every timed case carries this beside its number."""
    from . import _lib

    found = {}
    for symbol in ("feather_scaled_mm_status", "feather_int8_mm_status", "feather_conv3x3_status"):
        site, block = _lib.read_status(symbol)
        if site or block:
            found[symbol] = [site, block]
    return found


def time_launches(launch, sets: int, rounds: int = ROUNDS, round_ms: float = ROUND_MS) -> dict:
    """`{"us": median, "p20_us", "p80_us", "launches_per_round", "rounds"}` for `launch(i)`, which enqueues one launch
    on buffer set `i % sets`. A round replays a CUDA graph of up to GRAPH_LAUNCHES_MAX launches (a multiple of `sets`)
    as often as it takes to fill `round_ms`."""
    if PROFILE_MODE:
        for i in range(3):
            launch(i)
        torch.cuda.synchronize()
        return {"us": None, "p20_us": None, "p80_us": None, "launches_per_round": 3, "rounds": 0}
    for i in range(max(3, sets)):
        launch(i)
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for i in range(sets):
        launch(i)
    stop.record()
    torch.cuda.synchronize()
    estimate_ms = max(start.elapsed_time(stop) / sets, 1e-3)
    per_graph = int(min(GRAPH_LAUNCHES_MAX, max(1.0, round_ms / estimate_ms)))
    per_graph = max(sets, per_graph // sets * sets)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for i in range(per_graph):
            launch(i)
    graph.replay()
    torch.cuda.synchronize()
    start.record()
    graph.replay()
    stop.record()
    torch.cuda.synchronize()
    replays = int(max(1.0, round(round_ms / max(start.elapsed_time(stop), 1e-3))))
    samples = []
    for _ in range(rounds):
        start.record()
        for _ in range(replays):
            graph.replay()
        stop.record()
        torch.cuda.synchronize()
        samples.append(start.elapsed_time(stop) * 1e3 / (per_graph * replays))
    return {"us": statistics.median(samples), "p20_us": _percentile(samples, 0.2), "p80_us": _percentile(samples, 0.8),
            "launches_per_round": per_graph * replays, "rounds": rounds, "wait_status": wait_records()}


def set_device_limits(device) -> None:
    """Take the L2 size from the device, so that "cold" means larger than twice THIS part's L2."""
    global L2_BYTES
    size = getattr(torch.cuda.get_device_properties(device), "L2_cache_size", 0)
    if size:
        L2_BYTES = int(size)


def sets_for(bytes_per_set: int, cold: bool, cap: int = 8) -> int:
    """Buffer sets to rotate over: enough to exceed twice the L2 when cold, one when warm."""
    return min(cap, max(2, -(-2 * L2_BYTES // max(bytes_per_set, 1)))) if cold else 1


def _round(value, digits=3):
    return None if value is None else round(value, digits)


def _rates(record: dict, timing: dict, *, flop: float | None, algorithmic_bytes: float | None, bound: str, peaks: dict, int8: bool = False) -> dict:
    """Fill in time, achieved rate, peak and fractions. `bound` is "tensor" (rate = flop / time against the tensor peak)
    or "hbm" (rate = algorithmic bytes / time against the copy bandwidth)."""
    us = timing["us"]
    record.update(us=_round(us, 2), p20_us=_round(timing["p20_us"], 2), p80_us=_round(timing["p80_us"], 2), launches_per_round=timing["launches_per_round"],
                  rounds=timing["rounds"], bound=bound, flop=flop, algorithmic_bytes=algorithmic_bytes)
    if timing.get("wait_status"):
        record["wait_status"] = timing["wait_status"]
    if us is None:
        return record
    if flop is not None:
        record["tops" if int8 else "tflops"] = _round(flop / us / 1e6, 1)
    if algorithmic_bytes is not None:
        record["gbs"] = _round(algorithmic_bytes / us / 1e3, 1)
    if bound == "tensor":
        achieved = flop / us / 1e6
        nominal = NOMINAL["int8_tops" if int8 else "bf16_tflops"]
        measured = peaks.get("int8_tops") if int8 else peaks.get("bf16_tflops")
        unit = "TOP/s" if int8 else "TFLOP/s"
    else:
        achieved = algorithmic_bytes / us / 1e3
        nominal = NOMINAL["hbm_gbs"]
        measured = peaks.get("hbm_gbs")
        unit = "GB/s"
    record.update(achieved=_round(achieved, 1), unit=unit, peak=measured, frac=None if not measured else _round(achieved / measured),
                  peak_nominal=nominal, frac_of_nominal=_round(achieved / nominal))
    return record


# ------------------------------------------------------------------------------------------------------------- scaled_mm
def _scaled_mm_path(m, n, k):
    """What the public path runs for this shape, as a label."""
    from . import scaled_mm as smm

    if m <= 128 and smm.warp_mma_takes(m, n, k):
        return "vector kernel" if m <= 2 and n >= 64 * smm.sm_count() else "warp-MMA kernel"
    if smm.select_pair_splits(m, n, k) > 1:
        return f"CTA-pair kernel, 256x256 tiles, {smm.select_pair_splits(m, n, k)} K splits"
    if smm.select_row_tile_splits_256(m, n, k) > 1:
        return f"one-CTA kernel, 128x256 tiles, {smm.select_row_tile_splits_256(m, n, k)} K splits"
    splits = smm.select_wide_splits(m, n, k)
    if splits > 1:
        return f"one-CTA kernel, 128x128 tiles, {splits} K splits"
    if 64 < m <= 128 and -(-n // 128) >= smm.sm_count() // 2:
        return "one-CTA kernel, 128x128 tiles"
    if m <= 128:
        return f"skinny tcgen05 kernel, {smm.select_scaled_mm_splits(m, n, k)} K splits"
    width = 16 * smm.select_scaled_mm_config(m, n, k)[1] * smm.select_scaled_mm_config(m, n, k)[4]
    if width >= 256:
        from . import _lib

        columns = _lib.load().feather_scaled_mm_pair_tile_width(m, n, smm.sm_count() // 2)   # the launcher narrows the tile where that fills a round
        return f"CTA-pair kernel, 256x{columns} tiles"
    return f"one-CTA kernel, 128x{width} tiles"


def scaled_mm_case(key, m, n, k, a_dtype, out_dtype, cold, device, peaks, bound=None) -> dict:
    from . import scaled_mm as smm

    algorithmic = m * k * 2 + k * n + m * n * 2
    sets = sets_for(algorithmic, cold)
    gen = torch.Generator(device=device).manual_seed(m + n + k)
    weights = (torch.randn((k, n), device=device, generator=gen) * 8).to(torch.float8_e5m2)
    packed = [smm.prepack_b_for_scaled_mm(weights)]
    del weights
    packed += [packed[0].clone() for _ in range(sets - 1)]
    acts = [torch.randn((m, k), device=device, generator=gen).to(a_dtype) for _ in range(sets)]
    outs = [torch.empty((m, n), device=device, dtype=out_dtype) for _ in range(sets)]
    scale = torch.tensor(0.01, device=device)

    def launch(i):
        j = i % sets
        smm._scaled_mm_auto(acts[j], packed[j], scale, None, outs[j])  # the public path: tile and split heuristics included

    timing = time_launches(launch, sets)
    if bound is None:
        bound = "hbm" if m <= 128 else "tensor"
    record = {"case": key, "op": "scaled_mm", "M": m, "N": n, "K": k, "dtype": str(a_dtype).replace("torch.", "") + " x e5m2", "cold": cold,
              "buffer_sets": sets, "path": _scaled_mm_path(m, n, k)}
    return _rates(record, timing, flop=2.0 * m * n * k, algorithmic_bytes=float(algorithmic), bound=bound, peaks=peaks)


def library_bf16_gemm_case(m, n, k, device, peaks) -> dict:
    """The vendor library's plain bf16 GEMM (both operands already bf16: no fp8 decode, no scale) with the same buffer rotation:
    the measured tensor-core denominator at exactly this shape."""
    sets = sets_for(m * k * 2 + k * n * 2 + m * n * 2, True)
    acts = [torch.randn((m, k), device=device).to(torch.bfloat16) for _ in range(sets)]
    weights = [torch.randn((k, n), device=device).to(torch.bfloat16) for _ in range(sets)]
    outs = [torch.empty((m, n), device=device, dtype=torch.bfloat16) for _ in range(sets)]
    timing = time_launches(lambda i: torch.matmul(acts[i % sets], weights[i % sets], out=outs[i % sets]), sets)
    record = {"case": f"vendor bf16 GEMM {m}x{n}x{k} (torch.matmul)", "op": "vendor_gemm", "M": m, "N": n, "K": k, "cold": True, "buffer_sets": sets}
    return _rates(record, timing, flop=2.0 * m * n * k, algorithmic_bytes=None, bound="tensor", peaks=peaks)


def bench_scaled_mm(device, peaks) -> list[dict]:
    out = [scaled_mm_case("cfg1 scaled_mm fp16 256x4096x4096", 256, 4096, 4096, torch.float16, torch.float16, True, device, peaks, bound="tensor")]
    for n, k in ((12288, 3072), (3072, 12288), (9216, 3072)):
        out.append(scaled_mm_case(f"cfg2 scaled_mm bf16 4096x{n}x{k}", 4096, n, k, torch.bfloat16, torch.bfloat16, True, device, peaks))
    if not PROFILE_MODE:
        vendor = library_bf16_gemm_case(4096, 12288, 3072, device, peaks)
        out.append(vendor)
        if vendor.get("tflops") and out[1].get("tflops"):
            out[1]["frac_of_vendor_bf16_gemm_same_shape"] = _round(out[1]["tflops"] / vendor["tflops"])
    return out


def bench_msweep(device, peaks, include_65536: bool = True) -> list[dict]:
    out = []
    for m in (1, 16, 128, 1024, 8192):
        for cold in (True, False):
            out.append(scaled_mm_case(f"cfg5 scaled_mm M-sweep M={m} {'cold' if cold else 'warm'}", m, 12288, 3072, torch.bfloat16, torch.bfloat16, cold, device, peaks))
    if include_65536 and not PROFILE_MODE:   # 2 GB of output: nothing to hold on the device under a profiler
        out.append(scaled_mm_case("cfg5 scaled_mm M-sweep M=65536 (one GPU)", 65536, 12288, 3072, torch.bfloat16, torch.bfloat16, True, device, peaks))
    return out


# ------------------------------------------------------------------------------------------------------------- int8
def measure_vendor_int8(device, m=8192, n=8192, k=8192, sets=1) -> float | None:
    """TOP/s of the vendor library's int8 GEMM (`torch._int_mm`, int32 output, no scales) over `sets` rotating operand sets. At a
    large square it is the measured int8 denominator (the driver-measured peaks have no int8 figure); at a case's own shape it is
    the comparator beside the case. None if the private entry point is missing or refuses the layout."""
    if PROFILE_MODE:
        return None
    try:
        a = [torch.randint(-127, 128, (m, k), device=device, dtype=torch.int8) for _ in range(sets)]
        w_t = [torch.randint(-127, 128, (n, k), device=device, dtype=torch.int8).t() for _ in range(sets)]  # [K, N] column-major, as the library wants
        timing = time_launches(lambda i: torch._int_mm(a[i % sets], w_t[i % sets]), sets)   # the result comes from the graph's private pool
        return 2.0 * m * n * k / timing["us"] / 1e6
    except Exception:  # noqa: BLE001
        return None


def bench_int8(device, peaks) -> list[dict]:
    from . import int8_convrot as ic

    peaks = dict(peaks)
    peaks["int8_tops"] = measure_vendor_int8(device)
    m, k, n = 4096, 3072, 3072
    gen = torch.Generator(device=device).manual_seed(0)
    x = torch.randn((m, k), device=device, generator=gen)
    x[:, torch.randperm(k, device=device, generator=gen)[:31]] *= 20
    x = x.to(torch.bfloat16)
    w = (torch.randn((n, k), device=device, generator=gen) * 0.02).to(torch.bfloat16)
    wq, ws = ic.quantize_convrot_weight(w)
    packed = ic.prepack_int8_weight(wq)
    sets = 4
    xs = [x.clone() for _ in range(sets)]
    qs = [torch.empty((m, k), device=device, dtype=torch.int8) for _ in range(sets)]
    ss = [torch.empty((m,), device=device, dtype=torch.float32) for _ in range(sets)]
    outs = [torch.empty((m, n), device=device, dtype=torch.bfloat16) for _ in range(sets)]
    packs = [packed.clone().reshape(-1) for _ in range(sets)]
    tile = ic.select_int8_config(m, n, k, False)

    def quant(i):
        j = i % sets
        torch.ops.feather_ops.convrot_quantize.default(xs[j], None, qs[j], ss[j], True)

    def gemm(i, transposed=False):
        j = i % sets
        torch.ops.feather_ops.int8_scaled_mm.default(qs[j], packs[j], ss[j], None if transposed else ws, None, outs[j], transposed, *tile)

    def linear(i):
        j = i % sets
        outs[j] = ic.convrot_int8_linear(xs[j], packs[j], ws, None, torch.bfloat16, weight_packed=True)

    out = []
    q_bytes = float(m * k * 3 + m * 4)
    out.append(_rates({"case": "cfg3 convrot_quantize 4096x3072 bf16", "op": "convrot_quantize", "M": m, "K": k, "cold": True, "buffer_sets": sets},
                      time_launches(quant, sets), flop=None, algorithmic_bytes=q_bytes, bound="hbm", peaks=peaks))
    flop = 2.0 * m * n * k
    gemm_bytes = float(m * k + n * k + m * n * 2)
    vendor_here = measure_vendor_int8(device, m, n, k, sets)
    for transposed in (False, True):
        record = {"vendor_same_shape_tops": _round(vendor_here, 1), "vendor_same_shape_us": None if not vendor_here else _round(flop / vendor_here / 1e6, 2),
                  "vendor_same_shape": "torch._int_mm at this shape over the same number of rotating operand sets: int32 output, no scales, no rounding",
                  **{"case": f"cfg3 int8_scaled_mm 4096x3072x3072 {'backward (transposed_b)' if transposed else 'forward'}", "op": "int8_scaled_mm", "M": m, "N": n,
                  "K": k, "tile": list(tile), "cold": True, "buffer_sets": sets, "peak_source": "vendor int8 GEMM (torch._int_mm 8192^3) timed in this run"}}
        out.append(_rates(record, time_launches(lambda i, t=transposed: gemm(i, t), sets), flop=flop, algorithmic_bytes=gemm_bytes, bound="tensor", peaks=peaks, int8=True))
    record = {"case": "cfg3 convrot_int8_linear 4096x3072x3072 (quantize + GEMM, the public call)", "op": "convrot_int8_linear", "M": m, "N": n, "K": k, "cold": True,
              "buffer_sets": sets, "peak_source": "vendor int8 GEMM (torch._int_mm 8192^3) timed in this run"}
    out.append(_rates(record, time_launches(linear, sets), flop=flop, algorithmic_bytes=float(m * k * 2 + n * k + m * n * 2), bound="tensor", peaks=peaks, int8=True))
    del packs

    # The same three over the unpacked [N, K] weight (`weight_packed=False`): the copy engine's boxes are operands as they land
    weights = [wq.clone() for _ in range(sets)]

    def gemm_plain(i, transposed=False):
        j = i % sets
        torch.ops.feather_ops.int8_scaled_mm_plain.default(qs[j], weights[j], ss[j], None if transposed else ws, None, outs[j], transposed)

    def linear_plain(i):
        j = i % sets
        outs[j] = ic.convrot_int8_linear(xs[j], weights[j], ws, None, torch.bfloat16)

    plain = []
    for transposed in (False, True):
        record = {"vendor_same_shape_tops": _round(vendor_here, 1), "vendor_same_shape_us": None if not vendor_here else _round(flop / vendor_here / 1e6, 2),
                  "case": f"cfg3 int8_scaled_mm_plain 4096x3072x3072 {'backward (transposed_b)' if transposed else 'forward'}, unpacked weight", "op": "int8_scaled_mm_plain",
                  "M": m, "N": n, "K": k, "cold": True, "buffer_sets": sets, "peak_source": "vendor int8 GEMM (torch._int_mm 8192^3) timed in this run"}
        plain.append(_rates(record, time_launches(lambda i, t=transposed: gemm_plain(i, t), sets), flop=flop, algorithmic_bytes=gemm_bytes, bound="tensor", peaks=peaks, int8=True))
    record = {"case": "cfg3 convrot_int8_linear 4096x3072x3072, unpacked weight (quantize + GEMM, the public call with weight_packed=False)", "op": "convrot_int8_linear",
              "M": m, "N": n, "K": k, "cold": True, "buffer_sets": sets, "peak_source": "vendor int8 GEMM (torch._int_mm 8192^3) timed in this run"}
    plain.append(_rates(record, time_launches(linear_plain, sets), flop=flop, algorithmic_bytes=float(m * k * 2 + n * k + m * n * 2), bound="tensor", peaks=peaks, int8=True))
    del xs, qs, ss, outs, weights

    # a large square GEMM: many waves of tiles, so the steady state of the kernel shows
    m = n = k = 8192
    a8 = torch.randint(-127, 128, (m, k), device=device, dtype=torch.int8)
    w8 = torch.randint(-127, 128, (n, k), device=device, dtype=torch.int8)
    packed8 = ic.prepack_int8_weight(w8).reshape(-1)
    a_scale = torch.rand((m,), device=device) + 0.5
    w_scale = torch.rand((n,), device=device) + 0.5
    out8 = [torch.empty((m, n), device=device, dtype=torch.bfloat16) for _ in range(2)]
    tile8 = ic.select_int8_config(m, n, k, False)
    record = {"case": "int8_scaled_mm 8192x8192x8192 (steady state)", "op": "int8_scaled_mm", "M": m, "N": n, "K": k, "tile": list(tile8), "cold": True, "buffer_sets": 2,
              "peak_source": "vendor int8 GEMM (torch._int_mm 8192^3) timed in this run"}
    out.append(_rates(record, time_launches(lambda i: torch.ops.feather_ops.int8_scaled_mm.default(a8, packed8, a_scale, w_scale, None, out8[i % 2], False, *tile8), 2),
                      flop=2.0 * m * n * k, algorithmic_bytes=None, bound="tensor", peaks=peaks, int8=True))
    record = {"case": "int8_scaled_mm_plain 8192x8192x8192, unpacked weight (steady state)", "op": "int8_scaled_mm_plain", "M": m, "N": n, "K": k, "cold": True, "buffer_sets": 2,
              "peak_source": "vendor int8 GEMM (torch._int_mm 8192^3) timed in this run"}
    plain.append(_rates(record, time_launches(lambda i: torch.ops.feather_ops.int8_scaled_mm_plain.default(a8, w8, a_scale, w_scale, None, out8[i % 2], False), 2),
                        flop=2.0 * m * n * k, algorithmic_bytes=None, bound="tensor", peaks=peaks, int8=True))
    return out + plain


# ------------------------------------------------------------------------------------------------------------- conv
def _vendor_conv_us(x, w, bias, channels_last: bool) -> float | None:
    """Microseconds of the vendor convolution library (`F.conv2d`, cuDNN with its heuristic pick) on the same problem."""
    import torch.nn.functional as F

    try:
        sets = 3
        fmt = torch.channels_last if channels_last else torch.contiguous_format
        xs = [x.clone().contiguous(memory_format=fmt) for _ in range(sets)]
        wv = w.contiguous(memory_format=fmt)
        with torch.no_grad():
            return time_launches(lambda i: F.conv2d(xs[i % sets], wv, bias, 1, 1), sets)["us"]
    except Exception:  # noqa: BLE001
        return None


def bench_conv(device, peaks) -> list[dict]:
    from . import conv2d as fc

    out = []
    for channels, size in ((512, 128), (256, 256), (128, 512)):
        for dtype in (torch.bfloat16, torch.float16):
            gen = torch.Generator(device=device).manual_seed(channels)
            sets = 3
            xs = [torch.randn((1, channels, size, size), device=device, generator=gen).to(dtype) for _ in range(sets)]
            w = (torch.randn((channels, channels, 3, 3), device=device, generator=gen) / (9 * channels) ** 0.5).to(dtype)
            packed = fc.prepack_conv2d_weight_3x3(w)
            bias = (torch.randn(channels, device=device, generator=gen) * 0.01).to(dtype)
            outs = [torch.empty_like(xs[0]) for _ in range(sets)]
            tile = fc.select_conv3x3_config(channels, size)

            def launch(i):
                j = i % sets
                torch.ops.feather_ops.conv2d_3x3.default(xs[j], packed, bias, outs[j], *tile, False)

            flop = 2.0 * channels * channels * 9 * size * size
            record = {"case": f"cfg4 conv3x3 {channels}->{channels} @{size}x{size} {str(dtype).replace('torch.', '')}", "op": "conv2d_3x3", "C": channels, "H": size, "W": size,
                      "tile": list(tile), "cold": True, "buffer_sets": sets}
            record = _rates(record, time_launches(launch, sets), flop=flop, algorithmic_bytes=float(2 * xs[0].numel() * 2 + packed.numel() * 2), bound="tensor", peaks=peaks)
            if not PROFILE_MODE:
                for name, channels_last in (("nchw", False), ("channels_last", True)):
                    us = _vendor_conv_us(xs[0], w, bias, channels_last)
                    record[f"vendor_conv_{name}_us"] = _round(us, 2)
                    record[f"vendor_conv_{name}_tflops"] = None if not us else _round(flop / us / 1e6, 1)
                best = min((record[f"vendor_conv_{name}_us"] for name in ("nchw", "channels_last") if record[f"vendor_conv_{name}_us"]), default=None)
                record["speedup_over_vendor_conv"] = None if best is None or record["us"] is None else _round(best / record["us"])
            out.append(record)
    return out


# ------------------------------------------------------------------------------------------------------------- grids
# A spread of linear-layer shapes (rows x output width x contraction) of the kind the library meets in diffusion
# transformers: text bands of a few rows, 4k-25k image/video rows including ragged ones, narrow and very wide
# outputs, short and very long contractions. Used to check the tile heuristic against the three tile widths.
GRID_SHAPES = [
    (16, 4096, 4096), (32, 3840, 2560), (192, 2560, 2560), (256, 12288, 4096), (512, 5120, 5120), (1024, 1280, 1280),
    (2048, 1152, 4304), (2304, 10240, 1280), (4096, 4608, 4608), (4112, 4096, 12288), (4128, 11520, 3840), (5251, 21504, 5376),
    (9232, 3072, 8192), (12032, 5120, 13824), (25343, 21504, 5376), (1, 96768, 2688),
]


def bench_grid(device, peaks) -> list[dict]:
    from . import scaled_mm as smm

    out = []
    for m, n, k in GRID_SHAPES:
        weights = (torch.randn((k, n), device=device) * 8).to(torch.float8_e5m2)
        packed = smm.prepack_b_for_scaled_mm(weights)
        del weights
        a = torch.randn((m, k), device=device).to(torch.bfloat16)
        c = torch.empty((m, n), device=device, dtype=torch.bfloat16)
        scale = torch.tensor(0.01, device=device)
        times = {}
        for name, tile in (("n64", smm._TILE_N64), ("n128", smm._TILE_N128), ("n256", smm._TILE_N256)):
            if name != "n256" and m * n > 64 * 1024 * 1024:
                continue  # the narrow single-CTA tiles are never candidates for very large outputs
            times[name] = time_launches(lambda i, tile=tile: smm._launch(a, packed, scale, None, c, tile), 1, rounds=3, round_ms=20.0)["us"]
        auto = time_launches(lambda i: smm._scaled_mm_auto(a, packed, scale, None, c), 1, rounds=3, round_ms=20.0)["us"]
        best = min(times.values())
        out.append({"case": f"grid {m}x{n}x{k}", "op": "scaled_mm", "M": m, "N": n, "K": k, "auto_us": _round(auto, 1), "tflops": _round(2 * m * n * k / auto / 1e6, 1),
                    "tiles_us": {key: _round(v, 1) for key, v in times.items()}, "auto_over_best": _round(auto / best)})
        del packed, a, c
    return out


# The reference's shared shape grid (bench/cells.py:37-91 there): `(M, N_w, K_w)` cells by model family. Both GEMM
# operators run them: scaled_mm forward, the int8 GEMM in both directions (the backward contracts N_w). The two
# weight-streaming cells and the 53248-long contraction are kept; the list is the reference's, in its order.
CELL_GROUPS = {
    "ladder-wide": [(1040, 6144, 6144), (2320, 6144, 6144), (4112, 6144, 6144), (6416, 6144, 6144), (9232, 6144, 6144), (16400, 6144, 6144)],
    "ladder-narrow": [(1040, 1536, 6144), (2320, 1536, 6144), (4112, 1536, 6144), (6416, 1536, 6144), (9232, 1536, 6144), (16400, 1536, 6144)],
    "ladder-small": [(1040, 1024, 5120), (2320, 1024, 5120), (4112, 1024, 5120), (9232, 1024, 5120), (16400, 1024, 5120)],
    "sdxl": [(1024, 1280, 1280), (1024, 10240, 1280), (2304, 1280, 1280), (2304, 10240, 1280), (4096, 1280, 5120), (9216, 1280, 5120), (4096, 5120, 1280)],
    "anima": [(512, 1024, 1024), (512, 2048, 1024), (4096, 2048, 2048), (4096, 8192, 2048), (4096, 2048, 8192), (9216, 2048, 2048), (9216, 8192, 2048), (4096, 1024, 4096)],
    "qwen21": [(4096, 3072, 3072), (4096, 12288, 3072), (4096, 3072, 12288), (9216, 18432, 3072)],
    "qwen2_1": [(2, 4096, 16384), (16, 4096, 4096), (4112, 4096, 4096), (4112, 4096, 12288), (4112, 24576, 4096), (9232, 16384, 4096), (9232, 4096, 4096)],
    "zimage": [(32, 3840, 2560), (4128, 3840, 3840), (4128, 11520, 3840), (4128, 3840, 10240), (9248, 10240, 3840), (9248, 3840, 3840)],
    "krea2": [(16, 6144, 6144), (192, 1536, 6144), (4112, 6144, 16384), (4112, 16384, 6144), (4112, 2560, 6912)],
    "ideogram4": [(4096, 4608, 4608), (4096, 4608, 12288), (4096, 4608, 53248), (9232, 12288, 4608), (9232, 18432, 512)],
    "klein9b": [(512, 4096, 4096), (4096, 4096, 4096), (4096, 4096, 12288), (4608, 36864, 4096), (4608, 4096, 16384), (9216, 12288, 4096), (9728, 4096, 4096)],
    "wan": [(512, 5120, 5120), (512, 13824, 5120), (12032, 5120, 5120), (12032, 5120, 13824), (12032, 30720, 5120)],
    "ltx2_3": [(1024, 4096, 4096), (1536, 4096, 4096), (8960, 4096, 16384), (8960, 8192, 4096)],
    "h3": [(16, 5376, 5376), (512, 5376, 5120), (5251, 21504, 5376), (5376, 21504, 5376), (5376, 5376, 7168), (5376, 28672, 5376), (5376, 5376, 14336),
           (25343, 21504, 5376), (25344, 21504, 5376)],
    "moss": [(4112, 9216, 3072), (4112, 3072, 3072), (4112, 16384, 3072), (9232, 3072, 8192), (9232, 18432, 3072)],
    "short-prompt": [(32, 25600, 5120), (32, 5120, 25600), (128, 1024, 5120), (128, 8192, 5120)],
    "text-16": [(16, 3072, 3072)],
    "pad-256": [(192, 2560, 2560), (256, 2560, 2560), (192, 12288, 4096), (256, 12288, 4096), (256, 4096, 4096)],
    "text-1152": [(512, 1152, 1152), (2048, 1152, 1152), (2048, 1152, 4304), (2048, 4304, 1152), (4096, 3456, 1152)],
    "weight-stream": [(512, 248320, 4096), (1, 96768, 2688)],
}


def bench_cells(device, peaks, groups=None) -> list[dict]:
    """The reference's shape grid through the public paths of scaled_mm (bf16 x e5m2) and the int8 GEMM (forward, and
    backward where the output axis allows: N_w % 16 == 0). One warm buffer set per cell, three rounds of 20 ms."""
    from . import int8_convrot as ic
    from . import scaled_mm as smm

    out = []
    for group, cell_list in CELL_GROUPS.items():
        if groups and group not in groups:
            continue
        for m, n, k in cell_list:
            record = {"case": f"cell {group} {m}x{n}x{k}", "group": group, "M": m, "N": n, "K": k}
            flop = 2.0 * m * n * k
            packed = smm.prepack_b_for_scaled_mm((torch.randn((k, n), device=device) * 8).to(torch.float8_e5m2))
            a = torch.randn((m, k), device=device).to(torch.bfloat16)
            c = torch.empty((m, n), device=device, dtype=torch.bfloat16)
            scale = torch.tensor(0.01, device=device)
            us = time_launches(lambda i: smm._scaled_mm_auto(a, packed, scale, None, c), 1, rounds=3, round_ms=20.0)["us"]
            record.update(scaled_mm_us=_round(us, 1), scaled_mm_tflops=None if us is None else _round(flop / us / 1e6, 1), scaled_mm_path=_scaled_mm_path(m, n, k))
            del packed, a
            if k % 16 == 0 and n % 4 == 0:
                w8 = torch.randint(-127, 128, (n, k), device=device, dtype=torch.int8)
                packed8 = ic.prepack_int8_weight(w8)
                a8 = torch.randint(-127, 128, (m, k), device=device, dtype=torch.int8)
                a_scale = torch.rand((m,), device=device) + 0.5
                w_scale = torch.rand((n,), device=device) + 0.5
                us = time_launches(lambda i: ic._int8_scaled_mm_auto(a8, packed8, a_scale, w_scale, None, c, False), 1, rounds=3, round_ms=20.0)["us"]
                record.update(int8_forward_us=_round(us, 1), int8_forward_tops=None if us is None else _round(flop / us / 1e6, 1))
                # the same product over the unpacked weight (what `weight_packed=False` calls run)
                us = time_launches(lambda i: ic._int8_scaled_mm_plain(a8, w8, a_scale, w_scale, None, c, False), 1, rounds=3, round_ms=20.0)["us"]
                record.update(int8_plain_forward_us=_round(us, 1), int8_plain_forward_tops=None if us is None else _round(flop / us / 1e6, 1))
                if n % 16 == 0:
                    g8 = torch.randint(-127, 128, (m, n), device=device, dtype=torch.int8)
                    dx = torch.empty((m, k), device=device, dtype=torch.bfloat16)
                    us = time_launches(lambda i: ic._int8_scaled_mm_auto(g8, packed8, a_scale, None, None, dx, True), 1, rounds=3, round_ms=20.0)["us"]
                    record.update(int8_backward_us=_round(us, 1), int8_backward_tops=None if us is None else _round(flop / us / 1e6, 1))
                    us = time_launches(lambda i: ic._int8_scaled_mm_plain(g8, w8, a_scale, None, None, dx, True), 1, rounds=3, round_ms=20.0)["us"]
                    record.update(int8_plain_backward_us=_round(us, 1), int8_plain_backward_tops=None if us is None else _round(flop / us / 1e6, 1))
                    del g8, dx
                del packed8, a8, w8
            del c
            out.append(record)
    return out


GROUPS = {"scaled_mm": bench_scaled_mm, "msweep": bench_msweep, "int8": bench_int8, "conv": bench_conv, "grid": bench_grid, "cells": bench_cells}


def main(argv):
    if not torch.cuda.is_available():
        raise SystemExit("the benchmarks need a CUDA device: the kernels have no CPU fallback")
    import feather_ops_b200  # noqa: F401

    global PROFILE_MODE
    PROFILE_MODE = "--profile" in argv
    peaks = {}
    if "--peaks" in argv:
        with open(argv[argv.index("--peaks") + 1]) as f:
            peaks = json.load(f)
    device = torch.device("cuda")
    set_device_limits(device)
    chosen = [a for a in argv if a in GROUPS] or [g for g in GROUPS if g != "cells"]
    for name in chosen:
        for record in GROUPS[name](device, peaks):
            print(json.dumps(record), flush=True)


if __name__ == "__main__":
    main(sys.argv[1:])
