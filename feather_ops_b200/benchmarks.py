"""Per-operator measurements of the BASELINE configurations (everything except the headline step of bench.py).

    python -m feather_ops_b200.benchmarks [scaled_mm] [msweep] [grid] [int8] [conv] [--profile]     # default: all groups

`--profile` is for runs under a profiler: every case makes three plain launches (no CUDA graph, no timing), so a
capture of one kernel stays a handful of launches; the printed times are then null.

Protocol (after the reference's bench/protocol.py): warm-up, then rounds of back-to-back launches inside
one CUDA-event pair, median over the rounds. The launches of a round are replayed from a CUDA graph so that
kernels of a few microseconds are not timed as Python call overhead. Inputs rotate over enough distinct
buffer sets to exceed the 126 MB L2 ("cold") unless stated; skinny shapes are reported both ways. One JSON
object per case on stdout.
"""

import json
import statistics
import sys

import torch

L2_BYTES = 126 * 1024 * 1024
HBM_PEAK_GBS = 6538.3   # measured copy bandwidth of this pool's B200 (MEASURED_PEAKS.json)
BF16_PEAK_TFLOPS = 1635.2  # measured cuBLAS bf16 burst
INT8_NOMINAL_TOPS = 4500.0
BF16_NOMINAL_TFLOPS = 2250.0


PROFILE_MODE = False


def time_graph(launch, sets: int, rounds: int = 5, launches_per_round: int = 20) -> float:
    """Median microseconds per launch. `launch(i)` enqueues one launch on buffer set `i % sets`."""
    if PROFILE_MODE:
        for i in range(3):
            launch(i)
        torch.cuda.synchronize()
        return float("nan")
    for i in range(max(3, sets)):
        launch(i)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for i in range(launches_per_round):
            launch(i)
    graph.replay()
    torch.cuda.synchronize()
    samples = []
    for _ in range(rounds):
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        graph.replay()
        stop.record()
        torch.cuda.synchronize()
        samples.append(start.elapsed_time(stop) * 1e3 / launches_per_round)
    return statistics.median(samples)


def sets_for(bytes_per_set: int, cold: bool) -> int:
    return max(1, -(-2 * L2_BYTES // max(bytes_per_set, 1))) if cold else 1


def emit(**fields) -> None:
    fields = {k: (None if isinstance(v, float) and v != v else v) for k, v in fields.items()}
    print(json.dumps(fields), flush=True)


def _scaled_mm_case(m, n, k, a_dtype, out_dtype, cold, device, label):
    from . import scaled_mm as smm

    algorithmic = m * k * 2 + k * n + m * n * 2
    sets = min(sets_for(algorithmic, cold), 8)
    weights = (torch.randn((k, n), device=device) * 8).to(torch.float8_e5m2)
    packed = [smm.prepack_b_for_scaled_mm(weights) if i == 0 else None for i in range(sets)]
    for i in range(1, sets):
        packed[i] = packed[0].clone()
    acts = [torch.randn((m, k), device=device).to(a_dtype) for _ in range(sets)]
    outs = [torch.empty((m, n), device=device, dtype=out_dtype) for _ in range(sets)]
    scale = torch.tensor(0.01, device=device)
    # what the public path picks, in its order of preference
    if m <= 128 and smm.warp_mma_takes(m, n, k):
        tile = ("vector or warp-MMA kernel",)
    elif smm.select_wide_splits(m, n, k) > 1:
        tile = ("one-CTA kernel, 128 x 128 tiles, K splits", smm.select_wide_splits(m, n, k))
    elif 64 < m <= 128 and -(-n // 128) >= 74:
        tile = smm._TILE_N128
    elif m <= 128:
        tile = ("skinny", smm.select_scaled_mm_splits(m, n, k))
    else:
        tile = smm.select_scaled_mm_config(m, n, k)

    def launch(i):
        j = i % sets
        smm._scaled_mm_auto(acts[j], packed[j], scale, None, outs[j])  # the public path: tile / split heuristics included

    us = time_graph(launch, sets)
    tflops = 2 * m * n * k / us / 1e6
    gbs = algorithmic / us / 1e3
    emit(case=label, op="scaled_mm", M=m, N=n, K=k, a_dtype=str(a_dtype), cold=cold, tile=list(tile), us=round(us, 2), tflops=round(tflops, 1),
         frac_of_measured_bf16=round(tflops / BF16_PEAK_TFLOPS, 3), frac_of_nominal=round(tflops / BF16_NOMINAL_TFLOPS, 3), gbs=round(gbs, 1),
         frac_of_measured_hbm=round(gbs / HBM_PEAK_GBS, 3), algorithmic_bytes=algorithmic)


def bench_scaled_mm(device):
    _scaled_mm_case(256, 4096, 4096, torch.float16, torch.float16, True, device, "cfg1 fp16 256x4096x4096")
    for n, k in ((12288, 3072), (3072, 12288), (9216, 3072)):
        _scaled_mm_case(4096, n, k, torch.bfloat16, torch.bfloat16, True, device, f"cfg2 bf16 4096x{n}x{k}")
    if not PROFILE_MODE:
        # the vendor library's plain bf16 GEMM at the metric shape (both operands already bf16, no fp8 decode, no
        # scale): the measured tensor-core denominator for exactly this shape, with the same rotation of buffers
        m, n, k = 4096, 12288, 3072
        sets = 4
        acts = [torch.randn((m, k), device=device).to(torch.bfloat16) for _ in range(sets)]
        weights = [torch.randn((k, n), device=device).to(torch.bfloat16) for _ in range(sets)]
        outs = [torch.empty((m, n), device=device, dtype=torch.bfloat16) for _ in range(sets)]
        us = time_graph(lambda i: torch.matmul(acts[i % sets], weights[i % sets], out=outs[i % sets]), sets)
        emit(case="library bf16 GEMM 4096x12288x3072 (torch.matmul)", op="library_gemm", us=round(us, 2), tflops=round(2 * m * n * k / us / 1e6, 1))


def bench_msweep(device):
    for m in (1, 16, 128, 1024, 8192):
        for cold in (True, False):
            _scaled_mm_case(m, 12288, 3072, torch.bfloat16, torch.bfloat16, cold, device, f"cfg5 M-sweep M={m}")
    _scaled_mm_case(65536, 12288, 3072, torch.bfloat16, torch.bfloat16, True, device, "cfg5 M-sweep M=65536 (one GPU)")


# A spread of linear-layer shapes (rows x output width x contraction) of the kind the library meets in diffusion
# transformers: text bands of a few rows, 4k-25k image/video rows including ragged ones, narrow and very wide
# outputs, short and very long contractions. Used to check the tile heuristic against the three tile widths.
GRID_SHAPES = [
    (16, 4096, 4096), (32, 3840, 2560), (192, 2560, 2560), (256, 12288, 4096), (512, 5120, 5120), (1024, 1280, 1280),
    (2048, 1152, 4304), (2304, 10240, 1280), (4096, 4608, 4608), (4112, 4096, 12288), (4128, 11520, 3840), (5251, 21504, 5376),
    (9232, 3072, 8192), (12032, 5120, 13824), (25343, 21504, 5376), (1, 96768, 2688),
]


def bench_grid(device):
    from . import scaled_mm as smm

    for m, n, k in GRID_SHAPES:
        weights = (torch.randn((k, n), device=device) * 8).to(torch.float8_e5m2)
        packed = smm.prepack_b_for_scaled_mm(weights)
        del weights
        a = torch.randn((m, k), device=device).to(torch.bfloat16)
        out = torch.empty((m, n), device=device, dtype=torch.bfloat16)
        scale = torch.tensor(0.01, device=device)
        launches = 3 if 2 * m * n * k > 2e12 else 10
        times = {}
        for name, tile in (("n64", smm._TILE_N64), ("n128", smm._TILE_N128), ("n256", smm._TILE_N256)):
            if name != "n256" and m * n > 64 * 1024 * 1024:
                continue  # the narrow single-CTA tiles are never candidates for very large outputs
            times[name] = time_graph(lambda i, tile=tile: smm._launch(a, packed, scale, None, out, tile), 1, rounds=3, launches_per_round=launches)
        auto = time_graph(lambda i: smm._scaled_mm_auto(a, packed, scale, None, out), 1, rounds=3, launches_per_round=launches)
        best = min(times.values())
        emit(case=f"grid {m}x{n}x{k}", op="scaled_mm", M=m, N=n, K=k, auto_us=round(auto, 1), tflops=round(2 * m * n * k / auto / 1e6, 1),
             tiles_us={key: round(v, 1) for key, v in times.items()}, auto_over_best=round(auto / best, 3))
        del packed, a, out


def bench_int8(device):
    from . import int8_convrot as ic

    m, k, n = 4096, 3072, 3072
    x = torch.randn((m, k), device=device)
    x[:, torch.randperm(k, device=device)[:31]] *= 20
    x = x.to(torch.bfloat16)
    w = (torch.randn((n, k), device=device) * 0.02).to(torch.bfloat16)
    wq, ws = ic.quantize_convrot_weight(w)
    packed = ic.prepack_int8_weight(wq)
    sets = 4
    xs = [x.clone() for _ in range(sets)]
    qs = [torch.empty((m, k), device=device, dtype=torch.int8) for _ in range(sets)]
    ss = [torch.empty((m,), device=device, dtype=torch.float32) for _ in range(sets)]
    outs = [torch.empty((m, n), device=device, dtype=torch.bfloat16) for _ in range(sets)]
    packs = [packed.clone() for _ in range(sets)]
    tile = ic.select_int8_config(m, n, k, False)

    def quant(i):
        j = i % sets
        torch.ops.feather_ops.convrot_quantize.default(xs[j], None, qs[j], ss[j], True)

    def gemm(i, transposed=False):
        j = i % sets
        torch.ops.feather_ops.int8_scaled_mm.default(qs[j], packs[j].reshape(-1), ss[j], None if transposed else ws, None, outs[j], transposed, *tile)

    def linear(i):
        quant(i)
        gemm(i)

    us = time_graph(quant, sets)
    q_bytes = m * k * 3 + m * 4
    emit(case="cfg3 convrot_quantize 4096x3072 bf16", op="convrot_quantize", us=round(us, 2), gbs=round(q_bytes / us / 1e3, 1),
         frac_of_measured_hbm=round(q_bytes / us / 1e3 / HBM_PEAK_GBS, 3), algorithmic_bytes=q_bytes)
    for transposed in (False, True):
        us = time_graph(lambda i: gemm(i, transposed), sets)
        tops = 2 * m * n * k / us / 1e6
        emit(case=f"cfg3 int8_scaled_mm 4096x3072x3072 transposed_b={transposed}", op="int8_scaled_mm", tile=list(tile), us=round(us, 2),
             tops=round(tops, 1), frac_of_nominal_int8=round(tops / INT8_NOMINAL_TOPS, 3))
    us = time_graph(linear, sets)
    emit(case="cfg3 convrot_int8_linear (quantize + GEMM) 4096x3072x3072", op="convrot_int8_linear", us=round(us, 2),
         tops=round(2 * m * n * k / us / 1e6, 1))

    # a large square GEMM: many waves of tiles, so the steady state of the kernel shows
    m = n = k = 8192
    a8 = torch.randint(-127, 128, (m, k), device=device, dtype=torch.int8)
    w8 = torch.randint(-127, 128, (n, k), device=device, dtype=torch.int8)
    packed8 = ic.prepack_int8_weight(w8).reshape(-1)
    a_scale = torch.rand((m,), device=device) + 0.5
    w_scale = torch.rand((n,), device=device) + 0.5
    out8 = [torch.empty((m, n), device=device, dtype=torch.bfloat16) for _ in range(2)]
    tile = ic.select_int8_config(m, n, k, False)

    def big(i):
        torch.ops.feather_ops.int8_scaled_mm.default(a8, packed8, a_scale, w_scale, None, out8[i % 2], False, *tile)

    us = time_graph(big, 2)
    tops = 2 * m * n * k / us / 1e6
    # the vendor library's int8 GEMM at the same size as a measured denominator (there is no driver-measured int8 peak)
    library_tops = None
    if not PROFILE_MODE:
        try:
            w_t = w8.t()  # [K, N] column-major view, the layout the library kernel wants
            lib_us = time_graph(lambda i: torch._int_mm(a8, w_t), 1)
            library_tops = 2 * m * n * k / lib_us / 1e6
        except Exception:  # noqa: BLE001 - the private torch entry point may be missing or refuse the layout
            library_tops = None
    emit(case="int8_scaled_mm 8192x8192x8192 (steady state)", op="int8_scaled_mm", tile=list(tile), us=round(us, 2), tops=round(tops, 1),
         frac_of_nominal_int8=round(tops / INT8_NOMINAL_TOPS, 3), library_int8_gemm_tops=None if library_tops is None else round(library_tops, 1),
         frac_of_library_int8_gemm=None if library_tops is None else round(tops / library_tops, 3))


def bench_conv(device):
    from . import conv2d as fc

    for channels, size in ((512, 128), (256, 256), (128, 512)):
        for dtype in (torch.bfloat16, torch.float16):
            x_bytes = channels * size * size * 2
            sets = 3
            xs = [torch.randn((1, channels, size, size), device=device).to(dtype) for _ in range(sets)]
            w = (torch.randn((channels, channels, 3, 3), device=device) / (9 * channels) ** 0.5).to(dtype)
            packed = fc.prepack_conv2d_weight_3x3(w)
            bias = (torch.randn(channels, device=device) * 0.01).to(dtype)
            outs = [torch.empty_like(xs[0]) for _ in range(sets)]
            tile = fc.select_conv3x3_config(channels, size)

            def launch(i):
                j = i % sets
                torch.ops.feather_ops.conv2d_3x3.default(xs[j], packed, bias, outs[j], *tile, False)

            us = time_graph(launch, sets)
            tflops = 2 * channels * channels * 9 * size * size / us / 1e6
            emit(case=f"cfg4 conv3x3 {channels}->{channels} @{size}x{size} {dtype}", op="conv2d_3x3", tile=list(tile), us=round(us, 2),
                 tflops=round(tflops, 1), frac_of_measured_bf16=round(tflops / BF16_PEAK_TFLOPS, 3),
                 frac_of_nominal=round(tflops / BF16_NOMINAL_TFLOPS, 3), algorithmic_bytes=2 * x_bytes + packed.numel() * 2)


def main(argv):
    if not torch.cuda.is_available():
        raise SystemExit("the benchmarks need a CUDA device: the kernels have no CPU fallback")
    import feather_ops_b200  # noqa: F401

    global PROFILE_MODE
    PROFILE_MODE = "--profile" in argv
    device = torch.device("cuda")
    groups = {"scaled_mm": bench_scaled_mm, "msweep": bench_msweep, "grid": bench_grid, "int8": bench_int8, "conv": bench_conv}
    chosen = [a for a in argv if a in groups] or list(groups)
    for name in chosen:
        groups[name](device)


if __name__ == "__main__":
    main(sys.argv[1:])
