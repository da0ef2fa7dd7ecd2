"""scaled_mm on the GPU against the CPU oracle, through the C ABI and through the torch operator.

Shapes, dtype combinations and tolerances are the reference's (tests/test_scaled_mm_hip.py:8-32 there):
Frobenius rel <= 0.01 and max-abs <= 2 (fp16) / 16 (bf16) against its naive path. Against the
fp32-accumulate restatement the bound used here is much tighter (rel <= 1e-3): the only differences are
the accumulation order and one-ulp output roundings.
"""

import pytest
import torch

from oracle import scaled_mm as osm
from tests import _cabi

pytestmark = pytest.mark.gpu

SHAPES = [(1, 128, 128), (17, 96, 64), (128, 128, 128), (256, 256, 256), (512, 1024, 5120), (4111, 512, 256), (4112, 1152, 1152),
          (4304, 4304, 1152), (5376, 512, 3072), (2048, 1024, 5120)]
TAIL_SHAPE = (67, 272, 304)
DTYPES = [(torch.float8_e5m2, torch.float16), (torch.float8_e5m2, torch.bfloat16), (torch.float8_e4m3fn, torch.bfloat16)]
ATOL = {torch.float16: 2.0, torch.bfloat16: 16.0}
STATUS = "feather_scaled_mm_status"


def _compare(out, ref, out_dtype, rtol):
    diff = (out.float().cpu() - ref.float()).abs()
    rel = (diff.norm() / ref.float().norm().clamp(min=1e-6)).item()
    assert rel <= rtol, f"rel={rel:.3g}"
    assert diff.max().item() <= ATOL[out_dtype], f"max_abs={diff.max().item():.3g}"


@pytest.mark.parametrize("a_dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("b_dtype,out_dtype", DTYPES)
@pytest.mark.parametrize("shape", SHAPES)
def test_shapes_through_the_c_abi(cuda_device, shape, b_dtype, out_dtype, a_dtype):
    m, n, k = shape
    a, packed, scale, bias = osm.make_inputs(m, n, k, a_dtype, b_dtype, out_dtype)
    out = _cabi.scaled_mm(a.to(cuda_device), packed.to(cuda_device), scale.to(cuda_device), bias.to(cuda_device), out_dtype)
    _cabi.assert_clean(STATUS)
    _compare(out, osm.scaled_mm_f32(a, packed, scale, bias, out_dtype, b_prepacked=True), out_dtype, 1e-3)
    if m <= 512:  # the reference's own oracle, with the reference's tolerance
        _compare(out, osm.scaled_mm_naive(a, packed, scale, bias, out_dtype, b_prepacked=True), out_dtype, 0.01)


def test_every_tile_on_a_shape_with_a_tail_in_every_axis(cuda_device):
    from feather_ops_b200.tiles import SCALED_MM_TILES

    m, n, k = TAIL_SHAPE
    a, packed, _, bias = osm.make_inputs(m, n, k, torch.float16, torch.float8_e5m2, torch.bfloat16)
    scale = torch.tensor(0.75)
    ref = osm.scaled_mm_f32(a, packed, scale, bias, torch.bfloat16, b_prepacked=True)
    dev = [t.to(cuda_device) for t in (a, packed, scale, bias)]
    for tile in SCALED_MM_TILES:
        out = _cabi.scaled_mm(*dev, torch.bfloat16, tile)
        _cabi.assert_clean(STATUS)
        _compare(out, ref, torch.bfloat16, 1e-3)


def test_python_api_heuristic_optional_arguments_and_views(cuda_device):
    import feather_ops_b200 as fo
    from feather_ops_b200.scaled_mm import prepack_b_for_scaled_mm

    for (m, n, k), scale_on, bias_on in (((96, 128, 64), False, False), ((4112, 1152, 1152), True, False), ((300, 2048, 512), True, True)):
        a, packed, scale, bias = osm.make_inputs(m, n, k, torch.bfloat16, torch.float8_e5m2, torch.bfloat16, with_scale=scale_on, with_bias=bias_on)
        b = osm.unpack_b(packed, k)
        packed_gpu = prepack_b_for_scaled_mm(b.to(cuda_device))
        assert torch.equal(packed_gpu.cpu().view(torch.uint8), packed.view(torch.uint8))
        out = fo.scaled_mm_hip(a.to(cuda_device), packed_gpu, None if scale is None else scale.to(cuda_device), None if bias is None else bias.to(cuda_device), torch.bfloat16)
        _cabi.assert_clean(STATUS)
        _compare(out, osm.scaled_mm_f32(a, packed, scale, bias, torch.bfloat16, b_prepacked=True), torch.bfloat16, 1e-3)
    # a bias that is a 2-byte-aligned view takes the scalar load path
    a, packed, scale, _ = osm.make_inputs(40, 64, 128, torch.float16, torch.float8_e5m2, torch.float16)
    storage = torch.randn(65).to(torch.float16).to(cuda_device)
    out = fo.scaled_mm_hip(a.to(cuda_device), packed.to(cuda_device), scale.to(cuda_device), storage[1:], torch.float16)
    _compare(out, osm.scaled_mm_f32(a, packed, scale, storage[1:].cpu(), torch.float16, b_prepacked=True), torch.float16, 1e-3)
    # an empty batch launches nothing
    empty = fo.scaled_mm_hip(torch.zeros((0, 128), device=cuda_device, dtype=torch.float16), packed.to(cuda_device), None, None, torch.float16)
    assert empty.shape == (0, 64)


def test_golden_vectors_of_the_reference_naive_path(cuda_device, golden):
    for case in golden["scaled_mm"]:
        b_dtype = torch.float8_e5m2 if case["b_dtype"].endswith("e5m2") else torch.float8_e4m3fn
        packed = case["b_prepacked"].view(b_dtype).to(cuda_device)
        out = _cabi.scaled_mm(case["a"].to(cuda_device), packed, case["scale"].to(cuda_device), case["bias"].to(cuda_device), case["y"].dtype)
        _compare(out, case["y"], case["y"].dtype, 0.01)


def test_every_fp8_code_decodes_exactly(cuda_device):
    # identity activations pick single weight entries: out[i, n] = up(B[i, n]) for all 256 codes of both formats
    for b_dtype in (torch.float8_e5m2, torch.float8_e4m3fn):
        codes = torch.arange(256, dtype=torch.uint8).repeat(16, 1)[:, :256].contiguous()  # [16, 256]: row i, column n -> code n
        b = codes.view(b_dtype)
        for a_dtype in (torch.float16, torch.bfloat16):
            a = torch.eye(16, dtype=a_dtype)
            out = _cabi.scaled_mm(a.to(cuda_device), osm.prepack_b(b).to(cuda_device), None, None, torch.float16 if a_dtype == torch.float16 else torch.bfloat16)
            expect = b.to(torch.float32)
            got = out.float().cpu()
            finite = torch.isfinite(expect)
            assert torch.equal(got[finite], expect[finite])  # every finite fp8 value is exact in fp16 and in bf16
            assert not torch.isfinite(got[~finite]).any()  # inf and NaN codes stay non-finite (0 * inf in the other rows)


def test_operator_errors(cuda_device):
    import feather_ops_b200  # noqa: F401

    op = torch.ops.feather_ops.scaled_mm.default
    tile = (1, 8, 4, 8, 2, False)
    a = torch.zeros((8, 64), device=cuda_device, dtype=torch.float16)
    b = torch.zeros((8, 32, 16), device=cuda_device, dtype=torch.float8_e5m2)
    c = torch.zeros((8, 32), device=cuda_device, dtype=torch.float16)
    op(a, b, None, None, c, *tile)
    with pytest.raises(RuntimeError, match="Unsupported config"):
        op(a, b, None, None, c, 3, 3, 3, 3, 3, False)
    with pytest.raises(RuntimeError, match="K must be divisible by 16"):
        op(a[:, :40].contiguous(), b, None, None, c, *tile)
    with pytest.raises(RuntimeError, match=r"a.stride\(0\) must equal K"):
        op(a[:, :32], b, None, None, c, *tile)
    with pytest.raises(RuntimeError, match="a must be float16 or bfloat16"):
        op(a.float(), b, None, None, c, *tile)
    with pytest.raises(RuntimeError, match="b_prepacked must be float8"):
        op(a, b.view(torch.uint8), None, None, c, *tile)
    with pytest.raises(RuntimeError, match="bias must have the same dtype as c"):
        op(a, b, None, torch.zeros(32, device=cuda_device, dtype=torch.bfloat16), c, *tile)
    with pytest.raises(RuntimeError, match="scale must have one element"):
        op(a, b, torch.zeros(2, device=cuda_device), None, c, *tile)
    with pytest.raises(RuntimeError, match="multiple of 8"):
        op(a, b[:4].contiguous(), None, None, c, *tile)
    with pytest.raises(RuntimeError, match=r"c.shape\[1\] must equal N"):
        op(a, b, None, None, torch.zeros((8, 16), device=cuda_device, dtype=torch.float16), *tile)


@pytest.mark.parametrize("dynamic", [False, True])
@pytest.mark.parametrize("shape", [(4112, 1152, 1152), (512, 1024, 5120)])
def test_compile_matches_eager(cuda_device, shape, dynamic):
    # the reference's compile test (tests/test_scaled_mm_hip_compile.py:19-33 there): default backend, static and
    # dynamic shapes, one opaque node, same result as eager and within the reference tolerance of its naive path
    import feather_ops_b200 as fo

    m, n, k = shape
    a, packed, scale, bias = osm.make_inputs(m, n, k, torch.bfloat16, torch.float8_e5m2, torch.bfloat16)
    args = [t.to(cuda_device) for t in (a, packed, scale, bias)]

    def run(a, b, s, bias):
        return fo.scaled_mm_hip(a, b, s, bias, torch.bfloat16)

    eager = run(*args)
    torch._dynamo.reset()
    compiled = torch.compile(run, fullgraph=True, dynamic=dynamic)(*args)
    assert torch.equal(compiled, eager)
    _compare(compiled, osm.scaled_mm_naive(a, packed, scale, bias, torch.bfloat16, b_prepacked=True), torch.bfloat16, 0.01)
    traced = torch.compile(run, fullgraph=True, backend="aot_eager")(*args)
    assert torch.equal(traced, eager)


@pytest.mark.parametrize("n,k", [(12288, 3072), (3072, 12288), (9216, 3072)])
def test_benchmark_shapes_whole_output(cuda_device, n, k):
    # M = 4096 on the benchmark distribution (per-tensor scale = absmax / 57344): every element of the output against
    # the fp32-accumulate oracle (an fp64 product on the host cores, about a second), then row independence (a row's
    # result does not depend on which tile or launch it is in) and exact scaling by a power of two.
    m = 4096
    a, packed, scale, _ = osm.make_inputs(m, n, k, torch.bfloat16, torch.float8_e5m2, torch.bfloat16, weight_std=0.02, with_bias=False)
    a_gpu, packed_gpu, scale_gpu = a.to(cuda_device), packed.to(cuda_device), scale.to(cuda_device)
    out = _cabi.scaled_mm(a_gpu, packed_gpu, scale_gpu, None, torch.bfloat16)
    _cabi.assert_clean(STATUS)
    assert torch.isfinite(out).all()
    ref = osm.scaled_mm_f32(a, packed, scale, None, torch.bfloat16, b_prepacked=True)
    _compare(out, ref, torch.bfloat16, 1e-3)
    # per 256 x 256 tile as well: a fault confined to one tile cannot hide in the norm of the whole matrix
    diff = (out.float().cpu() - ref.float()).reshape(m // 256, 256, n // 256, 256)
    tile_rel = diff.pow(2).sum(dim=(1, 3)).sqrt() / ref.float().reshape(m // 256, 256, n // 256, 256).pow(2).sum(dim=(1, 3)).sqrt()
    assert tile_rel.max().item() <= 2e-3, f"worst tile rel={tile_rel.max().item():.3g}"
    sub = _cabi.scaled_mm(a_gpu[1000:1130].contiguous(), packed_gpu, scale_gpu, None, torch.bfloat16)
    assert torch.equal(sub, out[1000:1130])
    doubled = _cabi.scaled_mm(a_gpu, packed_gpu, (scale_gpu * 2).contiguous(), None, torch.bfloat16)
    assert torch.equal(doubled.float(), out.float() * 2)
    _cabi.assert_clean(STATUS)


def test_reference_cpu_case_fp16(cuda_device):
    # 256 x 4096 x 4096 fp16 on the benchmark distribution, whole output against the fp32 oracle
    a, packed, scale, _ = osm.make_inputs(256, 4096, 4096, torch.float16, torch.float8_e5m2, torch.float16, weight_std=0.02, with_bias=False)
    out = _cabi.scaled_mm(a.to(cuda_device), packed.to(cuda_device), scale.to(cuda_device), None, torch.float16)
    _cabi.assert_clean(STATUS)
    _compare(out, osm.scaled_mm_f32(a, packed, scale, None, torch.float16, b_prepacked=True), torch.float16, 1e-3)


@pytest.mark.parametrize("a_dtype,b_dtype,out_dtype", [(torch.bfloat16, torch.float8_e5m2, torch.bfloat16), (torch.float16, torch.float8_e4m3fn, torch.float16)])
@pytest.mark.parametrize("shape", [(1, 128, 128), (1, 12288, 3072), (16, 12288, 3072), (17, 272, 1040), (33, 96, 4096), (128, 3072, 1024)])
def test_skinny_split_k_through_the_c_abi(cuda_device, shape, a_dtype, b_dtype, out_dtype):
    m, n, k = shape
    a, packed, scale, bias = osm.make_inputs(m, n, k, a_dtype, b_dtype, out_dtype, seed=m + k)
    ref = osm.scaled_mm_f32(a, packed, scale, bias, out_dtype, b_prepacked=True)
    dev = [t.to(cuda_device) for t in (a, packed, scale, bias)]
    partials = counters = None
    for splits in (1, 2, 3, 4, 4):
        out, partials_used, counters_used = _cabi.scaled_mm_splitk(*dev, out_dtype, splits, partials if splits == 4 else None, counters if splits == 4 else None)
        _cabi.assert_clean(STATUS)
        _compare(out, ref, out_dtype, 1e-3)
        assert int(counters_used.abs().sum().item()) == 0  # every launch leaves its tickets at zero
        if splits == 4:
            if partials is not None:
                assert torch.equal(out, previous)  # same scratch reused, split order fixed: bit identical
            partials, counters, previous = partials_used, counters_used, out


@pytest.mark.parametrize("a_dtype,b_dtype,out_dtype", [(torch.bfloat16, torch.float8_e5m2, torch.bfloat16), (torch.float16, torch.float8_e4m3fn, torch.float16)])
@pytest.mark.parametrize("shape", [(129, 272, 1040), (384, 3072, 4096), (256, 1040, 8192), (200, 48, 64), (700, 528, 2000 // 16 * 16)])
def test_split_k_of_the_one_cta_kernel_through_the_c_abi(cuda_device, shape, a_dtype, b_dtype, out_dtype):
    # (tile, K split) work items on the persistent kernel: ragged rows and columns, more splits than k blocks, a
    # persistent CTA that meets several items, tickets back at zero, and the same bits whoever draws the last ticket
    m, n, k = shape
    a, packed, scale, bias = osm.make_inputs(m, n, k, a_dtype, b_dtype, out_dtype, seed=m + k)
    ref = osm.scaled_mm_f32(a, packed, scale, bias, out_dtype, b_prepacked=True)
    dev = [t.to(cuda_device) for t in (a, packed, scale, bias)]
    for block_n in (128, 256):
        partials = counters = previous = None
        for splits in (1, 2, 3, 5, 5, 5):
            reuse = splits == 5 and partials is not None
            out, partials_used, counters_used = _cabi.scaled_mm_splitk_wide(*dev, out_dtype, block_n, splits, partials if reuse else None,
                                                                            counters if reuse else None)
            _cabi.assert_clean(STATUS)
            _compare(out, ref, out_dtype, 1e-3)
            assert int(counters_used.abs().sum().item()) == 0
            if splits == 5:
                if previous is not None:
                    assert torch.equal(out, previous)
                partials, counters, previous = partials_used, counters_used, out


def test_split_k_of_the_one_cta_kernel_is_what_the_heuristic_picks_for_few_tiles_and_long_k(cuda_device):
    import feather_ops_b200 as fo
    from feather_ops_b200 import scaled_mm as sm

    assert sm.select_wide_splits(384, 3072, 12288) == 2 and sm.select_wide_splits(256, 4096, 4096) == 2 and sm.select_wide_splits(256, 3072, 8192) == 3
    assert sm.select_wide_splits(4096, 12288, 3072) == 1 and sm.select_wide_splits(16, 3072, 12288) == 1 and sm.select_wide_splits(192, 2560, 2560) == 1
    assert sm.select_wide_splits(512, 2560, 2560) == 1 and sm.select_wide_splits(128, 12288, 3072) == 1
    assert sm.select_wide_splits(128, 3072, 12288) == 6 and sm.select_wide_splits(100, 5120, 5120) == 3 and sm.select_wide_splits(128, 4096, 4096) == 4
    assert sm.select_wide_splits(48, 8192, 3072) == 1 and sm.select_wide_splits(64, 5120, 5120) == 3
    # more than 128 rows and few 256 x 256 tiles: K splits on CTA pairs, from K = 4096 (K = 3072 with more than 256 rows)
    assert sm.select_pair_splits(256, 4096, 4096) == 4 and sm.select_pair_splits(512, 3072, 12288) == 3 and sm.select_pair_splits(768, 2048, 8192) == 3
    assert sm.select_pair_splits(256, 3072, 3072) == 1 and sm.select_pair_splits(512, 3072, 3072) == 3 and sm.select_pair_splits(512, 1280, 1280) == 1
    assert sm.select_pair_splits(128, 4096, 4096) == 1 and sm.select_pair_splits(4096, 12288, 3072) == 1 and sm.select_pair_splits(1024, 4096, 4096) == 1
    # one row tile of 64..128 rows and 32..74 column tiles of 256: three or more K splits of the one-CTA kernel with 128 x 256 tiles
    assert sm.select_row_tile_splits_256(128, 12288, 3072) == 3 and sm.select_row_tile_splits_256(64, 8192, 3072) == 4 and sm.select_row_tile_splits_256(48, 12288, 3072) == 1
    assert sm.select_row_tile_splits_256(128, 4096, 4096) == 1 and sm.select_row_tile_splits_256(129, 12288, 3072) == 1
    assert sm.warp_mma_takes(16, 4096, 4096) and sm.warp_mma_takes(64, 3072, 3072) and not sm.warp_mma_takes(64, 12288, 3072)
    assert not sm.warp_mma_takes(32, 3072, 12288) and not sm.warp_mma_takes(8, 256, 4096)
    for m, n, k in [(100, 2064, 1040), (65, 528, 4096), (48, 1040, 528), (128, 1296, 272), (33, 3072, 8192 + 64), (300, 1040, 4112), (513, 272, 8192)]:
        a, packed, scale, bias = osm.make_inputs(m, n, k, torch.float16, torch.float8_e4m3fn, torch.float16, seed=m + n)
        ref = osm.scaled_mm_f32(a, packed, scale, bias, torch.float16, b_prepacked=True)
        dev = [t.to(cuda_device) for t in (a, packed, scale, bias)]
        out = fo.scaled_mm_hip(*dev, torch.float16)
        _cabi.assert_clean(STATUS)
        _compare(out, ref, torch.float16, 1e-3)
        assert torch.equal(out, fo.scaled_mm_hip(*dev, torch.float16))
    a, packed, scale, bias = osm.make_inputs(384, 3072, 8192, torch.bfloat16, torch.float8_e5m2, torch.bfloat16, seed=5)
    ref = osm.scaled_mm_f32(a, packed, scale, bias, torch.bfloat16, b_prepacked=True)
    dev = [t.to(cuda_device) for t in (a, packed, scale, bias)]
    out = fo.scaled_mm_hip(*dev, torch.bfloat16)
    _cabi.assert_clean(STATUS)
    _compare(out, ref, torch.bfloat16, 1e-3)
    assert torch.equal(out, fo.scaled_mm_hip(*dev, torch.bfloat16))


@pytest.mark.parametrize("a_dtype,b_dtype,out_dtype", [(torch.bfloat16, torch.float8_e5m2, torch.bfloat16), (torch.float16, torch.float8_e4m3fn, torch.float16),
                                                       (torch.float16, torch.float8_e5m2, torch.bfloat16)])
@pytest.mark.parametrize("shape", [(1, 9472, 512), (2, 12288, 3072), (1, 20000, 1040), (2, 9600, 16)])
def test_one_and_two_rows_take_the_vector_kernel(cuda_device, shape, a_dtype, b_dtype, out_dtype):
    # wide outputs with one or two rows run on CUDA cores (no tensor core): same oracle, same tolerance, and the
    # result is the same on every call (the partial sums of the eight warps are added in warp order)
    m, n, k = shape
    a, packed, scale, bias = osm.make_inputs(m, n, k, a_dtype, b_dtype, out_dtype, seed=n + k)
    ref = osm.scaled_mm_f32(a, packed, scale, bias, out_dtype, b_prepacked=True)
    dev = [t.to(cuda_device) for t in (a, packed, scale, bias)]
    first = _cabi.scaled_mm(*dev, out_dtype, (1, 2, 4, 1, 2, 1))
    _cabi.assert_clean(STATUS)
    _compare(first, ref, out_dtype, 1e-3)
    again, _, _ = _cabi.scaled_mm_splitk(*dev, out_dtype, 1)   # one split through the split-K entry point: the same kernel
    assert torch.equal(first, again)
    split, _, _ = _cabi.scaled_mm_splitk(*dev, out_dtype, 2)   # an explicit K split runs the tcgen05 split-K kernel instead
    _compare(split, ref, out_dtype, 1e-3)
    no_bias = _cabi.scaled_mm(dev[0], dev[1], None, None, out_dtype, (1, 2, 4, 1, 2, 1))
    _compare(no_bias, osm.scaled_mm_f32(a, packed, None, None, out_dtype, b_prepacked=True), out_dtype, 1e-3)


@pytest.mark.parametrize("a_dtype,b_dtype,out_dtype", [(torch.bfloat16, torch.float8_e5m2, torch.bfloat16), (torch.float16, torch.float8_e4m3fn, torch.float16),
                                                       (torch.float16, torch.float8_e5m2, torch.bfloat16)])
@pytest.mark.parametrize("shape", [(3, 9472, 512), (8, 12288, 3072), (9, 9488, 1040), (16, 20000, 256), (16, 9600, 16), (1, 4096, 4096), (2, 528, 1040),
                                   (16, 3072, 3072), (7, 1296, 272), (17, 3072, 3072), (40, 1296, 272), (128, 1040, 528), (100, 528, 8192)])
def test_few_rows_take_the_warp_mma_kernel(cuda_device, shape, a_dtype, b_dtype, out_dtype):
    # 3..16 rows (1..16 for outputs too narrow for the vector kernel; up to 128 as grid rows of 16 while every CTA is
    # resident and K <= 8192) run on mma.sync with the contraction index permuted inside each 16-deep slab:
    # same oracle and tolerance, ragged last column block (9488 = 296.5 x 32), same bits on every call
    m, n, k = shape
    a, packed, scale, bias = osm.make_inputs(m, n, k, a_dtype, b_dtype, out_dtype, seed=n + k)
    ref = osm.scaled_mm_f32(a, packed, scale, bias, out_dtype, b_prepacked=True)
    dev = [t.to(cuda_device) for t in (a, packed, scale, bias)]
    first = _cabi.scaled_mm(*dev, out_dtype, (1, 2, 4, 1, 2, 1))
    _cabi.assert_clean(STATUS)
    _compare(first, ref, out_dtype, 1e-3)
    again, _, _ = _cabi.scaled_mm_splitk(*dev, out_dtype, 1)   # one split through the split-K entry point: the same kernel
    assert torch.equal(first, again)
    split, _, _ = _cabi.scaled_mm_splitk(*dev, out_dtype, 3)   # an explicit K split runs the tcgen05 split-K kernel instead
    _cabi.assert_clean(STATUS)
    _compare(split, ref, out_dtype, 1e-3)
    no_scale = _cabi.scaled_mm(dev[0], dev[1], None, None, out_dtype, (1, 2, 4, 1, 2, 1))
    _compare(no_scale, osm.scaled_mm_f32(a, packed, None, None, out_dtype, b_prepacked=True), out_dtype, 1e-3)


def test_skinny_shapes_through_the_python_api(cuda_device):
    import feather_ops_b200 as fo
    from feather_ops_b200.scaled_mm import select_scaled_mm_splits

    assert select_scaled_mm_splits(1, 3072, 12288) > 1 and select_scaled_mm_splits(64, 3072, 12288) == 1
    for m, n, k in ((1, 12288, 3072), (16, 3072, 12288), (100, 12288, 3072), (128, 3072, 1024), (77, 8208, 3088)):
        a, packed, scale, bias = osm.make_inputs(m, n, k, torch.bfloat16, torch.float8_e5m2, torch.bfloat16, weight_std=0.02, with_bias=False)
        out = fo.scaled_mm_hip(a.to(cuda_device), packed.to(cuda_device), scale.to(cuda_device), None, torch.bfloat16)
        _cabi.assert_clean(STATUS)
        _compare(out, osm.scaled_mm_f32(a, packed, scale, None, torch.bfloat16, b_prepacked=True), torch.bfloat16, 1e-3)
