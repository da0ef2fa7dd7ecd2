"""The int8 ConvRot path on the GPU: quantizer codes bit-exact against the CPU restatement of the reference
kernel's arithmetic, GEMM against the fp64 oracle with the reference's tolerance (tests/test_int8_convrot.py
there: max-rel < 0.02 with a 1e-3 floor), compositions bit-exact against their parts."""

import gc

import pytest
import torch

from oracle import int8_convrot as o8
from tests import _cabi

pytestmark = pytest.mark.gpu
STATUS = "feather_int8_mm_status"


def _max_rel(out, ref):
    return ((out.float().cpu() - ref.float()).abs() / ref.float().abs().clamp(min=1e-3)).max().item()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("rotate", [True, False])
@pytest.mark.parametrize("shape", [(1, 256), (5, 512), (64, 1024), (33, 3072), (257, 4096), (4, 12288), (3, 33024), (2, 65536), (2, 248320)])
def test_quantizer_codes_and_scales_are_bit_exact(cuda_device, shape, rotate, dtype):
    m, k = shape
    x = o8.make_activation(m, k, dtype, seed=m + k)
    col = None if rotate else torch.rand(k, generator=torch.Generator().manual_seed(k)) + 0.5
    q_ref, s_ref = o8.convrot_quantize(x, rotate, col)
    q, s = _cabi.convrot_quantize(x.to(cuda_device), rotate, None if col is None else col.to(cuda_device))
    assert torch.equal(q.cpu(), q_ref)
    assert torch.equal(s.cpu(), s_ref)


def _recipe_bounds(q, s, q_recipe, s_recipe):
    # the reference's own bounds (tests/test_int8_convrot.py:280-286 there): the kernel sums in another order than the
    # matmul recipe, so codes on a .5 boundary may flip by one; fewer than one in a thousand may
    assert (q != q_recipe).float().mean().item() < 1e-3
    assert (q.int() - q_recipe.int()).abs().max().item() <= 1
    assert ((s - s_recipe).abs() / s_recipe.abs()).max().item() < 1e-2
    dq, ref_dq = q.float() * s[:, None], q_recipe.float() * s_recipe[:, None]
    assert ((dq - ref_dq).norm() / ref_dq.norm()).item() < 1e-3


def test_quantizer_against_the_reference_recipe(cuda_device, golden):
    # fixtures produced by the reference's rotate + quantize_rowwise_int8 (see tests/golden/make_golden.py)
    for case in golden["activation"]:
        q, s = _cabi.convrot_quantize(case["x"].to(cuda_device), True)
        _recipe_bounds(q.cpu(), s.cpu(), case["q_recipe"], case["scale_recipe"])
        assert q.abs().max().item() == 127  # the row maximum maps to +-127
    from tests.golden import make_golden as mg

    for case in golden["activation_reference_shapes"]:
        dtype = torch.bfloat16 if "bfloat16" in case["dtype"] else torch.float16
        x = mg.reference_activation(*case["shape"], dtype)
        assert mg.checksum(x) == case["x_checksum"], "the seeded activation is not the one the fixture was made from"
        q, s = _cabi.convrot_quantize(x.to(cuda_device), True)
        _recipe_bounds(q.cpu(), s.cpu(), case["q_recipe"], case["scale_recipe"])
    _cabi.check_guards()


def _recipe(x, rotate, col_scale=None):
    """The matmul rotation + row-wise quantize recipe of the reference's tests (tests/test_int8_convrot.py:256-266)."""
    if col_scale is not None:
        x = (x.float() * col_scale.float()).to(x.dtype)
    y = o8.rotate(x, o8.build_hadamard(256)) if rotate else x
    return o8.quantize_rowwise_int8(y)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("rotate", [True, False])
@pytest.mark.parametrize("shape", [(1, 256), (4, 512), (512, 1024), (1024, 2048), (300, 4096), (16, 8192), (8, 16384)])
def test_quantizer_matches_the_reference_recipe_on_the_reference_shapes(cuda_device, shape, rotate, dtype):
    # the reference's seven shapes at full size and its distribution, recipe computed on the host cores
    m, k = shape
    torch.manual_seed(0)
    x = (torch.randn(m, k, dtype=torch.float32) * 2.0).to(dtype)
    q, s = _cabi.convrot_quantize(x.to(cuda_device), rotate)
    _cabi.check_guards()
    q_ref, s_ref = _recipe(x, rotate)
    _recipe_bounds(q.cpu(), s.cpu(), q_ref, s_ref)
    q_exact, s_exact = o8.convrot_quantize(x, rotate)
    assert torch.equal(q.cpu(), q_exact) and torch.equal(s.cpu(), s_exact)


# every group-256 activation width of the reference's model plan (tests/test_int8_convrot.py:293-315 there)
PLAN_PRODUCER_WIDTHS = [1024, 2048, 3072, 3840, 4096, 5120, 5376, 6144, 7168, 8192, 10240, 11520, 12288, 14336, 16384, 21504, 24576, 25600, 28672,
                        36864, 248320]


@pytest.mark.parametrize("rotate", [True, False])
@pytest.mark.parametrize("k", PLAN_PRODUCER_WIDTHS)
def test_quantizer_every_plan_width(cuda_device, k, rotate):
    torch.manual_seed(k)
    x = (torch.randn(3, k, dtype=torch.float32) * 2.0).to(torch.bfloat16)
    q, s = _cabi.convrot_quantize(x.to(cuda_device), rotate)
    _cabi.check_guards()
    q_exact, s_exact = o8.convrot_quantize(x, rotate)
    assert torch.equal(q.cpu(), q_exact) and torch.equal(s.cpu(), s_exact)
    _recipe_bounds(q.cpu(), s.cpu(), *_recipe(x, rotate))


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("k", [16384, 16640, 32768, 248320])
def test_quantizer_wide_rows_fold_the_column_scale(cuda_device, k, dtype):
    # the input gradient's producer (no rotation, weight scale folded in) on wide rows (tests/test_int8_convrot.py:334-346)
    torch.manual_seed(k)
    x = (torch.randn(5, k, dtype=torch.float32) * 2.0).to(dtype)
    col = torch.rand(k, dtype=torch.float32) * 0.5 + 0.5
    q, s = _cabi.convrot_quantize(x.to(cuda_device), False, col.to(cuda_device))
    _cabi.check_guards()
    q_exact, s_exact = o8.convrot_quantize(x, False, col)
    assert torch.equal(q.cpu(), q_exact) and torch.equal(s.cpu(), s_exact)
    q_ref, s_ref = _recipe(x, False, col)
    assert (q.cpu() != q_ref).float().mean().item() < 1e-3


def test_quantizer_edge_cases(cuda_device):
    import feather_ops_b200 as fo

    zeros = torch.zeros((3, 512), device=cuda_device, dtype=torch.bfloat16)
    q, s = fo.quantize_convrot_activation(zeros)
    assert q.abs().max().item() == 0 and torch.equal(s.cpu(), torch.full((3,), 1e-30 * 0.0625))
    with pytest.raises(RuntimeError, match="multiple of the ConvRot group size"):
        fo.quantize_convrot_activation(torch.zeros((2, 300), device=cuda_device, dtype=torch.bfloat16))
    with pytest.raises(RuntimeError, match="x must be float16 or bfloat16"):
        fo.quantize_convrot_activation(torch.zeros((2, 256), device=cuda_device, dtype=torch.float32))
    q, s = fo.quantize_convrot_activation(torch.zeros((0, 256), device=cuda_device, dtype=torch.float16))
    assert q.shape == (0, 256) and s.shape == (0,)
    # full-size benchmark activation: 4096 x 3072 with outlier channels
    x = o8.make_activation(4096, 3072, torch.bfloat16)
    q_ref, s_ref = o8.convrot_quantize(x, True)
    q, s = fo.quantize_convrot_activation(x.to(cuda_device))
    assert torch.equal(q.cpu(), q_ref) and torch.equal(s.cpu(), s_ref)


SHAPES = [(1, 64, 128), (17, 96, 64), (128, 128, 128), (67, 272, 304), (300, 516, 1040), (512, 1024, 2048), (4112, 1152, 1152)]


def _gemm_case(m, n, k, transposed, out_dtype, seed):
    gen = torch.Generator().manual_seed(seed)
    w = torch.randint(-127, 128, (n, k), generator=gen, dtype=torch.int8)
    kc, n_out = (n, k) if transposed else (k, n)
    a = torch.randint(-127, 128, (m, kc), generator=gen, dtype=torch.int8)
    a_scale = torch.rand(m, generator=gen) * 0.01 + 0.001
    w_scale = None if transposed else torch.rand(n, generator=gen) * 0.01 + 0.001
    bias = None if transposed else torch.randn(n, generator=gen).to(out_dtype)
    return w, a, a_scale, w_scale, bias, n_out


@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("transposed", [False, True])
@pytest.mark.parametrize("shape", SHAPES)
def test_gemm_against_the_fp64_oracle(cuda_device, shape, transposed, out_dtype):
    m, n, k = shape
    if (n if transposed else k) % 16:
        pytest.skip("the contraction axis must be a multiple of 16")
    w, a, a_scale, w_scale, bias, n_out = _gemm_case(m, n, k, transposed, out_dtype, seed=m + n)
    ref = o8.int8_scaled_mm(a, w, a_scale, w_scale, bias, out_dtype, transposed)
    dev = lambda t: None if t is None else t.to(cuda_device)  # noqa: E731
    out = _cabi.int8_scaled_mm(dev(a), dev(o8.prepack_int8_weight(w)), dev(a_scale), dev(w_scale), dev(bias), out_dtype, transposed, n_out)
    _cabi.assert_clean(STATUS)
    assert _max_rel(out, ref) < 0.02


PLAIN_SHAPES = SHAPES + [(1, 256, 256), (130, 132, 144), (257, 2064, 1040), (700, 640, 4112),
                         # forward with at most 64 rows: the warp-MMA kernel reading the rows of the weight (ragged column blocks, half k blocks)
                         (5, 3072, 3072), (16, 1040, 528), (9, 260, 16), (33, 260, 16), (47, 3072, 1040), (64, 3072, 3072), (16, 12288, 1024)]


@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("transposed", [False, True])
@pytest.mark.parametrize("shape", PLAIN_SHAPES)
def test_gemm_over_the_plain_weight(cuda_device, shape, transposed, out_dtype):
    # the row-major [N, K] weight through the copy engine, no prepack: fp64 oracle, and the same bits as the prepacked kernel
    m, n, k = shape
    w, a, a_scale, w_scale, bias, n_out = _gemm_case(m, n, k, transposed, out_dtype, seed=m + n + 1)
    dev = lambda t: None if t is None else t.to(cuda_device)  # noqa: E731
    out = _cabi.int8_scaled_mm_plain(dev(a), dev(w), dev(a_scale), dev(w_scale), dev(bias), out_dtype, transposed)
    if k % 16 or n % (16 if transposed else 4):
        assert out is None   # refused: the rows of the weight (and of the activation) must be multiples of 16 bytes
        return
    _cabi.assert_clean(STATUS)
    ref = o8.int8_scaled_mm(a, w, a_scale, w_scale, bias, out_dtype, transposed)
    assert _max_rel(out, ref) < 0.02
    packed = _cabi.int8_scaled_mm(dev(a), dev(o8.prepack_int8_weight(w)), dev(a_scale), dev(w_scale), dev(bias), out_dtype, transposed, n_out)
    _cabi.assert_clean(STATUS)
    assert torch.equal(out, packed)


@pytest.mark.parametrize("transposed", [False, True])
def test_plain_weight_int32_accumulators_are_exact(cuda_device, transposed):
    gen = torch.Generator().manual_seed(3)
    n, k, m = (512, 384, 300) if transposed else (384, 512, 300)
    w = torch.randint(-2, 3, (n, k), generator=gen, dtype=torch.int8)
    a = torch.randint(-2, 3, (m, n if transposed else k), generator=gen, dtype=torch.int8)
    ones = torch.ones(max(m, n, k), device=cuda_device)
    out = _cabi.int8_scaled_mm_plain(a.to(cuda_device), w.to(cuda_device), ones[:m].contiguous(), None if transposed else ones[:n].contiguous(), None,
                                     torch.float16, transposed)
    acc = o8.int8_accumulators(a, w, transposed)
    assert acc.abs().max().item() < 2048
    assert torch.equal(out.cpu().float().long(), acc)


def test_plain_weight_operator_and_dispatch(cuda_device, monkeypatch):
    import feather_ops_b200 as fo
    from feather_ops_b200 import int8_convrot as ic

    op = torch.ops.feather_ops.int8_scaled_mm_plain.default
    a = torch.zeros((8, 64), device=cuda_device, dtype=torch.int8)
    w = torch.zeros((32, 64), device=cuda_device, dtype=torch.int8)
    s = torch.ones(8, device=cuda_device)
    c = torch.zeros((8, 32), device=cuda_device, dtype=torch.bfloat16)
    op(a, w, s, None, None, c, False)
    with pytest.raises(RuntimeError, match="a and weight must be int8"):
        op(a, w.to(torch.uint8), s, None, None, c, False)
    with pytest.raises(RuntimeError, match="row length must equal"):
        op(a, w, s, None, None, c, True)
    with pytest.raises(RuntimeError, match="c has the wrong shape"):
        op(a, w, s, None, None, torch.zeros((8, 64), device=cuda_device, dtype=torch.bfloat16), False)
    with pytest.raises(RuntimeError, match="takes neither b_scale nor bias"):
        op(torch.zeros((8, 32), device=cuda_device, dtype=torch.int8), w, s, torch.ones(32, device=cuda_device), None,
           torch.zeros((8, 64), device=cuda_device, dtype=torch.bfloat16), True)
    with pytest.raises(RuntimeError, match="multiples of 16"):
        op(a[:, :40].contiguous(), w[:, :40].contiguous(), s, None, None, c, False)
    with pytest.raises(ValueError, match="weight_scale must be None"):
        fo.int8_scaled_mm_plain(a, w, s, torch.ones(32, device=cuda_device), None, torch.bfloat16, True)
    # which calls take the plain weight: unpacked weights whose rows the copy engine can address
    assert ic.plain_weight_eligible(w, False) and ic.plain_weight_eligible(w, True)
    assert not ic.plain_weight_eligible(w[:, :40].contiguous(), False)
    assert not ic.plain_weight_eligible(w.t(), False)
    assert ic.plain_weight_eligible(torch.zeros((36, 64), device=cuda_device, dtype=torch.int8), False)
    assert not ic.plain_weight_eligible(torch.zeros((36, 64), device=cuda_device, dtype=torch.int8), True)
    calls = []
    real = ic.int8_scaled_mm_plain
    monkeypatch.setattr(ic, "int8_scaled_mm_plain", lambda *args: calls.append(args[6]) or real(*args))
    gen = torch.Generator().manual_seed(8)
    x = torch.randn((96, 512), generator=gen).to(torch.bfloat16).to(cuda_device)
    wq, ws = fo.quantize_convrot_weight((torch.randn((768, 512), generator=gen) * 0.02).to(torch.bfloat16).to(cuda_device))
    y = ic.convrot_int8_linear(x, wq, ws)
    dx = ic.convrot_int8_dgrad(torch.randn((96, 768), generator=gen).to(torch.bfloat16).to(cuda_device), wq, ws)
    assert calls == [False, True] and y.shape == (96, 768) and dx.shape == (96, 512)
    ic.convrot_int8_linear(x[:3], wq, ws)                                           # a few rows too: a permute per call costs more
    ic.convrot_int8_linear(x, fo.prepack_int8_weight(wq), ws, weight_packed=True)   # a prepacked weight stays on the kernels that read it
    assert calls == [False, True, False]
    # opt-in: a row-major copy of a prepacked weight, made once per weight version, then the plain-weight kernel (same bits)
    packed = fo.prepack_int8_weight(wq)
    y_packed = ic.convrot_int8_linear(x, packed, ws, weight_packed=True)
    ic.cache_unpacked_weights(True)
    try:
        assert torch.equal(ic.convrot_int8_linear(x, packed, ws, weight_packed=True), y_packed)
        assert torch.equal(ic.convrot_int8_linear(x, packed.reshape(-1), ws, weight_packed=True), y_packed)   # a flattened view: the same entry
        ic.convrot_int8_linear(x, packed, ws, weight_packed=True)
        ic.convrot_int8_dgrad(torch.zeros((4, 768), device=cuda_device, dtype=torch.bfloat16), packed, ws, weight_packed=True)
        ic.convrot_int8_linear(x[:8], packed, ws, weight_packed=True)   # few rows: the warp-MMA kernel on the prepack
        assert calls == [False, True, False, False, False, False, True]
        assert len(ic._UNPACKED_CACHE._entries) == 1
        packed.add_(1)                                                   # a new version of the weight: a new copy replaces the old one
        assert torch.equal(ic.convrot_int8_linear(x, packed, ws, weight_packed=True),
                           ic.convrot_int8_linear(x, fo.unpack_int8_weight(packed).contiguous(), ws))
        assert len(ic._UNPACKED_CACHE._entries) == 1
        del packed
        gc.collect()
        assert len(ic._UNPACKED_CACHE._entries) == 0                     # the copy goes with the weight
    finally:
        ic.cache_unpacked_weights(False)
    _cabi.assert_clean(STATUS)


@pytest.mark.parametrize("transposed", [False, True])
def test_every_tile_in_both_directions(cuda_device, transposed):
    from feather_ops_b200.tiles import INT8_TILES

    m, n, k = (67, 272, 304)
    w, a, a_scale, w_scale, bias, n_out = _gemm_case(m, n, k, transposed, torch.bfloat16, seed=7)
    ref = o8.int8_scaled_mm(a, w, a_scale, w_scale, bias, torch.bfloat16, transposed)
    dev = lambda t: None if t is None else t.to(cuda_device)  # noqa: E731
    args = (dev(a), dev(o8.prepack_int8_weight(w)), dev(a_scale), dev(w_scale), dev(bias))
    for tile in INT8_TILES:
        out = _cabi.int8_scaled_mm(*args, torch.bfloat16, transposed, n_out, tile)
        _cabi.assert_clean(STATUS)
        assert _max_rel(out, ref) < 0.02


@pytest.mark.parametrize("transposed", [False, True])
def test_int32_accumulators_are_exact(cuda_device, transposed):
    # unit scales and codes small enough that every accumulator is an integer below 2048: exact in fp16
    gen = torch.Generator().manual_seed(2)
    n, k, m = (256, 128, 130) if transposed else (128, 256, 130)
    w = torch.randint(-3, 4, (n, k), generator=gen, dtype=torch.int8)
    a = torch.randint(-3, 4, (m, n if transposed else k), generator=gen, dtype=torch.int8)
    n_out = k if transposed else n
    ones = torch.ones(max(m, n_out), device=cuda_device)
    out = _cabi.int8_scaled_mm(a.to(cuda_device), o8.prepack_int8_weight(w).to(cuda_device), ones[:m].contiguous(),
                               None if transposed else ones[:n_out].contiguous(), None, torch.float16, transposed, n_out)
    acc = o8.int8_accumulators(a, w, transposed)
    assert acc.abs().max().item() < 2048
    assert torch.equal(out.cpu().float().long(), acc)


def test_linear_and_dgrad_equal_their_compositions(cuda_device):
    import feather_ops_b200 as fo
    from feather_ops_b200 import int8_convrot as ic

    gen = torch.Generator().manual_seed(4)
    m, n, k = 200, 768, 512
    x = torch.randn((2, m // 2, k), generator=gen).to(torch.bfloat16).to(cuda_device)
    w = (torch.randn((n, k), generator=gen) * 0.02).to(torch.bfloat16).to(cuda_device)
    bias = torch.randn(n, generator=gen).to(torch.bfloat16).to(cuda_device)
    wq, ws = fo.quantize_convrot_weight(w)
    packed = fo.prepack_int8_weight(wq)
    assert torch.equal(fo.unpack_int8_weight(packed), wq)

    y = fo.convrot_int8_linear(x, wq, ws, bias)
    q, s = fo.quantize_convrot_activation(x.reshape(-1, k))
    assert torch.equal(y, fo.int8_scaled_mm(q, packed, s, ws, bias).reshape(2, m // 2, n))
    assert torch.equal(y, fo.convrot_int8_linear(x, packed, ws, bias, weight_packed=True))
    # end to end against the unquantized product (reference bound: rel < 2e-2)
    ref = x.float().reshape(-1, k) @ w.float().T + bias.float()
    assert ((y.float().reshape(-1, n) - ref).norm() / ref.norm()).item() < 2e-2

    g = torch.randn((m, n), generator=gen).to(torch.bfloat16).to(cuda_device)
    dx = fo.convrot_int8_dgrad(g, wq, ws)
    gq, gs = fo.quantize_convrot_activation(g, False, col_scale=ws)
    composed = ic.rotate(fo.int8_scaled_mm(gq, packed, gs, None, None, torch.bfloat16, True), ic.build_hadamard(256, device=cuda_device, dtype=torch.bfloat16))
    assert torch.equal(dx, composed)
    ref_dx = g.float() @ w.float()
    assert ((dx.float() - ref_dx).norm() / ref_dx.norm()).item() < 3e-2
    _cabi.assert_clean(STATUS)


def test_operator_errors(cuda_device):
    import feather_ops_b200  # noqa: F401

    op = torch.ops.feather_ops.int8_scaled_mm.default
    a = torch.zeros((8, 64), device=cuda_device, dtype=torch.int8)
    w = torch.zeros(64 * 32, device=cuda_device, dtype=torch.int8)
    s = torch.ones(8, device=cuda_device)
    c = torch.zeros((8, 32), device=cuda_device, dtype=torch.bfloat16)
    tile = (4, 4, 2, 4, 4)
    op(a, w, s, None, None, c, False, *tile)
    with pytest.raises(RuntimeError, match="Unsupported config"):
        op(a, w, s, None, None, c, False, 5, 5, 5, 5, 5)
    with pytest.raises(RuntimeError, match="a must be int8"):
        op(a.to(torch.uint8), w, s, None, None, c, False, *tile)
    with pytest.raises(RuntimeError, match="weight_in \\* weight_out bytes"):
        op(a, w[:100], s, None, None, c, False, *tile)
    with pytest.raises(RuntimeError, match="multiple of 16"):
        op(a[:, :40].contiguous(), torch.zeros(40 * 32, device=cuda_device, dtype=torch.int8), s, None, None, c, False, *tile)
    with pytest.raises(RuntimeError, match="a_scale must have M elements"):
        op(a, w, s[:4], None, None, c, False, *tile)


def test_benchmark_shape_whole_output(cuda_device):
    # 4096 x 3072 x 3072: quantize -> GEMM with the offline weight recipe; every element against the fp64 oracle
    import feather_ops_b200 as fo

    x = o8.make_activation(4096, 3072, torch.bfloat16)
    w = o8.make_weight(3072, 3072, torch.bfloat16)
    wq, ws = o8.quantize_convrot_weight(w)
    q_ref, s_ref = o8.convrot_quantize(x, True)
    y = fo.convrot_int8_linear(x.to(cuda_device), wq.to(cuda_device), ws.to(cuda_device))
    _cabi.assert_clean(STATUS)
    ref = o8.int8_scaled_mm(q_ref, wq, s_ref, ws, None, torch.bfloat16)
    assert _max_rel(y, ref) < 0.02
    # the GEMM alone through the C ABI, both directions, every element (guard bands around the outputs)
    packed = o8.prepack_int8_weight(wq).to(cuda_device)
    fwd = _cabi.int8_scaled_mm(q_ref.to(cuda_device), packed, s_ref.to(cuda_device), ws.to(cuda_device), None, torch.bfloat16, False, 3072)
    assert torch.equal(fwd, y)
    bwd = _cabi.int8_scaled_mm(q_ref.to(cuda_device), packed, s_ref.to(cuda_device), None, None, torch.bfloat16, True, 3072)
    _cabi.assert_clean(STATUS)
    assert _max_rel(bwd, o8.int8_scaled_mm(q_ref, wq, s_ref, None, None, torch.bfloat16, True)) < 0.02
    full = x.float() @ w.float().T
    assert ((y.float().cpu() - full).norm() / full.norm()).item() < 2e-2


# the reference's model cells (tests/test_int8_convrot.py:25-39 there): (M, N_w, K_w), the weight's output / input axes
MODEL_CELLS = [(512, 2048, 1024), (4096, 2048, 2048), (4096, 8192, 2048), (4096, 2048, 8192), (4112, 1536, 6144), (4112, 6144, 6144), (4128, 11520, 3840),
               (5376, 21504, 5376), (4112, 3072, 8192), (2048, 4304, 1152), (1024, 3456, 1152), (1, 36864, 6144), (16, 128, 128)]


def _exact_accumulators(a, w_t):
    """`a [m, kc] int8 @ w_t [kc, n] int8` as exact integers held in fp64: fp32 products of 1024-deep slices are exact
    (127 * 127 * 1024 < 2^24), their sum is taken in fp64."""
    acc = torch.zeros((a.shape[0], w_t.shape[1]), dtype=torch.float64)
    for k0 in range(0, a.shape[1], 1024):
        acc += (a[:, k0 : k0 + 1024].float() @ w_t[k0 : k0 + 1024].float()).double()
    return acc


@pytest.mark.parametrize("transposed", [False, True])
@pytest.mark.parametrize("cell", MODEL_CELLS)
def test_model_cells_against_the_oracle(cuda_device, cell, transposed):
    # both directions of every model cell of the reference's test, through the public API with its own tile choice;
    # the oracle is evaluated in bands of 1024 rows on the host cores with exact integer accumulators
    import feather_ops_b200 as fo

    m, n_w, k_w = cell
    contraction, out = (n_w, k_w) if transposed else (k_w, n_w)
    gen = torch.Generator().manual_seed(m + n_w)
    wq = torch.randint(-127, 128, (n_w, k_w), generator=gen, dtype=torch.int8)
    a = torch.randint(-127, 128, (m, contraction), generator=gen, dtype=torch.int8)
    a_scale = torch.rand(m, generator=gen) * 0.02 + 1e-4
    w_scale = None if transposed else torch.rand(out, generator=gen) * 0.02 + 1e-4
    packed = fo.prepack_int8_weight(wq.to(cuda_device))
    got = fo.int8_scaled_mm(a.to(cuda_device), packed, a_scale.to(cuda_device), None if transposed else w_scale.to(cuda_device), None, torch.bfloat16, transposed)
    _cabi.assert_clean(STATUS)
    assert got.shape == (m, out)
    got = got.cpu()
    w_t = wq if transposed else wq.T.contiguous()
    for r0 in range(0, m, 1024):
        acc = _exact_accumulators(a[r0 : r0 + 1024], w_t) * a_scale[r0 : r0 + 1024].double()[:, None]
        if not transposed:
            acc = acc * w_scale.double()[None, :]
        assert _max_rel(got[r0 : r0 + 1024], acc.to(torch.bfloat16)) < 0.02, (cell, transposed, r0)


def test_compiled_caller_matches_eager(cuda_device):
    # tests/test_int8_convrot.py:387-401 of the reference: dynamic shapes, default backend, one opaque node
    import feather_ops_b200 as fo

    gen = torch.Generator().manual_seed(0)
    m, n_w, k_w = 4112, 1152, 1152
    packed = fo.prepack_int8_weight(torch.randint(-127, 128, (n_w, k_w), generator=gen, dtype=torch.int8).to(cuda_device))
    a = torch.randint(-127, 128, (m, k_w), generator=gen, dtype=torch.int8).to(cuda_device)
    a_scale = (torch.rand(m, generator=gen) * 0.02).to(cuda_device)
    w_scale = (torch.rand(n_w, generator=gen) * 0.02).to(cuda_device)

    def run(a, a_scale):
        return fo.int8_scaled_mm(a, packed, a_scale, w_scale, None, torch.bfloat16, False)

    eager = run(a, a_scale)
    torch._dynamo.reset()
    compiled = torch.compile(run, fullgraph=True, dynamic=True)(a, a_scale)
    assert torch.equal(compiled, eager)
    _cabi.assert_clean(STATUS)

    # the same through the unpacked weight's operator
    plain = fo.unpack_int8_weight(packed).contiguous()

    def run_plain(a, a_scale):
        return fo.int8_scaled_mm_plain(a, plain, a_scale, w_scale, None, torch.bfloat16, False)

    torch._dynamo.reset()
    compiled = torch.compile(run_plain, fullgraph=True, dynamic=True)(a, a_scale)
    assert torch.equal(compiled, eager)
    _cabi.assert_clean(STATUS)


@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("shape", [(1, 256, 64), (5, 3072, 3072), (16, 1040, 528), (9, 260, 16), (16, 12288, 1024), (17, 3072, 3072), (32, 1040, 528),
                                   (33, 260, 16), (47, 3072, 1040), (64, 3072, 3072)])
def test_few_rows_take_the_warp_mma_kernel(cuda_device, shape, out_dtype):
    # forward direction with at most 16 rows (64 for narrow outputs; two 16-row tiles per warp, one grid row per 32 rows) runs on mma.sync with a permuted contraction index: exact int32 sums, the
    # same oracle and tolerance, ragged last column block (260, 1040), a contraction with a half block (528 = 16.5 x 32)
    m, n, k = shape
    w, a, a_scale, w_scale, bias, n_out = _gemm_case(m, n, k, False, out_dtype, seed=m + n + k)
    ref = o8.int8_scaled_mm(a, w, a_scale, w_scale, bias, out_dtype, False)
    dev = lambda t: None if t is None else t.to(cuda_device)  # noqa: E731
    packed = dev(o8.prepack_int8_weight(w))
    out = _cabi.int8_scaled_mm(dev(a), packed, dev(a_scale), dev(w_scale), dev(bias), out_dtype, False, n_out)
    _cabi.assert_clean(STATUS)
    assert _max_rel(out, ref) < 0.02
    plain = _cabi.int8_scaled_mm(dev(a), packed, dev(a_scale), None, None, out_dtype, False, n_out)
    assert _max_rel(plain, o8.int8_scaled_mm(a, w, a_scale, None, None, out_dtype, False)) < 0.02
    # unit scales: the result is the exact integer product wherever it is representable in the output dtype
    ones = torch.ones(m, device=cuda_device)
    exact = _cabi.int8_scaled_mm(dev(a), packed, ones, None, None, torch.float16, False, n_out).double().cpu()
    want = a.double() @ w.double().T
    small = want.abs() <= 2048
    assert torch.equal(exact[small], want[small])
