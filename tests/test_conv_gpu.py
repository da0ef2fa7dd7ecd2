"""conv2d 3x3 on the GPU against fp64 `F.conv2d`, with the reference's shapes and tolerances
(tests/test_conv3x3.py there: rel < 4e-3 for bf16, < 6e-4 for fp16)."""

import pytest
import torch
import torch.nn.functional as F

from oracle import conv2d as oc
from tests import _cabi

pytestmark = pytest.mark.gpu
STATUS = "feather_conv3x3_status"
TOL = {torch.bfloat16: 4e-3, torch.float16: 6e-4}

# (B, C_in, C_out, H, W): channel counts that are not multiples of 16 / 128, odd heights, widths with tails,
# widths below one segment, odd widths (pixel-by-pixel gather), batch > 1
SHAPES = [
    (1, 16, 16, 8, 32), (1, 8, 32, 9, 40), (2, 24, 48, 13, 50), (1, 64, 128, 32, 128), (1, 32, 64, 17, 33), (2, 128, 256, 16, 256),
    (1, 40, 144, 7, 300), (1, 8, 8, 1, 1), (1, 16, 320, 5, 64), (3, 48, 96, 31, 96), (1, 128, 128, 64, 64), (1, 256, 128, 3, 513),
    (1, 72, 200, 11, 130), (1, 512, 512, 8, 128),
    # widths that are multiples of 8 take their halo tiles through the copy engine: a tile narrower than the box, channels that end
    # inside a 16-channel group, a ragged second segment, a ragged channel tile on the CTA-pair kernel, batch > 1, one row
    (2, 24, 40, 5, 8), (1, 8, 136, 3, 16), (2, 40, 272, 9, 136), (1, 24, 130, 2, 264), (1, 136, 264, 1, 392),
    # more tiles than SMs, so that a CTA walks a range of tiles and consecutive tiles share their weight slots: ranges of two and
    # three tiles over two images; a range that straddles two output-channel tiles on the one-CTA kernel (3 x 75 tiles of one row)
    # and on the CTA-pair kernel (3 x 40 tiles of two rows), where the tile before the boundary must run alone
    (2, 24, 96, 90, 136), (1, 16, 272, 75, 128), (1, 16, 520, 80, 128),
]
TILES = [(4, 4, 2, 4, 1), (4, 4, 2, 2, 1), (2, 2, 2, 2, 1), (4, 4, 2, 2, 2)]


def _rel(y, ref):
    return ((y.double().cpu() - ref).norm() / ref.norm().clamp(min=1e-12)).item()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("with_bias", [True, False])
@pytest.mark.parametrize("shape", SHAPES)
def test_shapes_through_the_c_abi(cuda_device, shape, with_bias, dtype):
    b, c_in, c_out, h, w = shape
    x, weight, bias = oc.make_inputs(b, c_in, c_out, h, w, dtype, seed=c_in + w, with_bias=with_bias)
    ref = oc.conv3x3_fp64(x, weight, bias)
    packed = oc.prepack_conv2d_weight_3x3(weight).to(cuda_device)
    for tile in TILES:
        if tile[4] == 2 and w % 2:
            continue
        y = _cabi.conv3x3(x.to(cuda_device), packed, None if bias is None else bias.to(cuda_device), tile)
        _cabi.assert_clean(STATUS)
        assert _rel(y, ref) < TOL[dtype], tile


def test_every_tile_and_row_variants_agree_bit_for_bit(cuda_device):
    # all tiles accumulate in the same k order (groups ascending, taps 0..8), so every tile gives the same bits
    from feather_ops_b200.tiles import CONV_TILES

    x, weight, bias = oc.make_inputs(2, 40, 136, 10, 144, torch.bfloat16, seed=3)
    packed = oc.prepack_conv2d_weight_3x3(weight).to(cuda_device)
    ref = oc.conv3x3_fp64(x, weight, bias)
    first = None
    for tile in CONV_TILES:
        y = _cabi.conv3x3(x.to(cuda_device), packed, bias.to(cuda_device), tile)
        _cabi.assert_clean(STATUS)
        assert _rel(y, ref) < TOL[torch.bfloat16]
        first = y if first is None else first
        assert torch.equal(y, first), tile


def test_python_api_drop_in_and_module(cuda_device):
    import feather_ops_b200 as fo
    from feather_ops_b200 import conv2d as fc

    x, weight, bias = oc.make_inputs(2, 64, 96, 20, 72, torch.bfloat16, seed=8)
    x, weight, bias = x.to(cuda_device), weight.to(cuda_device), bias.to(cuda_device)
    ref = oc.conv3x3_fp64(x.cpu(), weight.cpu(), bias.cpu())
    with torch.no_grad():
        assert fc.conv3x3_eligibility(x, weight, bias) is None
        y = fc.conv2d(x, weight, bias, 1, 1)
        assert _rel(y, ref) < TOL[torch.bfloat16]
        assert torch.equal(y, fo.conv3x3_prepacked(x, fo.prepack_conv2d_weight_3x3(weight), bias))
        # not covered by the kernel: goes to torch and still matches
        y_stride = fc.conv2d(x, weight, bias, 2, 1)
        assert torch.equal(y_stride, F.conv2d(x, weight, bias, 2, 1))
        assert fc.conv3x3_eligibility(x, weight, bias, stride=2) == "stride (2, 2), dilation (1, 1)"
        assert fc.conv3x3_eligibility(x, weight, bias, padding=0) == "padding (0, 0)"
        assert fc.conv3x3_eligibility(x.permute(0, 1, 3, 2), weight, bias) == "input or weight is not contiguous"
        assert fc.conv3x3_eligibility(x, weight, bias.float()).startswith("bias torch.float32")

        module = fo.Conv2d(64, 96, 3, padding=1, device=cuda_device, dtype=torch.bfloat16)
        module.weight.copy_(weight)
        module.bias.copy_(bias)
        assert torch.equal(module(x), y)
        module.weight.mul_(2)  # a new weight version must invalidate the prepack
        assert _rel(module(x), oc.conv3x3_fp64(x.cpu(), (weight * 2).cpu(), bias.cpu())) < TOL[torch.bfloat16]
    x.requires_grad_(True)
    assert fc.conv3x3_eligibility(x, weight, bias) == "autograd is enabled"
    _cabi.assert_clean(STATUS)


def test_operator_errors(cuda_device):
    import feather_ops_b200  # noqa: F401

    op = torch.ops.feather_ops.conv2d_3x3.default
    x = torch.zeros((1, 16, 8, 32), device=cuda_device, dtype=torch.bfloat16)
    w = torch.zeros((18, 24, 8), device=cuda_device, dtype=torch.bfloat16)
    out = torch.zeros((1, 24, 8, 32), device=cuda_device, dtype=torch.bfloat16)
    op(x, w, None, out, 4, 4, 2, 4, 1, False)
    with pytest.raises(RuntimeError, match="unsupported tile"):
        op(x, w, None, out, 7, 7, 7, 7, 1, False)
    with pytest.raises(RuntimeError, match="w_prepacked must have x's dtype"):
        op(x, w.to(torch.float16), None, out, 4, 4, 2, 4, 1, False)
    with pytest.raises(RuntimeError, match="ceil\\(C_in/16\\)\\*18"):
        op(x, w[:9].contiguous(), None, out, 4, 4, 2, 4, 1, False)
    with pytest.raises(RuntimeError, match="multiple of 8 input channels"):
        op(torch.zeros((1, 12, 8, 32), device=cuda_device, dtype=torch.bfloat16), w, None, out, 4, 4, 2, 4, 1, False)
    with pytest.raises(RuntimeError, match="x must be contiguous NCHW"):
        op(x.permute(0, 1, 3, 2), w, None, torch.zeros((1, 24, 32, 8), device=cuda_device, dtype=torch.bfloat16), 4, 4, 2, 4, 1, False)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("channels,size", [(512, 128), (256, 256), (128, 512)])
def test_benchmark_shapes_whole_output(cuda_device, channels, size, dtype):
    # VAE-decoder shapes: every output element against the fp64 oracle (under a second on the host cores), per output
    # channel as well as over the whole tensor; then a sub-image computed alone equals the same pixels of the whole
    # image away from its border rows, and a zero input gives exactly the bias.
    import feather_ops_b200 as fo

    x, weight, bias = oc.make_inputs(1, channels, channels, size, size, dtype)
    xg, bg = x.to(cuda_device), bias.to(cuda_device)
    packed = fo.prepack_conv2d_weight_3x3(weight.to(cuda_device))
    y = _cabi.conv3x3(xg, packed, bg, fo.conv2d.select_conv3x3_config(channels, size))
    _cabi.assert_clean(STATUS)
    assert torch.equal(y, fo.conv3x3_prepacked(xg, packed, bg))
    ref = oc.conv3x3_fp64(x, weight, bias)
    assert _rel(y, ref) < TOL[dtype]
    per_channel = (y.double().cpu() - ref).flatten(2).norm(dim=2) / ref.flatten(2).norm(dim=2)
    assert per_channel.max().item() < 2 * TOL[dtype]
    band = fo.conv3x3_prepacked(xg[:, :, 16:48].contiguous(), packed, bg)
    assert torch.equal(band[:, :, 1:-1], y[:, :, 17:47])
    zero = fo.conv3x3_prepacked(torch.zeros_like(xg[:, :, :4]), packed, bg)
    assert torch.equal(zero, bg.reshape(1, -1, 1, 1).expand_as(zero))


@pytest.mark.parametrize("channels,size", [(128, 512), (256, 256), (64, 264)])
def test_back_to_back_launches_repeat_the_same_bits(cuda_device, channels, size):
    # The copy engine fills the slots of the halo ring in any order; a gather that mistook an older phase of a slot's
    # barrier for its own would show as a launch that differs from the first one or as a wait that ran out. 300 launches
    # in a row over rotating inputs (so that the tiles come from DRAM with scattered latencies), every output compared.
    import feather_ops_b200 as fo

    x, weight, bias = oc.make_inputs(1, channels, channels, size, size, torch.bfloat16, seed=channels)
    packed = fo.prepack_conv2d_weight_3x3(weight.to(cuda_device))
    bg = bias.to(cuda_device)
    xs = [x.to(cuda_device).clone() for _ in range(6)]
    ys = [torch.empty_like(xs[0]) for _ in range(6)]
    tile = fo.conv2d.select_conv3x3_config(channels, size)
    first = _cabi.conv3x3(xs[0], packed, bg, tile)
    op = torch.ops.feather_ops.conv2d_3x3.default
    for rounds in range(50):
        for i in range(6):
            op(xs[i], packed, bg, ys[i], *tile, False)
        for i in range(6):
            assert torch.equal(ys[i], first), (rounds, i)
    _cabi.assert_clean(STATUS)


def test_compiled_caller_matches_the_oracle(cuda_device):
    # tests/test_conv3x3.py:276-291 of the reference: the prepacked op under torch.compile with the default backend
    import feather_ops_b200 as fo
    from feather_ops_b200.conv2d import select_conv3x3_config

    x, weight, _ = oc.make_inputs(1, 96, 96, 64, 64, torch.bfloat16, seed=3, with_bias=False)
    packed = fo.prepack_conv2d_weight_3x3(weight.to(cuda_device))
    tile = select_conv3x3_config(96, 64)
    assert tile is not None

    def run(inp, wk):
        return fo.conv3x3_prepacked(inp, wk, None, tile=tile)

    torch._dynamo.reset()
    out = torch.compile(run, fullgraph=True)(x.to(cuda_device), packed)
    assert _rel(out, oc.conv3x3_fp64(x, weight, None)) < 4e-3
    assert torch.equal(out, run(x.to(cuda_device), packed))
    auto = torch.compile(lambda inp, wk: fo.conv3x3_prepacked(inp, wk, None), fullgraph=True, dynamic=True)(x.to(cuda_device), packed)
    assert torch.equal(auto, out)
    _cabi.assert_clean(STATUS)
