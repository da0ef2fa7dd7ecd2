"""Host-side logic that needs no GPU: tile tables, heuristics, prepacks, eligibility, caches, module glue."""

import pytest
import torch
from torch import nn

import feather_ops_b200
from feather_ops_b200 import _build, conv2d, conv2d_module, int8_convrot, modules, scaled_mm, tiles
from oracle import conv2d as oc
from oracle import int8_convrot as o8
from oracle import scaled_mm as osm


def test_tile_vocabulary_is_the_reference_one(golden):
    assert tiles.SCALED_MM_TILES == golden["tiles"]["scaled_mm"]
    assert tiles.INT8_TILES == golden["tiles"]["int8"]
    assert tiles.CONV_TILES == golden["tiles"]["conv"]
    assert len(tiles.CONV_TILES) == 38
    for table in (tiles.SCALED_MM_TILES, tiles.INT8_TILES, tiles.CONV_TILES):
        assert len(set(table)) == len(table)
    boxes = [tiles.conv_block_sizes(tile) for tile in tiles.CONV_TILES]
    assert len(set(boxes)) == len(boxes)


def test_generated_header_is_current():
    assert _build.TILE_HEADER.read_text() == tiles.render_header()


def test_every_tuple_maps_to_a_umma_tile():
    for table, mapping in ((tiles.SCALED_MM_TILES, tiles.SCALED_MM_UMMA), (tiles.INT8_TILES, tiles.INT8_UMMA), (tiles.CONV_TILES, tiles.CONV_UMMA)):
        for tile in table:
            umma = mapping[tile]
            assert umma.block_m in (64, 128) and umma.block_n % 16 == 0 and 16 <= umma.block_n <= 512
    assert scaled_mm.tile_shape((1, 8, 4, 8, 2, 0)) == (128, 256, 64)
    assert scaled_mm.umma_tile((1, 2, 4, 1, 2, 1)).block_n == 64


def test_heuristics_return_table_rows():
    for module, table in ((scaled_mm, tiles.SCALED_MM_TILES), (int8_convrot, tiles.INT8_TILES), (conv2d, tiles.CONV_TILES)):
        for name in dir(module):
            if name.startswith("_TILE_") and isinstance(getattr(module, name), tuple):
                assert getattr(module, name) in table, name
    for m in (1, 16, 128, 1024, 4096, 8192, 65536):
        for n, k in ((12288, 3072), (3072, 12288), (9216, 3072), (128, 128), (1152, 1152)):
            assert scaled_mm.select_scaled_mm_config(m, n, k) in tiles.SCALED_MM_TILES
            for transposed in (False, True):
                assert int8_convrot.select_int8_config(m, n, k, transposed) in tiles.INT8_TILES
    assert scaled_mm.select_scaled_mm_config(4096, 12288, 3072) == (1, 8, 4, 8, 2, 0)
    for c_out in (3, 64, 128, 512):
        for width in (1, 33, 64, 128, 129, 256, 512):
            assert conv2d.select_conv3x3_config(c_out, width) in tiles.CONV_TILES
    assert conv2d.select_conv3x3_config(128, 0) is None
    assert conv2d.select_conv3x3_config(512, 128)[4] == 2
    assert conv2d.select_conv3x3_config(512, 129)[4] == 1  # two-row tiles need an even width
    assert conv2d.select_conv3x3_config(128, 512) == (4, 4, 2, 4, 1) and conv2d.select_conv3x3_config(128, 264)[4] == 2  # one row of 256 pixels only without much padding
    assert conv2d.select_conv3x3_config(256, 512)[4] == 2  # more than 128 output channels: the CTA-pair kernel's tile


def test_prepacks_equal_the_oracle(golden):
    gen = torch.Generator().manual_seed(1)
    for k in (144, 256, 300):
        b = torch.randn((k, 48), generator=gen).to(torch.float8_e5m2)
        assert torch.equal(scaled_mm.prepack_b_for_scaled_mm(b).view(torch.uint8), osm.prepack_b(b).view(torch.uint8))
    case = golden["scaled_mm"][0]
    assert torch.equal(scaled_mm.prepack_b_for_scaled_mm(case["b"].view(torch.float8_e5m2)).view(torch.uint8), case["b_prepacked"])
    w = golden["weight"]
    assert torch.equal(int8_convrot.prepack_int8_weight(w["q"]), w["prepacked"])
    assert torch.equal(int8_convrot.unpack_int8_weight(w["prepacked"]), w["q"])
    with pytest.raises(ValueError, match=r"must end in \(4, 4\)"):
        int8_convrot.unpack_int8_weight(torch.zeros(2, 2, 4, 2, dtype=torch.int8))
    cw = golden["conv_prepack"]
    assert torch.equal(conv2d.prepack_conv2d_weight_3x3(cw["w"]), cw["packed"])
    with pytest.raises(ValueError, match="expected a"):
        conv2d.prepack_conv2d_weight_3x3(torch.zeros(4, 4, 5, 5))


def test_offline_weight_recipe_equals_the_reference(golden):
    w = golden["weight"]
    q, scale = int8_convrot.quantize_convrot_weight(w["w"])
    assert torch.equal(q, w["q"]) and torch.equal(scale, w["scale"])
    assert torch.equal(int8_convrot.build_hadamard(256), o8.build_hadamard(256))
    r = golden["rowwise_stored_scale"]
    q, scale = int8_convrot.quantize_rowwise_int8(r["x"], scale=1.0)
    assert torch.equal(q, r["q"]) and torch.equal(scale, r["scale"])
    deq = int8_convrot.dequantize_convrot_weight(w["q"], w["scale"])
    assert ((deq - w["w"].float()).norm() / w["w"].float().norm()).item() < 0.02
    for shape, expected in golden["int8_supported"].items():
        assert int8_convrot.convrot_int8_supported(shape) == expected
    with pytest.raises(ValueError):
        int8_convrot.build_hadamard(128)
    with pytest.raises(ValueError, match="not divisible by the group size"):
        int8_convrot.rotate(torch.zeros(2, 300), int8_convrot.build_hadamard(256))


def test_int8_argument_errors_are_raised_before_any_launch():
    a = torch.zeros((4, 0), dtype=torch.int8)
    with pytest.raises(ValueError, match="nonzero contraction axis"):
        int8_convrot.int8_scaled_mm(a, torch.zeros(16, dtype=torch.int8), torch.ones(4))
    a = torch.zeros((4, 16), dtype=torch.int8)
    with pytest.raises(ValueError, match="weight_scale must be None"):
        int8_convrot.int8_scaled_mm(a, torch.zeros(256, dtype=torch.int8), torch.ones(4), torch.ones(16), transposed_b=True)
    with pytest.raises(ValueError, match="does not divide"):
        int8_convrot.convrot_int8_linear(torch.zeros(2, 256), torch.zeros(1000, dtype=torch.int8), torch.ones(3))
    with pytest.raises(ValueError, match="features"):
        int8_convrot.convrot_int8_linear(torch.zeros(2, 512), torch.zeros(4 * 256, dtype=torch.int8), torch.ones(4))


def test_conv_eligibility_strings():
    x = torch.zeros(1, 8, 8, 8, dtype=torch.bfloat16)
    w = torch.zeros(8, 8, 3, 3, dtype=torch.bfloat16)
    reason = conv2d.conv3x3_eligibility
    assert reason(x, w, groups=2) == "2 groups"
    assert reason(x[0], w) == "input has 3 dimensions"
    assert reason(x.float(), w.float()).startswith("dtype torch.float32")
    assert reason(x, w) == "input and weight are not on the same CUDA device"  # CPU tensors
    assert conv2d.select_backend(torch.bfloat16, 8, 8, 8, 8) == "kernel"
    assert conv2d.select_backend(torch.float16, 512, 512, 128, 128) == "kernel"
    assert conv2d.select_backend(torch.float16, 3, 8, 8, 8) == "miopen"
    assert conv2d.select_backend(torch.float32, 8, 8, 8, 8) == "torch"
    # the drop-in falls back to torch for a call the kernel does not cover (here: CPU tensors)
    y = conv2d.conv2d(x.float(), w.float(), None, 1, 1)
    assert y.shape == (1, 8, 8, 8)


def test_module_glue_and_caches():
    conv = conv2d_module.Conv2d(8, 16, 3, padding=1, dtype=torch.bfloat16)
    assert conv2d_module.conv3x3_module_reason(conv) is None
    assert conv2d_module.conv3x3_module_reason(nn.Conv2d(8, 8, 1)) == "kernel is (1, 1)"
    assert conv2d_module.conv3x3_module_reason(nn.Conv2d(8, 8, 3, stride=2, padding=1)) == "stride is (2, 2)"
    assert conv2d_module.conv3x3_module_reason(nn.Conv2d(8, 8, 3)) == "padding is (0, 0)"
    assert conv2d_module.conv3x3_module_reason(nn.Conv2d(8, 8, 3, padding=0), padding=(1, 1)) is None
    assert conv2d_module.conv3x3_module_reason(nn.Conv2d(8, 8, 3, padding=1, groups=2)) == "2 groups"
    assert conv2d_module.conv3x3_module_reason(nn.Conv2d(8, 8, 3, padding=1, padding_mode="reflect")) == "'reflect' padding"
    assert conv2d_module.conv3x3_module_reason(nn.Linear(2, 2)) == "not a conv2d"
    keys_before = set(conv.state_dict())
    packed, bias = conv2d_module.prepacked_conv3x3(conv)
    assert packed.shape == (18, 16, 8) and bias.shape == (16,)
    assert conv2d_module.prepacked_conv3x3(conv)[0] is packed  # cached
    assert set(conv.state_dict()) == keys_before  # the prepack is not a buffer
    with torch.no_grad():
        conv.weight.add_(1)  # bumps the version counter
    assert conv2d_module.prepacked_conv3x3(conv)[0] is not packed
    conv.to(torch.float16)
    assert conv2d_module._CACHE.peek(conv) is None  # a dtype move drops the entry
    # CPU forward goes to torch
    assert conv(torch.zeros(1, 8, 4, 4, dtype=torch.float16)).shape == (1, 16, 4, 4)

    class Mixin:
        def forward(self, x):
            return super().forward(x) + 1

    root = nn.Sequential(nn.Conv2d(2, 2, 3, padding=1), nn.ReLU(), nn.Conv2d(2, 2, 1))
    changed = modules.relabel_modules(root, Mixin, lambda m: isinstance(m, nn.Conv2d) and m.kernel_size == (3, 3))
    assert changed == 1 and isinstance(root[0], nn.Conv2d) and isinstance(root[0], Mixin)
    assert modules.relabel_modules(root, Mixin, lambda m: isinstance(m, nn.Conv2d) and m.kernel_size == (3, 3)) == 0
    assert type(root[0]) is modules.relabelled_class(nn.Conv2d, Mixin)

    cache = conv2d._PackedWeightCache(max_entries=2)
    w1 = torch.zeros(8, 8, 3, 3)
    p1 = cache.get(w1)
    assert cache.get(w1) is p1
    w1.add_(1)
    assert cache.get(w1) is not p1


def test_public_api_surface():
    for name in feather_ops_b200.__all__:
        assert hasattr(feather_ops_b200, name)
    for op in ("scaled_mm", "int8_scaled_mm", "convrot_quantize", "conv2d_3x3", "scaled_mm_auto", "int8_scaled_mm_auto", "conv3x3_auto"):
        assert hasattr(torch.ops.feather_ops, op)
    x = torch.zeros(4, 32, dtype=torch.float16)  # CPU tensors: the operators exist for CUDA only
    with pytest.raises((RuntimeError, NotImplementedError)):
        torch.ops.feather_ops.scaled_mm.default(x, torch.zeros(8, 16, 16).to(torch.float8_e5m2), None, None, torch.zeros(4, 16, dtype=torch.float16), 1, 8, 4, 8, 2, False)
    assert oc.prepack_conv2d_weight_3x3(torch.zeros(4, 8, 3, 3)).shape == (18, 4, 8)
